"""Builds and runs the C++ spec tests (tests/cpp/spec_tests.cc): the
reference's exercise specs against the C++ host mirror, on CPU with a
test-only oracle backend and on the GPU through B200Backend."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "tests", "cpp", "spec_tests.bin")


def build():
    from oxmera_b200 import capi
    capi.load()  # the CUDA library must exist: the test links against it
    from tests.oracle_lib import Oracle
    Oracle()     # builds the oracle library on demand
    src = os.path.join(ROOT, "tests", "cpp", "spec_tests.cc")
    deps = [src, os.path.join(ROOT, "oxmera_b200", "host", "oxmera.hpp"), capi.library_path()]
    if os.path.exists(BIN) and all(os.path.getmtime(d) <= os.path.getmtime(BIN) for d in deps):
        return BIN
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-o", BIN, src,
           "-L" + os.path.join(ROOT, "oxmera_b200"), "-loxmera_b200",
           "-L" + os.path.join(ROOT, "oracle"), "-loxm_oracle",
           "-Wl,-rpath," + os.path.join(ROOT, "oxmera_b200"), "-Wl,-rpath," + os.path.join(ROOT, "oracle"), "-lpthread"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    return BIN


def run(mode):
    res = subprocess.run([build(), mode], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "0 failed" in res.stdout, res.stdout
    return res.stdout


def test_cpp_specs_on_cpu():
    out = run("cpu")
    assert "cpu:" in out


@pytest.mark.gpu
def test_cpp_a4_spec_on_b200():
    out = run("gpu")
    assert "gpu:" in out
