"""Build the CUDA library in-tree: oxmera_b200/liboxmera_b200.so.

`python -m oxmera_b200.build [--force]`.  nvcc cross-compiles for sm_100a
without a GPU.  This is the same command line a Rust build.rs would run.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
SOURCES = ["api.cu"]
HEADERS = ["gemm_tcgen05.cuh", "kernels_simt.cuh", "ptx.cuh", os.path.join("..", "..", "include", "oxmera_b200.h")]
OUT = os.path.join(HERE, "liboxmera_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-shared", "-Xcompiler", "-fPIC",
]


def nvcc_command(extra=()):
    return ["nvcc", *NVCC_FLAGS, *extra, "-o", OUT, *[os.path.join(CSRC, s) for s in SOURCES]]


def is_stale() -> bool:
    if not os.path.exists(OUT):
        return True
    built = os.path.getmtime(OUT)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS]
    return any(os.path.getmtime(d) > built for d in deps)


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compile when the library is missing or older than its sources."""
    if not force and not is_stale():
        return OUT
    cmd = nvcc_command(("-Xptxas", "-v") if verbose else ())
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed ({res.returncode}):\n{' '.join(cmd)}\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stderr.write(res.stderr)
    return OUT


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
