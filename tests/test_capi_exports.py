"""The C-ABI library loads without a GPU and exports every symbol the header
declares; on a box with no CUDA device it reports BackendUnavailable rather
than crashing."""
import ctypes as C
import os
import re

import pytest

from oxmera_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "oxmera_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(oxm_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    assert header_symbols() == sorted(capi.EXPORTS)


def test_rust_binding_declares_exactly_the_header():
    """rust/oxmera-b200/src/ffi.rs cannot be compiled here (no Rust toolchain),
    but its `extern "C"` block must name exactly the functions the header
    declares, and its status and dtype constants must carry the header's values."""
    text = open(os.path.join(ROOT, "rust", "oxmera-b200", "src", "ffi.rs")).read()
    block = text[text.index('extern "C" {'):]
    assert sorted(set(re.findall(r"pub fn (oxm_[a-z0-9_]+)\s*\(", block))) == header_symbols()
    header = open(os.path.join(ROOT, "include", "oxmera_b200.h")).read()
    for name, value in re.findall(r"\b(OXM_[A-Z0-9_]+)\s*=\s*(\d+)", header):
        m = re.search(r"pub const %s: \w+ = (\d+);" % name, text)
        assert m and int(m.group(1)) == int(value), name
    lib_rs = open(os.path.join(ROOT, "rust", "oxmera-b200", "src", "lib.rs")).read()
    for trait in ("UnaryOps", "BinaryOps", "MatmulOps", "ReduceOps", "Backend"):
        assert f"impl {trait} for B200Backend" in lib_rs, trait


def test_library_exports_every_declared_symbol():
    lib = capi.load()
    for name in header_symbols():
        assert hasattr(lib, name), name


def test_identity_and_status_names():
    lib = capi.load()
    assert lib.oxm_backend_name() == b"b200-tcgen05"
    assert lib.oxm_status_name(1) == b"ShapeMismatch"
    assert lib.oxm_status_name(8) == b"BackendUnavailable"


def test_view_struct_matches_the_header_layout():
    # int32 x2, int64 x8, int64 x8, int64, void*, int32 x2
    assert C.sizeof(capi.View) == 8 + 64 + 64 + 8 + 8 + 8


def test_missing_device_is_backend_unavailable():
    lib = capi.load()
    n = C.c_int(-1)
    assert lib.oxm_device_count(C.byref(n)) == 0
    ctx = C.c_void_p()
    st = lib.oxm_ctx_create(n.value + 64, C.byref(ctx))  # an index no box has
    assert st == capi.BACKEND_UNAVAILABLE and not ctx.value
    assert b"no backend available" in lib.oxm_last_error()
