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
