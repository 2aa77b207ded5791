"""ctypes binding of include/oxmera_b200.h.

The library is built in-tree (see oxmera_b200/build.py).  Loading fails
loudly when it is missing: there is no fallback implementation.
"""
from __future__ import annotations

import ctypes as C
import os

MAX_DIMS = 8
LIB_NAME = "liboxmera_b200.so"

# every symbol include/oxmera_b200.h declares
EXPORTS = [
    "oxm_device_count", "oxm_ctx_create", "oxm_ctx_destroy", "oxm_ctx_device", "oxm_backend_name",
    "oxm_last_error", "oxm_status_name",
    "oxm_alloc", "oxm_free", "oxm_h2d", "oxm_d2h", "oxm_memset", "oxm_copy_peer", "oxm_sync", "oxm_host_alloc", "oxm_host_free",
    "oxm_matmul", "oxm_batched_matmul", "oxm_batched_matmul_host", "oxm_contiguous",
    "oxm_matmul_f32_noalloc", "oxm_matmul_fused", "oxm_matmul_mx", "oxm_unary", "oxm_binary", "oxm_reduce",
    "oxm_event_create", "oxm_event_destroy", "oxm_event_record", "oxm_event_elapsed_ms", "oxm_stream_handle", "oxm_fill", "oxm_selftest_bounded_wait",
    "oxm_set_option", "oxm_get_option", "oxm_launch_counts", "oxm_last_kernel", "oxm_memory_stats", "oxm_plan_matmul",
]

OK, SHAPE_MISMATCH, BROADCAST_INCOMPATIBLE, DTYPE_MISMATCH, UNSUPPORTED_DTYPE = 0, 1, 2, 3, 4
DEVICE_MISMATCH, INDEX_OUT_OF_BOUNDS, RANK_MISMATCH, BACKEND_UNAVAILABLE, NOT_IMPLEMENTED = 5, 6, 7, 8, 9
CUDA_ERROR, TIMEOUT, INVALID_ARGUMENT, DIVIDE_BY_ZERO = 10, 11, 12, 13


class View(C.Structure):
    """oxm_view"""

    _fields_ = [
        ("dtype", C.c_int32),
        ("ndim", C.c_int32),
        ("shape", C.c_int64 * MAX_DIMS),
        ("strides", C.c_int64 * MAX_DIMS),
        ("offset", C.c_int64),
        ("base", C.c_void_p),
        ("device", C.c_int32),
        ("reserved", C.c_int32),
    ]


class Epilogue(C.Structure):
    """oxm_epilogue"""

    _fields_ = [("bias", C.POINTER(View)), ("activation", C.c_int32), ("accumulate", C.c_int32)]


ACT = {"none": 0, "relu": 1, "gelu": 2}


def make_view(dtype: int, shape, strides, offset: int, base: int | None, device: int) -> View:
    if len(shape) > MAX_DIMS:
        raise ValueError(f"rank {len(shape)} exceeds {MAX_DIMS}")
    v = View()
    v.dtype = int(dtype)
    v.ndim = len(shape)
    for i, (s, st) in enumerate(zip(shape, strides)):
        v.shape[i] = int(s)
        v.strides[i] = int(st)
    v.offset = int(offset)
    v.base = base
    v.device = int(device)
    return v


def library_path() -> str:
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), LIB_NAME)


_lib = None


def load() -> C.CDLL:
    """Load the CUDA library.  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if not os.path.exists(path):
        raise RuntimeError(
            f"{path} is missing: build it with `python -m oxmera_b200.build` "
            "(needs nvcc).  There is no fallback implementation."
        )
    lib = C.CDLL(path)
    p, i, i64, sz = C.c_void_p, C.c_int, C.c_int64, C.c_size_t
    PV = C.POINTER(View)
    sig = {
        "oxm_device_count": ([C.POINTER(i)], i),
        "oxm_ctx_create": ([i, C.POINTER(p)], i),
        "oxm_ctx_destroy": ([p], i),
        "oxm_ctx_device": ([p, C.POINTER(i)], i),
        "oxm_backend_name": ([], C.c_char_p),
        "oxm_last_error": ([], C.c_char_p),
        "oxm_status_name": ([i], C.c_char_p),
        "oxm_alloc": ([p, sz, C.POINTER(p)], i),
        "oxm_free": ([p, p], i),
        "oxm_h2d": ([p, p, p, sz], i),
        "oxm_d2h": ([p, p, p, sz], i),
        "oxm_memset": ([p, p, i, sz], i),
        "oxm_copy_peer": ([p, p, p, p, sz], i),
        "oxm_sync": ([p], i),
        "oxm_host_alloc": ([sz, C.POINTER(p)], i),
        "oxm_host_free": ([p], i),
        "oxm_matmul": ([p, PV, PV, PV], i),
        "oxm_batched_matmul": ([p, PV, PV, PV], i),
        "oxm_batched_matmul_host": ([p, PV, PV, PV], i),
        "oxm_contiguous": ([p, PV, PV], i),
        "oxm_unary": ([p, i, PV, PV], i),
        "oxm_binary": ([p, i, PV, PV, PV], i),
        "oxm_reduce": ([p, i, PV, C.POINTER(C.c_int32), i, PV], i),
        "oxm_matmul_fused": ([p, PV, PV, PV, C.POINTER(Epilogue)], i),
        "oxm_matmul_mx": ([p, PV, PV, PV, PV, PV], i),
        "oxm_matmul_f32_noalloc": ([p, PV, PV, PV], i),
        "oxm_event_create": ([p, C.POINTER(p)], i),
        "oxm_event_destroy": ([p], i),
        "oxm_event_record": ([p, p], i),
        "oxm_event_elapsed_ms": ([p, p, C.POINTER(C.c_float)], i),
        "oxm_stream_handle": ([p, C.POINTER(p)], i),
        "oxm_fill": ([p, p, i, i64, C.c_uint64, C.c_uint64, i, C.c_double], i),
        "oxm_selftest_bounded_wait": ([p, i64], i),
        "oxm_set_option": ([p, C.c_char_p, i64], i),
        "oxm_get_option": ([p, C.c_char_p, C.POINTER(i64)], i),
        "oxm_launch_counts": ([p, C.POINTER(i64)], i),
        "oxm_last_kernel": ([p], C.c_char_p),
        "oxm_memory_stats": ([p, C.POINTER(i64)], i),
        "oxm_plan_matmul": ([PV, PV, PV, i, C.POINTER(C.c_int32)], i),
    }
    for name, (argtypes, restype) in sig.items():
        fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
        fn.argtypes = argtypes
        fn.restype = restype
    _lib = lib
    return lib


def last_error() -> str:
    return load().oxm_last_error().decode()
