"""ctypes wrapper around the CPU oracle (oracle/oxm_oracle.c) for the tests,
the smoke check and the bench's CPU-baseline leg.  Test infrastructure: the
package never imports this."""
from __future__ import annotations

import ctypes as C
import importlib.util
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
MAX_DIMS = 8
F32, F64, BF16, F16 = 0, 1, 6, 7
F8E4M3, F8E5M2 = 8, 9
ACC_NATIVE, ACC_F64 = 0, 1
I32, I64 = 2, 3
U8 = 4
_NP = {F32: np.float32, F64: np.float64, I32: np.int32, I64: np.int64, BF16: np.uint16, F16: np.float16,
       F8E4M3: np.uint8, F8E5M2: np.uint8, U8: np.uint8}
_SIZE = {F32: 4, F64: 8, 2: 4, 3: 8, 4: 1, 5: 1, BF16: 2, F16: 2, F8E4M3: 1, F8E5M2: 1}


class OView(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("ndim", C.c_int32), ("shape", C.c_int64 * MAX_DIMS),
                ("strides", C.c_int64 * MAX_DIMS), ("offset", C.c_int64), ("base", C.c_void_p)]


def _view(arr: np.ndarray, tag: int) -> OView:
    v = OView()
    v.dtype, v.ndim = tag, arr.ndim
    for i in range(arr.ndim):
        v.shape[i] = arr.shape[i]
        v.strides[i] = arr.strides[i] // _SIZE[tag]
    v.offset = 0
    v.base = arr.ctypes.data
    return v


def _build() -> str:
    spec = importlib.util.spec_from_file_location("oracle_build", os.path.join(ROOT, "oracle", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.build_oracle()


class Oracle:
    def __init__(self):
        path = os.path.join(ROOT, "oracle", "liboxm_oracle.so")
        if not os.path.exists(path):
            path = _build()
        self.lib = C.CDLL(path)
        PV = C.POINTER(OView)
        self.lib.orc_matmul.argtypes = [PV, PV, PV, C.c_int, C.c_int]
        self.lib.orc_batched_matmul.argtypes = [PV, PV, PV, C.c_int, C.c_int]
        self.lib.orc_check_matmul.argtypes = [PV, PV, PV, C.c_int]
        self.lib.orc_matmul_fused.argtypes = [PV, PV, PV, PV, C.c_int, C.c_int, C.c_int, C.c_int]
        self.lib.orc_matmul_mx.argtypes = [PV, PV, PV, PV, PV]
        self.lib.orc_unary.argtypes = [C.c_int, PV, PV]
        self.lib.orc_binary.argtypes = [C.c_int, PV, PV, PV]
        self.lib.orc_reduce.argtypes = [C.c_int, PV, C.POINTER(C.c_int32), C.c_int, PV]
        self.lib.orc_broadcast_shapes.argtypes = [C.POINTER(C.c_int64), C.c_int, C.POINTER(C.c_int64), C.c_int,
                                                  C.POINTER(C.c_int64), C.POINTER(C.c_int)]
        self.lib.orc_f32_to_bf16.argtypes = [C.c_float]; self.lib.orc_f32_to_bf16.restype = C.c_uint16
        self.lib.orc_bf16_to_f32.argtypes = [C.c_uint16]; self.lib.orc_bf16_to_f32.restype = C.c_float
        self.lib.orc_f32_to_f16.argtypes = [C.c_float]; self.lib.orc_f32_to_f16.restype = C.c_uint16
        self.lib.orc_f16_to_f32.argtypes = [C.c_uint16]; self.lib.orc_f16_to_f32.restype = C.c_float
        self.lib.orc_f32_to_fp8.argtypes = [C.c_float, C.c_int32]; self.lib.orc_f32_to_fp8.restype = C.c_uint8
        self.lib.orc_fp8_to_f32.argtypes = [C.c_uint8, C.c_int32]; self.lib.orc_fp8_to_f32.restype = C.c_float
        self.lib.orc_fill.argtypes = [C.c_void_p, C.c_int32, C.c_int64, C.c_uint64, C.c_uint64, C.c_int, C.c_double, C.c_int]
        self.lib.orc_fill.restype = C.c_int
        self.threads = os.cpu_count() or 1

    def matmul(self, a: np.ndarray, b: np.ndarray, tag: int, acc: int = ACC_NATIVE, out_tag: int | None = None,
               batched: bool | None = None, nthreads: int | None = None):
        """Returns (status, out).  a, b: numpy arrays with any strides (bf16 as
        uint16 bits).  out_tag defaults to f32 (native) / f64 (f64 acc)."""
        if out_tag is None:
            out_tag = F64 if acc == ACC_F64 else F32
        if batched is None:
            batched = not (a.ndim == 2 and b.ndim == 2)
        va, vb = _view(a, tag), _view(b, tag)
        st = self.lib.orc_check_matmul(C.byref(va), C.byref(vb), None, 1 if batched else 0)
        if st != 0:
            return st, None
        lead = np.broadcast_shapes(a.shape[:-2], b.shape[:-2])
        out = np.zeros(tuple(lead) + (a.shape[-2], b.shape[-1]), dtype=_NP[out_tag])
        vo = _view(out, out_tag)
        fn = self.lib.orc_batched_matmul if batched else self.lib.orc_matmul
        st = fn(C.byref(va), C.byref(vb), C.byref(vo), acc, nthreads or self.threads)
        return st, out

    def matmul_fused(self, a, b, tag, bias=None, act=0, prev=None, acc=ACC_F64, nthreads=None):
        """act(a.b + bias) (+ prev).  `prev` is the previous output as a float
        array of the result's shape; the result has the accumulator's dtype."""
        lead = np.broadcast_shapes(a.shape[:-2], b.shape[:-2])
        odt = F64 if acc == ACC_F64 else F32
        out = np.zeros(tuple(lead) + (a.shape[-2], b.shape[-1]), dtype=_NP[odt])
        if prev is not None:
            out[...] = prev
        va, vb, vo = _view(a, tag), _view(b, tag), _view(out, odt)
        vbias = _view(bias, tag) if bias is not None else None
        st = self.lib.orc_matmul_fused(C.byref(va), C.byref(vb), C.byref(vo), C.byref(vbias) if vbias is not None else None,
                                       act, 1 if prev is not None else 0, acc, nthreads or self.threads)
        return st, out

    def matmul_mx(self, a, a_scale, b, b_scale, tag):
        """The block-scaled fp8 product in double: a, b fp8 bytes; a_scale
        [.., M, K/32] and b_scale [.., K/32, N] E8M0 bytes."""
        lead = np.broadcast_shapes(a.shape[:-2], b.shape[:-2])
        out = np.zeros(tuple(lead) + (a.shape[-2], b.shape[-1]), dtype=np.float64)
        va, vsa, vb, vsb, vo = _view(a, tag), _view(a_scale, U8), _view(b, tag), _view(b_scale, U8), _view(out, F64)
        st = self.lib.orc_matmul_mx(C.byref(va), C.byref(vsa), C.byref(vb), C.byref(vsb), C.byref(vo))
        return st, out

    def unary(self, op: int, a: np.ndarray, tag: int):
        out = np.zeros(a.shape, dtype=_NP[tag])
        va, vo = _view(a, tag), _view(out, tag)
        return self.lib.orc_unary(op, C.byref(va), C.byref(vo)), out

    def binary(self, op: int, a: np.ndarray, b: np.ndarray, tag: int):
        try:
            shape = np.broadcast_shapes(a.shape, b.shape)
        except ValueError:
            return 2, None
        out = np.zeros(shape, dtype=_NP[tag])
        va, vb, vo = _view(a, tag), _view(b, tag), _view(out, tag)
        return self.lib.orc_binary(op, C.byref(va), C.byref(vb), C.byref(vo)), out

    def reduce(self, op: int, a: np.ndarray, axes, tag: int):
        ax = sorted(set(axes)) if axes else list(range(a.ndim))
        out = np.zeros([s for d, s in enumerate(a.shape) if d not in ax], dtype=_NP[tag])
        arr = (C.c_int32 * max(len(axes), 1))(*axes)
        va, vo = _view(a, tag), _view(out, tag)
        return self.lib.orc_reduce(op, C.byref(va), arr, len(axes), C.byref(vo)), out

    def broadcast_shapes(self, lhs, rhs):
        l = (C.c_int64 * MAX_DIMS)(*lhs)
        r = (C.c_int64 * MAX_DIMS)(*rhs)
        o = (C.c_int64 * MAX_DIMS)()
        n = C.c_int()
        st = self.lib.orc_broadcast_shapes(l, len(lhs), r, len(rhs), o, C.byref(n))
        return st, tuple(o[i] for i in range(n.value)) if st == 0 else None

    def fill(self, shape, tag: int, seed: int, stream: int, dist: str, scale: float = 1.0) -> np.ndarray:
        """Seeded synthetic data: dist 'uniform' = U(-1,1), 'normal' = N(0,1)*scale."""
        out = np.empty(shape, dtype=_NP[tag])
        st = self.lib.orc_fill(out.ctypes.data, tag, out.size, seed, stream, 0 if dist == "uniform" else 1, scale, self.threads)
        assert st == 0, f"orc_fill refuses dtype tag {tag}"
        return out

    def fp8_to_f32(self, bits: np.ndarray, tag: int) -> np.ndarray:
        table = np.array([self.lib.orc_fp8_to_f32(i, tag) for i in range(256)], np.float32)
        return table[bits]

    def bf16_to_f32(self, bits: np.ndarray) -> np.ndarray:
        return (bits.astype(np.uint32) << 16).view(np.float32)
