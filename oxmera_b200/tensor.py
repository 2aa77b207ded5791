"""Storage and Tensor: shared device storage viewed through a layout.

Mirrors oxmera-tensor (crates/oxmera-tensor/src/{storage,tensor}.rs) with the
device variant of StorageData the reference leaves out: the bytes live in
B200 HBM, owned through the backend's C ABI.  Host data is exchanged as numpy
arrays; bf16 travels as raw uint16 bit patterns.
"""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import numpy as np

from . import capi
from .core import (DType, Device, Layout, ShapeMismatch, OxmeraError, UnsupportedDType, DeviceMismatch,
                   contiguous_strides, numel)

_NP_OF = {DType.F32: np.float32, DType.F64: np.float64, DType.I32: np.int32, DType.I64: np.int64,
          DType.U8: np.uint8, DType.Bool: np.bool_, DType.BF16: np.uint16, DType.F16: np.float16,
          DType.F8E4M3: np.uint8, DType.F8E5M2: np.uint8}


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round float32 to bfloat16 (nearest, ties to even); returns uint16 bits."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return r.astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


class Storage:
    """An owned buffer of elements on one device
    (crates/oxmera-tensor/src/storage.rs:12-17).  Freed when the last tensor
    viewing it goes away."""

    def __init__(self, backend, nbytes: int, dtype: DType, numel_: int):
        self.backend = backend
        self.dtype = dtype
        self.numel = numel_
        self.nbytes = nbytes
        self.ptr = backend._alloc(nbytes)

    def device(self) -> Device:
        return self.backend.device()

    def cpu_bytes(self):
        """None for device storage (crates/oxmera-tensor/src/storage.rs:59-67)."""
        return None

    def __del__(self):
        try:
            if getattr(self, "ptr", None):
                self.backend._free(self.ptr)
                self.ptr = None
        except Exception:
            pass


class Tensor:
    """storage + layout (crates/oxmera-tensor/src/tensor.rs:15-19).  Views
    share storage; nothing here copies except `contiguous` and the host
    transfers."""

    def __init__(self, storage: Storage, layout: Layout):
        lo, hi = layout.extent()
        if numel(layout.shape) > 0 and (lo < 0 or hi >= storage.numel):
            raise OxmeraError(f"layout {layout} addresses elements outside a storage of {storage.numel}")
        self._storage = storage
        self._layout = layout

    # ---- construction / host exchange ----
    @staticmethod
    def from_storage(storage: Storage, layout: Layout) -> "Tensor":
        return Tensor(storage, layout)

    @staticmethod
    def from_host(data: np.ndarray, shape: Sequence[int], dtype: DType, backend) -> "Tensor":
        """A contiguous device tensor holding `data` (the device analogue of
        Tensor::from_vec_f32, crates/oxmera-tensor/src/tensor.rs:29-36)."""
        shape = tuple(int(s) for s in shape)
        arr = np.ascontiguousarray(data, dtype=_NP_OF[dtype]).reshape(-1)
        if arr.size != numel(shape):
            raise ShapeMismatch(shape, (arr.size,), "from_host")
        t = Tensor.empty(shape, dtype, backend)
        if arr.size:
            backend._h2d(t._storage.ptr, arr.ctypes.data, arr.nbytes)
        t._keepalive = arr  # the copy is asynchronous
        return t

    @staticmethod
    def empty(shape: Sequence[int], dtype: DType, backend) -> "Tensor":
        shape = tuple(int(s) for s in shape)
        n = numel(shape)
        st = Storage(backend, n * dtype.size_in_bytes(), dtype, n)
        return Tensor(st, Layout.contiguous(shape))

    def to_host(self) -> np.ndarray:
        """The elements in logical order as a numpy array of this view's shape
        (bf16 as uint16 bits).  The storage range the view touches is copied
        once and re-strided on the host; no device gather is needed."""
        L = self._layout
        npdt = _NP_OF[self.dtype]
        if numel(L.shape) == 0:
            self._storage.backend.synchronize()
            return np.empty(L.shape, dtype=npdt)
        lo, hi = L.extent()
        esz = self.dtype.size_in_bytes()
        raw = np.empty(hi - lo + 1, dtype=npdt)
        self._storage.backend._d2h(raw.ctypes.data, self._storage.ptr + lo * esz, raw.nbytes)
        view = np.lib.stride_tricks.as_strided(raw[L.offset - lo:], shape=L.shape,
                                               strides=tuple(st * esz for st in L.strides), writeable=False)
        return np.array(view, copy=True)

    def to_host_f32(self) -> np.ndarray:
        h = self.to_host()
        if self.dtype == DType.BF16:
            return bf16_bits_to_f32(h).reshape(self.shape)
        return h.astype(np.float32)

    # ---- accessors ----
    @property
    def shape(self):
        return self._layout.shape

    def layout(self) -> Layout:
        return self._layout

    @property
    def dtype(self) -> DType:
        return self._storage.dtype

    def device(self) -> Device:
        return self._storage.device()

    def storage(self) -> Storage:
        return self._storage

    # ---- views (crates/oxmera-tensor/src/tensor.rs:63-90) ----
    def reshape(self, shape: Sequence[int]) -> "Tensor":
        shape = tuple(int(s) for s in shape)
        if numel(shape) != numel(self.shape):
            raise ShapeMismatch(self.shape, shape, "reshape")
        if not self._layout.is_contiguous():
            raise OxmeraError("reshape of a non-contiguous view would copy; call contiguous() first")
        return Tensor(self._storage, Layout(shape, contiguous_strides(shape), self._layout.offset))

    def permute(self, perm: Sequence[int]) -> "Tensor":
        perm = [int(p) for p in perm]
        if sorted(perm) != list(range(len(self.shape))):
            raise OxmeraError(f"{perm} is not a permutation of 0..{len(self.shape)}")
        L = self._layout
        return Tensor(self._storage, Layout(tuple(L.shape[p] for p in perm), tuple(L.strides[p] for p in perm), L.offset))

    def narrow(self, dim: int, start: int, length: int) -> "Tensor":
        L = self._layout
        if dim < 0 or dim >= len(L.shape):
            raise OxmeraError(f"narrow: no dim {dim} in shape {list(L.shape)}")
        if start < 0 or length < 0 or start + length > L.shape[dim]:
            raise OxmeraError(f"narrow: [{start}, {start + length}) exceeds extent {L.shape[dim]}")
        shape = list(L.shape)
        shape[dim] = length
        return Tensor(self._storage, Layout(tuple(shape), L.strides, L.offset + start * L.strides[dim]))

    def flip(self, dim: int) -> "Tensor":
        """Reverse a dim: the negative-stride view signed strides exist for
        (crates/oxmera-core/src/layout.rs:8)."""
        L = self._layout
        strides = list(L.strides)
        off = L.offset + (L.shape[dim] - 1) * strides[dim] if L.shape[dim] > 0 else L.offset
        strides[dim] = -strides[dim]
        return Tensor(self._storage, Layout(L.shape, tuple(strides), off))

    def contiguous(self) -> "Tensor":
        """Logical order in fresh storage; shares storage when already
        contiguous.  The gather is the backend's strided-copy kernel."""
        if self._layout.is_contiguous():
            return self
        return self._storage.backend._materialize(self)

    # ---- the operator surface (TensorOps, crates/oxmera-runtime/src/lib.rs:57-72) ----
    def matmul(self, rhs: "Tensor") -> "Tensor":
        from .backend import backend_for
        return backend_for(self.device()).matmul(self, rhs)

    def batched_matmul(self, rhs: "Tensor") -> "Tensor":
        from .backend import backend_for
        return backend_for(self.device()).batched_matmul(self, rhs)

    def _be(self):
        from .backend import backend_for
        return backend_for(self.device())

    def add(self, rhs: "Tensor") -> "Tensor":
        return self._be().add(self, rhs)

    def sub(self, rhs: "Tensor") -> "Tensor":
        return self._be().sub(self, rhs)

    def mul(self, rhs: "Tensor") -> "Tensor":
        return self._be().mul(self, rhs)

    def div(self, rhs: "Tensor") -> "Tensor":
        return self._be().div(self, rhs)

    def neg(self) -> "Tensor":
        return self._be().neg(self)

    def sum(self, axes: Sequence[int] = ()) -> "Tensor":
        return self._be().sum(self, axes)

    def get_f32(self, index: Sequence[int]) -> float:
        """One element, for tests (crates/oxmera-tensor/src/tensor.rs:92-100)."""
        if not self.dtype.is_float():
            raise UnsupportedDType(self.dtype, "get_f32")
        off = self._layout.offset_of(list(index))
        esz = self.dtype.size_in_bytes()
        buf = np.empty(1, dtype=_NP_OF[self.dtype])
        self._storage.backend._d2h(buf.ctypes.data, self._storage.ptr + off * esz, esz)
        if self.dtype == DType.BF16:
            return float(bf16_bits_to_f32(buf)[0])
        return float(buf[0])

    def _view(self) -> capi.View:
        L = self._layout
        return capi.make_view(int(self.dtype), L.shape, L.strides, L.offset, self._storage.ptr,
                              self._storage.backend.device().index)
