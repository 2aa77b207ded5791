"""The B200 backend and the dispatch seam.

Mirrors oxmera-runtime (crates/oxmera-runtime/src/lib.rs:29-72): a `Backend`
is the union of the op traits plus identity; `backend_for` resolves a device
handle to the registered backend or raises BackendUnavailable; tensors route
`matmul` through it.  `B200Backend` implements MatmulOps
(crates/oxmera-ops/src/lib.rs:53-59) and its batched extension over the C ABI.
The elementwise and reduction families (UnaryOps, BinaryOps, ReduceOps) go
through `oxm_unary` / `oxm_binary` / `oxm_reduce`.
"""
from __future__ import annotations

import ctypes as C
import threading
from typing import Dict, List, Sequence

import numpy as np

from . import capi
from .core import (BackendFault, BackendUnavailable, BroadcastIncompatible, DType, Device, DeviceMismatch, DivisionByZero,
                   DTypeMismatch, IndexOutOfBounds, Layout, NotImplementedOp, OxmeraError, ShapeMismatch, UnsupportedDType,
                   broadcast_shapes)
from .tensor import Tensor


def _raise(status: int, op: str, a: Tensor | None = None, b: Tensor | None = None):
    """Turn a C-ABI status into the typed error of oxmera_core::Error."""
    detail = capi.last_error()
    if status == capi.SHAPE_MISMATCH:
        raise ShapeMismatch(a.shape if a is not None else (), b.shape if b is not None else (), op, detail)
    if status == capi.BROADCAST_INCOMPATIBLE:
        raise BroadcastIncompatible(a.shape if a is not None else (), b.shape if b is not None else (), detail)
    if status == capi.DTYPE_MISMATCH:
        raise DTypeMismatch(a.dtype if a is not None else None, b.dtype if b is not None else None, op, detail)
    if status == capi.UNSUPPORTED_DTYPE:
        raise UnsupportedDType(a.dtype if a is not None else None, op, detail)
    if status == capi.DEVICE_MISMATCH:
        raise DeviceMismatch(a.device() if a is not None else None, b.device() if b is not None else None, op, detail)
    if status == capi.INDEX_OUT_OF_BOUNDS:
        raise IndexOutOfBounds((), a.shape if a is not None else ())
    if status == capi.BACKEND_UNAVAILABLE:
        raise BackendUnavailable(None, detail)
    if status == capi.NOT_IMPLEMENTED:
        raise NotImplementedOp(op, detail)
    if status == capi.DIVIDE_BY_ZERO:
        raise DivisionByZero(op, detail)
    raise BackendFault(status, f"{op}: {capi.load().oxm_status_name(status).decode()}: {detail}")


class B200Backend:
    """One instance serves one Device::Cuda{index}.  Thread-safe: the C
    library serialises launches per context (`Backend: Send + Sync`)."""

    def __init__(self, index: int = 0):
        self._lib = capi.load()
        self._index = index
        ctx = C.c_void_p()
        st = self._lib.oxm_ctx_create(index, C.byref(ctx))
        if st != capi.OK:
            if st == capi.BACKEND_UNAVAILABLE:
                raise BackendUnavailable(Device.cuda(index), capi.last_error())
            _raise(st, "ctx_create")
        self._ctx = ctx
        self._pinned: List[int] = []

    # ---- identity (crates/oxmera-runtime/src/lib.rs:30-33) ----
    def device(self) -> Device:
        return Device.cuda(self._index)

    def name(self) -> str:
        return self._lib.oxm_backend_name().decode()

    # ---- MatmulOps ----
    def matmul(self, lhs: Tensor, rhs: Tensor) -> Tensor:
        """[m,k] x [k,n] -> [m,n], rank 2 exactly; a fresh contiguous tensor
        on the operands' device (crates/oxmera-ops/src/lib.rs:16-17,53-59)."""
        return self._mm(lhs, rhs, batched=False)

    def batched_matmul(self, lhs: Tensor, rhs: Tensor) -> Tensor:
        """Rank >= 2; leading dims broadcast by NumPy rules."""
        return self._mm(lhs, rhs, batched=True)

    def matmul_as(self, lhs: Tensor, rhs: Tensor, out_dtype: DType) -> Tensor:
        """Batched product of fp8 operands kept in a wider dtype (bf16, f16 or f32)."""
        bshape = broadcast_shapes(lhs.shape[:-2], rhs.shape[:-2])
        out = Tensor.empty(tuple(bshape) + (lhs.shape[-2], rhs.shape[-1]), out_dtype, self)
        return self.matmul_into(lhs, rhs, out, batched=True)

    def matmul_into(self, lhs: Tensor, rhs: Tensor, out: Tensor, batched: bool = True) -> Tensor:
        """Write the product through `out`'s layout (a shard writing into a
        window of its parent).  `out` must not alias the operands."""
        fn = self._lib.oxm_batched_matmul if batched else self._lib.oxm_matmul
        st = fn(self._ctx, C.byref(lhs._view()), C.byref(rhs._view()), C.byref(out._view()))
        if st != capi.OK:
            _raise(st, "batched_matmul" if batched else "matmul", lhs, rhs)
        return out

    def prepare_matmul(self, lhs: Tensor, rhs: Tensor, out: Tensor, batched: bool = True):
        """The same call as `matmul_into` with the three `oxm_view` structs built
        once: returns a function of no arguments that submits the product.  A
        loop that multiplies the same tensors again and again (a benchmark, a
        training step) then pays the C call alone, not the marshalling of the
        views - which for a product of a few microseconds is most of the time."""
        fn = self._lib.oxm_batched_matmul if batched else self._lib.oxm_matmul
        va, vb, vo = lhs._view(), rhs._view(), out._view()
        pa, pb, po, ctx = C.byref(va), C.byref(vb), C.byref(vo), self._ctx
        keep = (va, vb, vo, lhs, rhs, out)  # the structs and the storages stay alive with the closure

        def submit(_keep=keep):
            st = fn(ctx, pa, pb, po)
            if st != capi.OK:
                _raise(st, "batched_matmul" if batched else "matmul", lhs, rhs)

        return submit

    def matmul_fused(self, lhs: Tensor, rhs: Tensor, bias: Tensor | None = None, activation: str = "none",
                     accumulate_into: Tensor | None = None) -> Tensor:
        """act(lhs . rhs + bias), optionally added into an existing tensor
        (gradient accumulation), in one kernel.  Shapes broadcast as in
        batched_matmul; bias is a rank-1 tensor over the output's columns."""
        if accumulate_into is None:
            bshape = broadcast_shapes(lhs.shape[:-2], rhs.shape[:-2])
            out = Tensor.empty(tuple(bshape) + (lhs.shape[-2], rhs.shape[-1]), lhs.dtype, self)
        else:
            out = accumulate_into
        ep = capi.Epilogue()
        bias_view = bias._view() if bias is not None else None
        ep.bias = C.pointer(bias_view) if bias_view is not None else None
        ep.activation = capi.ACT[activation]
        ep.accumulate = 1 if accumulate_into is not None else 0
        st = self._lib.oxm_matmul_fused(self._ctx, C.byref(lhs._view()), C.byref(rhs._view()), C.byref(out._view()),
                                        C.byref(ep))
        if st != capi.OK:
            _raise(st, "matmul_fused", lhs, rhs)
        return out

    def matmul_mx(self, lhs: Tensor, lhs_scale: Tensor, rhs: Tensor, rhs_scale: Tensor,
                  out_dtype: DType = DType.BF16) -> Tensor:
        """The block-scaled fp8 product (MXFP8): lhs and rhs are fp8 tensors,
        lhs_scale [.., M, K/32] and rhs_scale [.., K/32, N] hold one E8M0
        exponent (a U8) per 32 contraction elements of every row of lhs and
        column of rhs.  Shapes broadcast as in batched_matmul; the result is
        a fresh tensor of `out_dtype`."""
        if len(lhs.shape) < 2 or len(rhs.shape) < 2:
            raise ShapeMismatch(lhs.shape, rhs.shape, "matmul_mx", "expected operands of rank >= 2")
        bshape = broadcast_shapes(lhs.shape[:-2], rhs.shape[:-2])
        rows, cols = lhs.shape[-2], rhs.shape[-1]
        out = Tensor.empty(tuple(bshape) + (rows, cols), out_dtype, self)
        self.matmul_mx_into(lhs, lhs_scale, rhs, rhs_scale, out)
        return out

    def prepare_matmul_mx(self, lhs: Tensor, lhs_scale: Tensor, rhs: Tensor, rhs_scale: Tensor, out: Tensor):
        """`matmul_mx_into` with the views marshalled once (see prepare_matmul)."""
        views = [t._view() for t in (lhs, lhs_scale, rhs, rhs_scale, out)]
        ptrs = [C.byref(v) for v in views]
        fn, ctx = self._lib.oxm_matmul_mx, self._ctx
        keep = (views, lhs, lhs_scale, rhs, rhs_scale, out)

        def submit(_keep=keep):
            st = fn(ctx, *ptrs)
            if st != capi.OK:
                _raise(st, "matmul_mx", lhs, rhs)

        return submit

    def matmul_mx_into(self, lhs: Tensor, lhs_scale: Tensor, rhs: Tensor, rhs_scale: Tensor, out: Tensor) -> None:
        st = self._lib.oxm_matmul_mx(self._ctx, C.byref(lhs._view()), C.byref(lhs_scale._view()), C.byref(rhs._view()),
                                     C.byref(rhs_scale._view()), C.byref(out._view()))
        if st != capi.OK:
            _raise(st, "matmul_mx", lhs, rhs)

    def _mm(self, lhs: Tensor, rhs: Tensor, batched: bool) -> Tensor:
        op = "batched_matmul" if batched else "matmul"
        for t in (lhs, rhs):
            if t.device() != self.device():
                raise DeviceMismatch(t.device(), self.device(), op)
        # The output shape: validation proper happens in the C library, which
        # reports the typed error; here only enough to allocate.
        la, lb = lhs.shape, rhs.shape
        if len(la) >= 2 and len(lb) >= 2 and (batched or (len(la) == 2 and len(lb) == 2)):
            try:
                bshape = broadcast_shapes(la[:-2], lb[:-2])
            except BroadcastIncompatible:
                raise BroadcastIncompatible(la, lb)
            oshape = tuple(bshape) + (la[-2], lb[-1])
        else:
            oshape = (1, 1)  # placeholder; the library refuses the ranks
        out = Tensor.empty(oshape, lhs.dtype, self)
        return self.matmul_into(lhs, rhs, out, batched)

    def matmul_host(self, a: np.ndarray, b: np.ndarray, dtype: DType, out: np.ndarray | None = None) -> np.ndarray:
        """Product of two HOST arrays (any numpy strides): staged to the
        device, multiplied, copied back (into `out` when given, e.g. a
        page-locked buffer).  bf16 arrays are uint16 bits."""
        bshape = broadcast_shapes(a.shape[:-2], b.shape[:-2])
        if out is None:
            out = np.empty(tuple(bshape) + (a.shape[-2], b.shape[-1]), dtype=a.dtype)
        esz = dtype.size_in_bytes()
        va = capi.make_view(int(dtype), a.shape, [s // esz for s in a.strides], 0, a.ctypes.data, self._index)
        vb = capi.make_view(int(dtype), b.shape, [s // esz for s in b.strides], 0, b.ctypes.data, self._index)
        vo = capi.make_view(int(dtype), out.shape, [s // esz for s in out.strides], 0, out.ctypes.data, self._index)
        st = self._lib.oxm_batched_matmul_host(self._ctx, C.byref(va), C.byref(vb), C.byref(vo))
        if st != capi.OK:
            _raise(st, "batched_matmul")
        return out

    # ---- UnaryOps / BinaryOps / ReduceOps (crates/oxmera-ops/src/lib.rs:27-50,61-69) ----
    def _unary(self, op: int, name: str, a: Tensor) -> Tensor:
        out = Tensor.empty(a.shape, a.dtype, self)
        st = self._lib.oxm_unary(self._ctx, op, C.byref(a._view()), C.byref(out._view()))
        if st != capi.OK:
            _raise(st, name, a)
        return out

    def _binary(self, op: int, name: str, lhs: Tensor, rhs: Tensor) -> Tensor:
        for t in (lhs, rhs):
            if t.device() != self.device():
                raise DeviceMismatch(t.device(), self.device(), name)
        out = Tensor.empty(broadcast_shapes(lhs.shape, rhs.shape), lhs.dtype, self)
        st = self._lib.oxm_binary(self._ctx, op, C.byref(lhs._view()), C.byref(rhs._view()), C.byref(out._view()))
        if st != capi.OK:
            _raise(st, name, lhs, rhs)
        return out

    def _reduce(self, op: int, name: str, a: Tensor, axes: Sequence[int]) -> Tensor:
        axes = [int(x) for x in axes]
        drop = set(axes) if axes else set(range(len(a.shape)))
        if any(x < 0 or x >= len(a.shape) for x in axes) or len(set(axes)) != len(axes):
            raise IndexOutOfBounds(axes, a.shape)
        out = Tensor.empty(tuple(s for d, s in enumerate(a.shape) if d not in drop), a.dtype, self)
        arr = (C.c_int32 * max(len(axes), 1))(*axes)
        st = self._lib.oxm_reduce(self._ctx, op, C.byref(a._view()), arr, len(axes), C.byref(out._view()))
        if st != capi.OK:
            _raise(st, name, a)
        return out

    def neg(self, a): return self._unary(0, "neg", a)
    def exp(self, a): return self._unary(1, "exp", a)
    def ln(self, a): return self._unary(2, "ln", a)
    def abs(self, a): return self._unary(3, "abs", a)
    def add(self, lhs, rhs): return self._binary(0, "add", lhs, rhs)
    def sub(self, lhs, rhs): return self._binary(1, "sub", lhs, rhs)
    def mul(self, lhs, rhs): return self._binary(2, "mul", lhs, rhs)
    def div(self, lhs, rhs): return self._binary(3, "div", lhs, rhs)
    def sum(self, a, axes=()): return self._reduce(0, "sum", a, axes)
    def max(self, a, axes=()): return self._reduce(1, "max", a, axes)

    # ---- storage plumbing used by Tensor ----
    def _alloc(self, nbytes: int) -> int:
        p = C.c_void_p()
        st = self._lib.oxm_alloc(self._ctx, nbytes, C.byref(p))
        if st != capi.OK:
            _raise(st, "alloc")
        return p.value

    def _free(self, ptr: int) -> None:
        if self._ctx:
            self._lib.oxm_free(self._ctx, ptr)

    def _h2d(self, dst: int, src: int, nbytes: int) -> None:
        st = self._lib.oxm_h2d(self._ctx, dst, src, nbytes)
        if st != capi.OK:
            _raise(st, "h2d")
        # numpy buffers are pageable: the runtime stages them before returning

    def _d2h(self, dst: int, src: int, nbytes: int) -> None:
        st = self._lib.oxm_d2h(self._ctx, dst, src, nbytes)
        if st != capi.OK:
            _raise(st, "d2h")

    def _materialize(self, t: Tensor) -> Tensor:
        out = Tensor.empty(t.shape, t.dtype, self)
        st = self._lib.oxm_contiguous(self._ctx, C.byref(t._view()), C.byref(out._view()))
        if st != capi.OK:
            _raise(st, "contiguous", t, out)
        return out

    def synthetic(self, shape: Sequence[int], dtype: DType, seed: int, stream: int, dist: str = "normal",
                  scale: float = 1.0) -> Tensor:
        """A contiguous tensor of seeded synthetic data generated on the device:
        dist "uniform" = U(-1,1), "normal" = N(0,1) * scale."""
        t = Tensor.empty(shape, dtype, self)
        n = 1
        for s_ in t.shape:
            n *= s_
        st = self._lib.oxm_fill(self._ctx, t.storage().ptr, int(dtype), n, seed, stream,
                                0 if dist == "uniform" else 1, scale)
        if st != capi.OK:
            _raise(st, "fill")
        return t

    def pinned_empty(self, shape: Sequence[int], np_dtype) -> np.ndarray:
        """A numpy array over page-locked host memory (freed with the backend)."""
        n = int(np.prod(shape)) * np.dtype(np_dtype).itemsize
        p = C.c_void_p()
        st = self._lib.oxm_host_alloc(max(n, 16), C.byref(p))
        if st != capi.OK:
            _raise(st, "host_alloc")
        self._pinned.append(p.value)
        buf = (C.c_uint8 * max(n, 16)).from_address(p.value)
        return np.frombuffer(buf, dtype=np_dtype, count=int(np.prod(shape))).reshape(shape)

    def synchronize(self) -> None:
        st = self._lib.oxm_sync(self._ctx)
        if st != capi.OK:
            _raise(st, "sync")

    # ---- instrumentation ----
    def set_option(self, key: str, value: int) -> None:
        st = self._lib.oxm_set_option(self._ctx, key.encode(), value)
        if st != capi.OK:
            _raise(st, "set_option")

    def launch_counts(self) -> Dict[str, int]:
        arr = (C.c_int64 * 4)()
        self._lib.oxm_launch_counts(self._ctx, arr)
        return {"total": arr[0], "tcgen05": arr[1], "simt": arr[2], "pack": arr[3]}

    def memory_stats(self) -> Dict[str, int]:
        """Bytes reserved / in use in the device's stream-ordered pool, and free / total on the device."""
        arr = (C.c_int64 * 4)()
        st = self._lib.oxm_memory_stats(self._ctx, arr)
        if st != capi.OK:
            _raise(st, "memory_stats")
        return {"pool_reserved": arr[0], "pool_used": arr[1], "device_free": arr[2], "device_total": arr[3]}

    def last_kernel(self) -> str:
        return self._lib.oxm_last_kernel(self._ctx).decode()

    def timer(self):
        return _Timer(self)

    def close(self) -> None:
        if self._ctx:
            self._lib.oxm_sync(self._ctx)
            for p in self._pinned:
                self._lib.oxm_host_free(p)
            self._pinned = []
            self._lib.oxm_ctx_destroy(self._ctx)
            self._ctx = None


class _Timer:
    """CUDA events on the backend's stream."""

    def __init__(self, backend: B200Backend):
        self.b = backend
        self.e0, self.e1 = C.c_void_p(), C.c_void_p()
        for e in (self.e0, self.e1):
            st = backend._lib.oxm_event_create(backend._ctx, C.byref(e))
            if st != capi.OK:
                _raise(st, "event_create")

    def start(self):
        self.b._lib.oxm_event_record(self.b._ctx, self.e0)

    def stop(self):
        self.b._lib.oxm_event_record(self.b._ctx, self.e1)

    def elapsed_ms(self) -> float:
        ms = C.c_float()
        st = self.b._lib.oxm_event_elapsed_ms(self.e0, self.e1, C.byref(ms))
        if st != capi.OK:
            _raise(st, "event_elapsed")
        return float(ms.value)


# ---------------------------------------------------------------------------
# registry (crates/oxmera-runtime/src/lib.rs:36-53)
# ---------------------------------------------------------------------------
_registry: Dict[Device, object] = {}
_registry_lock = threading.Lock()


def register_backend(backend) -> None:
    """Register a backend for its device, replacing any previous registration."""
    with _registry_lock:
        _registry[backend.device()] = backend


def backend_for(device: Device):
    """The backend serving `device`; an unregistered device is
    BackendUnavailable, never a crash."""
    with _registry_lock:
        b = _registry.get(device)
    if b is None:
        raise BackendUnavailable(device)
    return b


def unregister_all() -> None:
    with _registry_lock:
        _registry.clear()


# ---------------------------------------------------------------------------
# collective-free sharding over the GPUs of one box
# ---------------------------------------------------------------------------
def shard_ranges(total: int, parts: int) -> List[range]:
    """Split [0, total) into `parts` contiguous ranges whose sizes differ by at
    most one (the first `total % parts` ranges take the extra element)."""
    base, extra = divmod(total, parts)
    out, start = [], 0
    for r in range(parts):
        n = base + (1 if r < extra else 0)
        out.append(range(start, start + n))
        start += n
    return out


def shard_plan(a_shape: Sequence[int], b_shape: Sequence[int], parts: int):
    """How a matmul splits across `parts` devices with no exchange step:
    along the leading batch dim of the (broadcast) output when there is one,
    else along the M rows of A.  Returns (axis, ranges) with axis "batch" or
    "rows".  K is never split: that would need a reduction."""
    bshape = broadcast_shapes(tuple(a_shape)[:-2], tuple(b_shape)[:-2])
    if len(bshape) >= 1 and bshape[0] >= parts:
        return "batch", shard_ranges(bshape[0], parts)
    return "rows", shard_ranges(a_shape[-2], parts)


def sharded_matmul_host(backends: Sequence[B200Backend], a: np.ndarray, b: np.ndarray, dtype: DType) -> np.ndarray:
    """Multiply host arrays on several GPUs: each backend gets its slice of
    the batch (or of A's rows) plus whatever it needs of the other operand,
    one host thread per device; the first typed error is re-raised.  Nothing
    is reduced and no kernel reads another device's memory.

    An operand every device needs whole (B, unless it carries the sharded batch
    dim) crosses PCIe once, not once per device: each device uploads 1/N of its
    bytes and fetches the rest from its peers with device-to-device copies
    into its own memory (`oxm_copy_peer`) before its kernel is launched."""
    parts = len(backends)
    axis, ranges = shard_plan(a.shape, b.shape, parts)
    bshape = broadcast_shapes(a.shape[:-2], b.shape[:-2])
    out = np.empty(tuple(bshape) + (a.shape[-2], b.shape[-1]), dtype=a.dtype)
    errors: List[BaseException] = []
    lead = len(bshape)

    def cut(x, rg):
        if axis == "rows":
            return x
        pos = x.ndim - 2 - lead  # index of the leading batch dim in x, if it has one
        if pos < 0 or x.shape[pos] == 1:
            return x
        idx = [slice(None)] * x.ndim
        idx[pos] = slice(rg.start, rg.stop)
        return x[tuple(idx)]

    def a_part(rg):
        return a[..., rg.start:rg.stop, :] if axis == "rows" else cut(a, rg)

    esz = dtype.size_in_bytes()
    b_whole = all(cut(b, rg) is b for rg in ranges)
    per = b.nbytes // parts if parts else 0
    share_b = (parts > 1 and b_whole and b.flags["C_CONTIGUOUS"] and b.nbytes % (parts * 16) == 0 and
               all(len(rg) > 0 for rg in ranges) and all(isinstance(be, B200Backend) for be in backends))
    b_dev: List[Tensor | None] = [None] * parts
    gate = threading.Barrier(parts) if share_b else None

    def work(rank: int):
        try:
            rg = ranges[rank]
            if len(rg) == 0:
                return
            be = backends[rank]
            if not share_b:
                res = be.matmul_host(a_part(rg), cut(b, rg), dtype)
            else:
                try:
                    tb = Tensor.empty(b.shape, dtype, be)
                    flat = b.reshape(-1).view(np.uint8)
                    be._h2d(tb.storage().ptr + rank * per, flat[rank * per:(rank + 1) * per].ctypes.data, per)
                    b_dev[rank] = tb
                finally:
                    gate.wait()  # every device has queued the upload of its part (or failed: see below)
                if any(t is None for t in b_dev):
                    raise BackendFault(capi.CUDA_ERROR, "a peer could not stage its part of the shared operand")
                for q in range(parts):
                    if q != rank:
                        st = be._lib.oxm_copy_peer(be._ctx, tb.storage().ptr + q * per, backends[q]._ctx,
                                                   b_dev[q].storage().ptr + q * per, per)
                        if st != capi.OK:
                            _raise(st, "copy_peer")
                ha = np.ascontiguousarray(a_part(rg))
                ta = Tensor.from_host(ha, ha.shape, dtype, be)
                res = be.batched_matmul(ta, tb).to_host()
                gate.wait()  # nobody frees its copy while a peer may still be reading it
            if axis == "batch":
                out[rg.start:rg.stop] = res
            else:
                out[..., rg.start:rg.stop, :] = res
        except BaseException as e:  # propagate to the caller's thread
            errors.append(e)
            if gate is not None:
                gate.abort()

    threads = [threading.Thread(target=work, args=(r,)) for r in range(parts)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    if errors:
        first = [e for e in errors if not isinstance(e, threading.BrokenBarrierError)]
        raise (first or errors)[0]
    return out
