"""Vocabulary of the host mirror: dtypes, devices, shapes, layouts, errors.

Mirrors oxmera-core (crates/oxmera-core/src/{dtype,device,shape,layout,error}.rs)
so that host code and tests read like the reference's own.  Pure Python, no
GPU needed.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Sequence, Tuple


class DType(enum.IntEnum):
    """Element types.  0..5 follow crates/oxmera-core/src/dtype.rs:9-22; BF16,
    F16 and the two fp8 encodings are the variants the B200 backend adds.
    Values equal the C ABI's oxm_dtype."""

    F32 = 0
    F64 = 1
    I32 = 2
    I64 = 3
    U8 = 4
    Bool = 5
    BF16 = 6
    F16 = 7
    F8E4M3 = 8  # 1-4-3, finite only, max 448
    F8E5M2 = 9  # 1-5-2, IEEE-like

    def size_in_bytes(self) -> int:
        return {0: 4, 1: 8, 2: 4, 3: 8, 4: 1, 5: 1, 6: 2, 7: 2, 8: 1, 9: 1}[int(self)]

    def is_float(self) -> bool:
        return self in (DType.F32, DType.F64, DType.BF16, DType.F16, DType.F8E4M3, DType.F8E5M2)


@dataclass(frozen=True)
class Device:
    """A place, not a backend (crates/oxmera-core/src/device.rs:8-24)."""

    kind: str  # "cpu" | "metal" | "cuda"
    index: int = 0

    @staticmethod
    def cpu() -> "Device":
        return Device("cpu", 0)

    @staticmethod
    def cuda(index: int = 0) -> "Device":
        return Device("cuda", index)

    @staticmethod
    def metal(index: int = 0) -> "Device":
        return Device("metal", index)

    def kind_name(self) -> str:
        return self.kind

    def __repr__(self) -> str:  # mirrors Rust's Debug output
        if self.kind == "cpu":
            return "Cpu"
        return f"{self.kind.capitalize()} {{ index: {self.index} }}"


# ---------------------------------------------------------------------------
# errors: one exception class per variant of oxmera_core::Error
# (crates/oxmera-core/src/error.rs:12-102); messages follow its #[error] strings
# ---------------------------------------------------------------------------
class OxmeraError(Exception):
    """Any failure an oxmera operation can report."""


class ShapeMismatch(OxmeraError):
    def __init__(self, expected, got, op: str, detail: str | None = None):
        self.expected, self.got, self.op = tuple(expected), tuple(got), op
        super().__init__(detail or f"shape mismatch: expected {list(self.expected)}, got {list(self.got)} in {op}")


class BroadcastIncompatible(OxmeraError):
    def __init__(self, lhs, rhs, detail: str | None = None):
        self.lhs, self.rhs = tuple(lhs), tuple(rhs)
        super().__init__(detail or f"cannot broadcast {list(self.lhs)} with {list(self.rhs)}")


class DTypeMismatch(OxmeraError):
    def __init__(self, expected, got, op: str, detail: str | None = None):
        self.expected, self.got, self.op = expected, got, op
        super().__init__(detail or f"dtype mismatch: expected {getattr(expected, 'name', expected)}, got {getattr(got, 'name', got)} in {op}")


class UnsupportedDType(OxmeraError):
    def __init__(self, dtype, op: str, detail: str | None = None):
        self.dtype, self.op = dtype, op
        super().__init__(detail or f"dtype {getattr(dtype, 'name', dtype)} is not supported by {op}")


class DeviceMismatch(OxmeraError):
    def __init__(self, lhs, rhs, op: str, detail: str | None = None):
        self.lhs, self.rhs, self.op = lhs, rhs, op
        super().__init__(detail or f"device mismatch: {lhs!r} vs {rhs!r} in {op}")


class IndexOutOfBounds(OxmeraError):
    def __init__(self, index, shape):
        self.index, self.shape = list(index), tuple(shape)
        super().__init__(f"index {self.index} out of bounds for shape {list(self.shape)}")


class RankMismatch(OxmeraError):
    def __init__(self, index_rank: int, shape_rank: int):
        self.index_rank, self.shape_rank = index_rank, shape_rank
        super().__init__(f"rank mismatch: index of rank {index_rank} against shape of rank {shape_rank}")


class BackendUnavailable(OxmeraError):
    def __init__(self, device, detail: str | None = None):
        self.device = device
        super().__init__(detail or f"no backend available for device {device!r}")


class NotImplementedOp(OxmeraError):
    def __init__(self, op: str, detail: str):
        self.op, self.detail = op, detail
        super().__init__(f"{op} is not implemented for {detail}")


class DivisionByZero(OxmeraError):
    """Integer division met a zero divisor.  BinaryOps::div makes this "a typed
    error" (crates/oxmera-ops/src/lib.rs:47-49); oxmera's non_exhaustive Error
    has no variant for it yet, so this is the one the backend adds."""

    def __init__(self, op: str, detail: str | None = None):
        self.op = op
        super().__init__(detail or f"integer division by zero in {op}")


class BackendFault(OxmeraError):
    """A CUDA call failed or a bounded device-side wait expired.  The Rust
    side would fold this into NotImplemented{op, detail}; it is kept apart
    here so tests can tell the two."""

    def __init__(self, status: int, detail: str):
        self.status = status
        super().__init__(detail)


# ---------------------------------------------------------------------------
# shapes and layouts
# ---------------------------------------------------------------------------
Shape = Tuple[int, ...]


def numel(shape: Sequence[int]) -> int:
    """A scalar has one element; any zero extent empties the tensor
    (crates/oxmera-core/src/shape.rs:30-35)."""
    n = 1
    for d in shape:
        n *= int(d)
    return n


def contiguous_strides(shape: Sequence[int]) -> Tuple[int, ...]:
    """Row-major element strides (crates/oxmera-core/src/layout.rs:58-62).  An
    extent of 0 or 1 is stepped as if it were 1, so [2,1,3] gives [3,3,1]."""
    strides = [0] * len(shape)
    acc = 1
    for i in range(len(shape) - 1, -1, -1):
        strides[i] = acc
        acc *= max(int(shape[i]), 1)
    return tuple(strides)


def broadcast_shapes(lhs: Sequence[int], rhs: Sequence[int]) -> Shape:
    """NumPy's rule as a total function (crates/oxmera-core/src/shape.rs:49-58):
    align trailing dims; each pair must be equal or contain a 1."""
    lhs, rhs = tuple(int(x) for x in lhs), tuple(int(x) for x in rhs)
    n = max(len(lhs), len(rhs))
    out = [0] * n
    for i in range(n):
        l = lhs[len(lhs) - 1 - i] if i < len(lhs) else 1
        r = rhs[len(rhs) - 1 - i] if i < len(rhs) else 1
        if l == r:
            o = l
        elif l == 1:
            o = r
        elif r == 1:
            o = l
        else:
            raise BroadcastIncompatible(lhs, rhs)
        out[n - 1 - i] = o
    return tuple(out)


@dataclass(frozen=True)
class Layout:
    """shape + signed element strides + start offset in elements
    (crates/oxmera-core/src/layout.rs:26-56)."""

    shape: Shape
    strides: Tuple[int, ...]
    offset: int = 0

    @staticmethod
    def contiguous(shape: Sequence[int]) -> "Layout":
        shape = tuple(int(x) for x in shape)
        return Layout(shape, contiguous_strides(shape), 0)

    def offset_of(self, index: Sequence[int]) -> int:
        if len(index) != len(self.shape):
            raise RankMismatch(len(index), len(self.shape))
        off = self.offset
        for i, (ix, ext, st) in enumerate(zip(index, self.shape, self.strides)):
            if ix < 0 or ix >= ext:
                raise IndexOutOfBounds(index, self.shape)
            off += ix * st
        return off

    def is_contiguous(self) -> bool:
        """Row-major with no gaps; a scalar and any empty tensor count as
        contiguous.  Strides of extent-1 dims are never stepped and are
        ignored."""
        if numel(self.shape) == 0:
            return True
        acc = 1
        for ext, st in zip(reversed(self.shape), reversed(self.strides)):
            if ext != 1 and st != acc:
                return False
            acc *= ext
        return True

    def extent(self) -> Tuple[int, int]:
        """Lowest and highest storage element this layout touches."""
        lo = hi = self.offset
        for ext, st in zip(self.shape, self.strides):
            if ext > 0:
                span = (ext - 1) * st
                if span > 0:
                    hi += span
                else:
                    lo += span
        return lo, hi
