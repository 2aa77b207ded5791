"""Guard bands around device outputs (test infrastructure).

compute-sanitizer is not available to these tests, so an out-of-bounds store
has to be caught by hand: the output of a call is placed inside a larger
allocation whose every other byte holds a known pattern, and the pattern is
checked after the call.  Two layouts:

  "window"  the output is a window of a parent matrix with `ROWS` more rows
            above and below and `cols` more columns left and right (per batch
            entry), so a store that runs past a tile's edge in either
            direction lands in the margin;
  "flat"    the output is contiguous, with `PAD` elements before and after it,
            so a store past the end of a fresh contiguous tensor is seen.

The margins are written through oxm_memset and read back through oxm_d2h.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from oxmera_b200 import DType, Tensor, capi

PATTERN = 0xA5
ROWS = 40       # more than a 32-row store box
PAD = 4096      # elements; a multiple of 8, so a 16-byte-aligned parent keeps the output aligned


def _numel(shape):
    n = 1
    for s in shape:
        n *= int(s)
    return n


def _memset(backend, t: Tensor, byte: int):
    st = capi.load().oxm_memset(backend._ctx, t.storage().ptr, byte, _numel(t.shape) * t.dtype.size_in_bytes())
    assert st == capi.OK, capi.last_error()


class Guarded:
    """An output view of `shape` with guard bands around it.

    `aligned` keeps the view's base and row pitch on 16-byte boundaries (the
    bulk-tensor-store epilogue stays eligible); otherwise the margins are odd,
    which forces the strided-store epilogue."""

    def __init__(self, backend, shape, dtype: DType, layout: str = "window", aligned: bool = True):
        self.backend, self.shape, self.dtype, self.layout = backend, tuple(int(s) for s in shape), dtype, layout
        if layout == "flat" or len(self.shape) < 2:
            self.layout = "flat"
            self.pad = PAD if aligned else PAD + 3
            n = _numel(self.shape)
            self.parent = Tensor.empty((n + 2 * self.pad,), dtype, backend)
            _memset(backend, self.parent, PATTERN)
            self.view = self.parent.narrow(0, self.pad, n).reshape(self.shape) if n else Tensor.empty(self.shape, dtype, backend)
        else:
            self.cols = 64 if aligned else 67
            lead, (m, n) = self.shape[:-2], self.shape[-2:]
            self.parent = Tensor.empty(lead + (m + 2 * ROWS, n + 2 * self.cols), dtype, backend)
            _memset(backend, self.parent, PATTERN)
            nd = len(self.shape)
            self.view = self.parent.narrow(nd - 2, ROWS, m).narrow(nd - 1, self.cols, n)

    def result(self) -> np.ndarray:
        """Check every guard byte, then return the output as a host array."""
        if _numel(self.shape) == 0:
            return self.view.to_host()
        raw = self.parent.to_host()
        esz = self.dtype.size_in_bytes()
        bytes_ = raw.view(np.uint8).reshape(raw.shape + (esz,)) if raw.dtype.itemsize == esz else raw.view(np.uint8)
        if self.layout == "flat":
            n = _numel(self.shape)
            body = slice(self.pad, self.pad + n)
            mask = np.ones(raw.shape[0], bool)
            mask[body] = False
            touched = np.nonzero((bytes_[mask] != PATTERN).any(axis=-1))[0]
            assert touched.size == 0, f"{touched.size} guard elements around a contiguous {self.shape} output were written; first at guard index {int(touched[0])} (pad {self.pad})"
            return raw[body].reshape(self.shape)
        m, n = self.shape[-2:]
        mask = np.ones(raw.shape, bool)
        mask[..., ROWS:ROWS + m, self.cols:self.cols + n] = False
        bad = mask & (bytes_ != PATTERN).any(axis=-1)
        if bad.any():
            where = np.argwhere(bad)[0].tolist()
            where[-2] -= ROWS
            where[-1] -= self.cols
            raise AssertionError(f"{int(bad.sum())} guard elements around a {self.shape} window were written; first at (row, col) "
                                 f"relative to the window: {where}")
        return np.ascontiguousarray(raw[..., ROWS:ROWS + m, self.cols:self.cols + n])


def guarded_matmul(backend, a: Tensor, b: Tensor, batched: bool | None = None, layout: str = "window",
                   aligned: bool = True, out_dtype: DType | None = None, call=None) -> np.ndarray:
    """a . b written into a guarded output; returns the host result after the
    guard bands have been checked.  `call(view)` replaces the plain product
    (another entry point writing the same output)."""
    from oxmera_b200 import broadcast_shapes
    if batched is None:
        batched = not (len(a.shape) == 2 and len(b.shape) == 2)
    shape = tuple(broadcast_shapes(a.shape[:-2], b.shape[:-2])) + (a.shape[-2], b.shape[-1])
    g = Guarded(backend, shape, a.dtype if out_dtype is None else out_dtype, layout, aligned)  # DType.F32 is 0: no `or`
    if call is not None:
        call(g.view)
    else:
        backend.matmul_into(a, b, g.view, batched=batched)
    return g.result()
