"""Seeded random products through the C ABI against the oracle: random
extents (tile tails in M, N and K), random operand majors, windows with odd
offsets, flips, broadcast batch dims, tile widths of every kernel instance
and both kernels, each output inside guard bands that must stay untouched.
The cases are drawn from a fixed seed, so a failure names a reproducible
case index."""
import numpy as np
import pytest

from oxmera_b200 import DType, Tensor
from tests.guard import guarded_matmul
from tests.test_gpu_parity import TOL, fill, oracle_ref, rel_err, set_kernel, to_f64

pytestmark = pytest.mark.gpu


def _view(rng, h, t):
    """A random view of the last two dims, applied alike to the host array and the device tensor."""
    nd = h.ndim
    if rng.random() < 0.5:  # transpose the matrix dims
        perm = list(range(nd - 2)) + [nd - 1, nd - 2]
        h, t = h.transpose(perm), t.permute(perm)
    for d in (nd - 2, nd - 1):
        if h.shape[d] > 4 and rng.random() < 0.4:  # a window with an odd offset
            off = int(rng.integers(1, 4))
            ln = h.shape[d] - off - int(rng.integers(0, 3))
            sl = [slice(None)] * nd
            sl[d] = slice(off, off + ln)
            h, t = h[tuple(sl)], t.narrow(d, off, ln)
        if rng.random() < 0.15:  # a negative stride
            sl = [slice(None)] * nd
            sl[d] = slice(None, None, -1)
            h, t = h[tuple(sl)], t.flip(d)
    return h, t


@pytest.mark.parametrize("dtype", [DType.BF16, DType.F16, DType.F32], ids=lambda d: d.name)
def test_random_products(backend, oracle, dtype):
    rng = np.random.default_rng({DType.BF16: 11, DType.F16: 12, DType.F32: 13}[dtype])
    extents = [1, 2, 7, 8, 16, 31, 64, 65, 100, 127, 128, 129, 200, 256, 257, 300, 520]
    for case in range(40):
        m, n, k = (int(rng.choice(extents)) for _ in range(3))
        batch = [(), (), (3,), (2, 1), (1, 4)][int(rng.integers(0, 5))]
        b_batch = batch if rng.random() < 0.5 else tuple(1 for _ in batch)
        # build base tensors big enough for the windows, in the orientation that gives [.., m, k] x [.., k, n] after _view
        ha = fill(oracle, batch + (m + 6, k + 6), dtype, 500 + case, 0)
        hb = fill(oracle, b_batch + (k + 6, n + 6), dtype, 500 + case, 1)
        ta, tb = Tensor.from_host(ha, ha.shape, dtype, backend), Tensor.from_host(hb, hb.shape, dtype, backend)
        va, vta = _view(rng, ha, ta)
        vb, vtb = _view(rng, hb, tb)
        # trim both to a common contraction length
        kk = min(va.shape[-1], vb.shape[-2])
        va, vta = va[..., :kk], vta.narrow(va.ndim - 1, 0, kk)
        vb, vtb = vb[..., :kk, :], vtb.narrow(vb.ndim - 2, 0, kk)
        kernel = ["auto", "simt", "tcgen05", "tcgen05"][int(rng.integers(0, 4))]
        tile_n = int(rng.choice([0, 64, 96, 128, 192, 256, 320, 480, 512])) if kernel == "tcgen05" else 0
        set_kernel(backend, kernel, tile_n=tile_n)
        backend.set_option("split_k", int(rng.choice([-1, 0, 2])) if kernel == "tcgen05" and dtype != DType.F32 else -1)
        # every output sits inside guard bands; the layout (fresh contiguous, aligned or odd window) rotates
        layout, aligned = [("flat", True), ("window", True), ("window", False), ("flat", False)][case % 4]
        got = guarded_matmul(backend, vta, vtb, batched=bool(batch), layout=layout, aligned=aligned)
        ref = oracle_ref(oracle, va, vb, dtype)
        assert got.shape == ref.shape, (case, got.shape, ref.shape)
        err = rel_err(to_f64(got, dtype), ref)
        assert err <= TOL[dtype], (case, va.shape, vb.shape, kernel, tile_n, err, backend.last_kernel())
