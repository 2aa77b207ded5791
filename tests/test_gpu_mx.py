"""The block-scaled fp8 product (oxm_matmul_mx: MXFP8, one E8M0 scale per 32
contraction elements of every row of A and column of B) against the oracle on
identical bytes.

Tolerance: the 32 products of a block are exact in fp32 and so is the power-
of-two scaling; what differs from the oracle's double sum is the fp32
accumulation across blocks and the final rounding, so a bf16 / f16 result is
held to max |x - y| / max(|y|, rms) <= 1e-2 and an f32 result to 2e-4, as for
the unscaled fp8 product.  (The random scales stop at 2^2 so that no sum leaves
f16's range.)  Cases built from powers of two are exact."""
import numpy as np
import pytest

import oxmera_b200 as ox
from oxmera_b200 import DType, Tensor
from tests.guard import guarded_matmul
from tests.oracle_lib import F8E4M3, F8E5M2
from tests.test_gpu_parity import rel_err, to_f64

pytestmark = pytest.mark.gpu

TAG = {DType.F8E4M3: F8E4M3, DType.F8E5M2: F8E5M2}
TOL = {DType.BF16: 1e-2, DType.F16: 1e-2, DType.F32: 2e-4}


@pytest.fixture(autouse=True)
def _reset(backend):
    yield
    backend.set_option("tile_n", 0)


def dev(backend, arr, dtype):
    return Tensor.from_host(np.ascontiguousarray(arr), arr.shape, dtype, backend)


def scales(rng, shape, lo=119, hi=129):  # 2^-8 .. 4: products of N(0, 1) data stay inside f16's range
    return rng.integers(lo, hi + 1, size=shape, dtype=np.uint8)


def mx(backend, a, sa, b, sb, out_dtype, aligned=True, layout="window"):
    return guarded_matmul(backend, a, b, batched=True, out_dtype=out_dtype, aligned=aligned, layout=layout,
                          call=lambda view: backend.matmul_mx_into(a, sa, b, sb, view))


def test_powers_of_two_are_exact(backend):
    """a = 1, b = 2 everywhere; the scales differ per row, per column and per
    block, so every output element says which scale bytes its MMAs took."""
    m, n, k = 256, 1000, 256  # 1000 columns: tiles start 0 and 64 columns into a scale atom, and the last one is ragged
    a = np.full((m, k), 0x38, np.uint8)   # e4m3 1.0
    bt = np.full((n, k), 0x40, np.uint8)  # e4m3 2.0
    # (a narrow range of exponents: the sum of the eight block products then fits fp32 exactly)
    sa = (124 + (np.arange(m)[:, None] * 3 + np.arange(k // 32)[None, :]) % 5).astype(np.uint8)
    sbt = (125 + (np.arange(n)[:, None] * 5 + np.arange(k // 32)[None, :] * 2) % 4).astype(np.uint8)
    want = 64.0 * (np.ldexp(1.0, sa.astype(int) - 127) @ np.ldexp(1.0, sbt.astype(int) - 127).T)
    ta, tsa = dev(backend, a, DType.F8E4M3), dev(backend, sa, DType.U8)
    tb, tsb = dev(backend, bt, DType.F8E4M3).permute([1, 0]), dev(backend, sbt, DType.U8).permute([1, 0])
    for width in (128, 192, 256, 384):  # two-accumulator tiles up to 192, one-accumulator tiles above
        backend.set_option("tile_n", width)
        got = mx(backend, ta, tsa, tb, tsb, DType.F32)
        assert "mxf8" in backend.last_kernel() and backend.last_kernel().endswith(f"_w{width}")
        bad = np.argwhere(got != want)
        assert bad.size == 0, (width, bad[:5].tolist(), got[tuple(bad[0])], want[tuple(bad[0])])


@pytest.mark.parametrize("dtype", [DType.F8E4M3, DType.F8E5M2], ids=lambda d: d.name)
@pytest.mark.parametrize("m,n,k", [(256, 256, 128), (300, 520, 384), (128, 384, 1024), (1000, 700, 160), (77, 130, 32),
                                   (512, 1024, 4096)])
def test_against_the_oracle(backend, oracle, dtype, m, n, k):
    rng = np.random.default_rng(m + n + k)
    a = oracle.fill((m, k), TAG[dtype], 21, 0, "normal")
    bt = oracle.fill((n, k), TAG[dtype], 21, 1, "normal")
    sa, sbt = scales(rng, (m, k // 32)), scales(rng, (n, k // 32))
    st, ref = oracle.matmul_mx(a, sa, bt.T, sbt.T, TAG[dtype])
    assert st == 0
    ta, tsa = dev(backend, a, dtype), dev(backend, sa, DType.U8)
    tb, tsb = dev(backend, bt, dtype).permute([1, 0]), dev(backend, sbt, DType.U8).permute([1, 0])
    for out_dtype in (DType.BF16, DType.F16, DType.F32):
        for aligned in (True, False):
            got = mx(backend, ta, tsa, tb, tsb, out_dtype, aligned=aligned)
            err = rel_err(to_f64(got, out_dtype), ref)
            assert err <= TOL[out_dtype], (dtype.name, out_dtype.name, (m, n, k), aligned, err, backend.last_kernel())
    assert "mxf8" in backend.last_kernel()


def test_operands_and_scales_through_any_view(backend, oracle):
    """Row-major B (contraction dim not contiguous) and a transposed A are
    packed on the device; scale views are read through their strides."""
    dtype, tag = DType.F8E4M3, F8E4M3
    m, n, k = 200, 330, 256
    rng = np.random.default_rng(5)
    at = oracle.fill((k, m), tag, 22, 0, "normal")       # A stored transposed
    b = oracle.fill((k, n), tag, 22, 1, "normal")        # B row-major
    sat = scales(rng, (k // 32, m))                      # A's scales stored transposed
    sb_wide = scales(rng, (k // 32, n + 7))              # B's scales: a window of a wider array
    sb = np.ascontiguousarray(sb_wide[:, 3:3 + n])
    st, ref = oracle.matmul_mx(at.T, sat.T, b, sb, tag)
    assert st == 0
    ta, tsa = dev(backend, at, dtype).permute([1, 0]), dev(backend, sat, DType.U8).permute([1, 0])
    tsb = dev(backend, sb_wide, DType.U8).narrow(1, 3, n)
    tb = dev(backend, b, dtype)
    got = mx(backend, ta, tsa, tb, tsb, DType.F32)
    assert rel_err(got, ref) <= TOL[DType.F32], backend.last_kernel()


def test_batched_and_broadcast(backend, oracle):
    dtype, tag = DType.F8E4M3, F8E4M3
    rng = np.random.default_rng(9)
    a = oracle.fill((3, 1, 130, 128), tag, 23, 0, "normal")
    bt = oracle.fill((2, 260, 128), tag, 23, 1, "normal")
    sa, sbt = scales(rng, (3, 1, 130, 4)), scales(rng, (2, 260, 4))
    st, ref = oracle.matmul_mx(a, sa, np.swapaxes(bt, -1, -2), np.swapaxes(sbt, -1, -2), tag)
    assert st == 0 and ref.shape == (3, 2, 130, 260)
    ta, tsa = dev(backend, a, dtype), dev(backend, sa, DType.U8)
    tb, tsb = dev(backend, bt, dtype).permute([0, 2, 1]), dev(backend, sbt, DType.U8).permute([0, 2, 1])
    got = mx(backend, ta, tsa, tb, tsb, DType.BF16)
    assert rel_err(to_f64(got, DType.BF16), ref) <= TOL[DType.BF16]
    fresh = backend.matmul_mx(ta, tsa, tb, tsb, DType.F32)
    assert fresh.shape == (3, 2, 130, 260) and fresh.layout().is_contiguous()
    assert rel_err(fresh.to_host(), ref) <= TOL[DType.F32]


@pytest.mark.parametrize("dtype", [DType.F8E4M3, DType.F8E5M2], ids=lambda d: d.name)
def test_fp8_output_rounds_once(backend, oracle, dtype):
    """The product kept in the operands' own 8-bit type: one rounding of the
    fp32 sum, at most one fp8 ulp from the oracle's value, saturated rather
    than infinite."""
    m, n, k = 200, 300, 256
    rng = np.random.default_rng(17)
    a = oracle.fill((m, k), TAG[dtype], 24, 0, "normal", 0.5)
    bt = oracle.fill((n, k), TAG[dtype], 24, 1, "normal", 0.5)
    sa, sbt = scales(rng, (m, k // 32), 124, 128), scales(rng, (n, k // 32), 124, 128)
    st, ref = oracle.matmul_mx(a, sa, bt.T, sbt.T, TAG[dtype])
    assert st == 0
    got = mx(backend, dev(backend, a, dtype), dev(backend, sa, DType.U8), dev(backend, bt, dtype).permute([1, 0]),
             dev(backend, sbt, DType.U8).permute([1, 0]), dtype)
    g = oracle.fp8_to_f32(got, TAG[dtype]).astype(np.float64)
    assert np.all(np.isfinite(g))
    big = 448.0 if dtype == DType.F8E4M3 else 57344.0
    rms = float(np.sqrt(np.mean(ref * ref)))
    ulp = 2.0 ** -3 if dtype == DType.F8E4M3 else 2.0 ** -2
    assert np.max(np.abs(g - np.clip(ref, -big, big)) / np.maximum(np.abs(ref), rms)) <= ulp


def test_nan_scale_poisons_its_row_only(backend):
    m, n, k = 128, 256, 64
    a = np.full((m, k), 0x38, np.uint8)
    bt = np.full((n, k), 0x38, np.uint8)
    sa = np.full((m, 2), 127, np.uint8)
    sa[5, 1] = 255
    sbt = np.full((n, 2), 127, np.uint8)
    got = backend.matmul_mx(dev(backend, a, DType.F8E4M3), dev(backend, sa, DType.U8),
                            dev(backend, bt, DType.F8E4M3).permute([1, 0]), dev(backend, sbt, DType.U8).permute([1, 0]),
                            DType.F32).to_host()
    assert np.all(np.isnan(got[5])) and np.all(np.delete(got, 5, axis=0) == 64.0)


def test_refusals(backend):
    f8, u8 = DType.F8E4M3, DType.U8
    z = lambda shape, dt: Tensor.empty(shape, dt, backend)
    with pytest.raises(ox.ShapeMismatch):   # K = 48
        backend.matmul_mx(z((4, 48), f8), z((4, 1), u8), z((48, 4), f8), z((1, 4), u8))
    with pytest.raises(ox.ShapeMismatch):   # scale shape
        backend.matmul_mx(z((4, 64), f8), z((4, 3), u8), z((64, 4), f8), z((2, 4), u8))
    with pytest.raises(ox.DTypeMismatch):   # scales are bytes
        backend.matmul_mx(z((4, 64), f8), z((4, 2), DType.F32), z((64, 4), f8), z((2, 4), u8))
    with pytest.raises(ox.UnsupportedDType):
        backend.matmul_mx(z((4, 64), DType.BF16), z((4, 2), u8), z((64, 4), DType.BF16), z((2, 4), u8))
    # an empty product and an empty contraction
    assert backend.matmul_mx(z((0, 64), f8), z((0, 2), u8), z((64, 4), f8), z((2, 4), u8)).shape == (0, 4)
    out = backend.matmul_mx(z((4, 0), f8), z((4, 0), u8), z((0, 4), f8), z((0, 4), u8), DType.F32)
    assert np.all(out.to_host() == 0)
