"""fp8 (e4m3 / e5m2) products on the tensor cores and the FFMA kernel against
the oracle on identical fp8 inputs.

Tolerances: a widened output (bf16 / f16 / f32) is held to max |x-y| /
max(|y|, rms) <= 1e-2 (bf16, f16) or 1e-4 (f32) against the oracle's f32 /
f64-accumulated result — fp8 products are exact in fp32, so only the
accumulation differs.  An fp8 output is compared with the oracle's value after
its single rounding to fp8: at most one fp8 ulp apart (2^-3 relative for e4m3,
2^-2 for e5m2), and saturated rather than infinite."""
import numpy as np
import pytest

import oxmera_b200 as ox
from oxmera_b200 import DType, Tensor
from tests.oracle_lib import ACC_F64, ACC_NATIVE, F8E4M3, F8E5M2
from tests.test_gpu_parity import rel_err, set_kernel, to_f64

pytestmark = pytest.mark.gpu

TAG = {DType.F8E4M3: F8E4M3, DType.F8E5M2: F8E5M2}
ULP = {DType.F8E4M3: 2.0 ** -3, DType.F8E5M2: 2.0 ** -2}
FP8 = [DType.F8E4M3, DType.F8E5M2]


def decode(oracle, x, dtype):
    if dtype in TAG:
        return oracle.fp8_to_f32(x, TAG[dtype]).astype(np.float64)
    return to_f64(x, dtype)


@pytest.fixture(autouse=True)
def _reset(backend):
    yield
    set_kernel(backend, "auto")


@pytest.mark.parametrize("dtype", FP8, ids=lambda d: d.name)
@pytest.mark.parametrize("kernel", ["simt", "tcgen05"])
@pytest.mark.parametrize("a_t,b_t", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_fp8_products_in_wider_outputs(backend, oracle, kernel, dtype, a_t, b_t):
    set_kernel(backend, kernel)
    for m, n, k in ((256, 384, 512), (130, 70, 200), (300, 1100, 136)):
        ha = oracle.fill((k, m) if a_t else (m, k), TAG[dtype], 5, 0, "normal")
        hb = oracle.fill((n, k) if b_t else (k, n), TAG[dtype], 5, 1, "normal")
        ta, tb = Tensor.from_host(ha, ha.shape, dtype, backend), Tensor.from_host(hb, hb.shape, dtype, backend)
        if a_t:
            ha, ta = ha.T, ta.permute([1, 0])
        if b_t:
            hb, tb = hb.T, tb.permute([1, 0])
        for out_dtype, tol, acc in ((DType.BF16, 1e-2, ACC_NATIVE), (DType.F16, 1e-2, ACC_NATIVE), (DType.F32, 1e-4, ACC_F64)):
            got = backend.matmul_as(ta, tb, out_dtype)
            st, ref = oracle.matmul(ha, hb, TAG[dtype], acc=acc)
            assert st == 0
            err = rel_err(to_f64(got.to_host(), out_dtype), ref)
            assert err <= tol, (kernel, dtype.name, out_dtype.name, (m, n, k), err, backend.last_kernel())
        if kernel == "tcgen05":
            assert "_f8_" in backend.last_kernel()


@pytest.mark.parametrize("dtype", FP8, ids=lambda d: d.name)
@pytest.mark.parametrize("kernel", ["simt", "tcgen05"])
def test_fp8_output_rounds_once_and_saturates(backend, oracle, kernel, dtype):
    set_kernel(backend, kernel)
    a = oracle.fill((192, 256), TAG[dtype], 6, 0, "normal", 0.5)
    b = oracle.fill((256, 320), TAG[dtype], 6, 1, "normal", 0.5)
    got = backend.matmul(Tensor.from_host(a, a.shape, dtype, backend), Tensor.from_host(b, b.shape, dtype, backend))
    assert got.dtype == dtype
    st, ref = oracle.matmul(a, b, TAG[dtype], acc=ACC_F64)
    g = decode(oracle, got.to_host(), dtype)
    assert np.all(np.isfinite(g))
    rms = float(np.sqrt(np.mean(ref * ref)))
    assert np.max(np.abs(g - ref) / np.maximum(np.abs(ref), rms)) <= ULP[dtype]
    # products far beyond the format's range saturate to its largest finite value
    big = np.full((64, 64), 0x7e if dtype == DType.F8E4M3 else 0x7b, np.uint8)
    sat = backend.matmul(Tensor.from_host(big, big.shape, dtype, backend), Tensor.from_host(big, big.shape, dtype, backend))
    assert np.all(sat.to_host() == big[0, 0])


@pytest.mark.parametrize("dtype", FP8, ids=lambda d: d.name)
def test_fp8_batched_broadcast_and_fused(backend, oracle, dtype):
    set_kernel(backend, "tcgen05")
    a = oracle.fill((3, 1, 96, 256), TAG[dtype], 7, 0, "normal")
    b = oracle.fill((1, 2, 256, 72), TAG[dtype], 7, 1, "normal", 0.25)
    out = backend.matmul_as(Tensor.from_host(a, a.shape, dtype, backend), Tensor.from_host(b, b.shape, dtype, backend), DType.BF16)
    st, ref = oracle.matmul(a, b, TAG[dtype], acc=ACC_NATIVE)
    assert out.shape == ref.shape and rel_err(to_f64(out.to_host(), DType.BF16), ref) <= 1e-2


def test_fp8_dtype_rules(backend):
    f = lambda shape, dt: Tensor.empty(shape, dt, backend)
    with pytest.raises(ox.DTypeMismatch):
        backend.matmul(f((8, 16), DType.F8E4M3), f((16, 8), DType.F8E5M2))
    with pytest.raises(ox.DTypeMismatch):  # only fp8 products may be widened
        backend.matmul_into(f((8, 16), DType.BF16), f((16, 8), DType.BF16), f((8, 8), DType.F32), batched=False)
    with pytest.raises(ox.DTypeMismatch):  # and never narrowed to the other fp8 encoding
        backend.matmul_into(f((8, 16), DType.F8E4M3), f((16, 8), DType.F8E4M3), f((8, 8), DType.F8E5M2), batched=False)
