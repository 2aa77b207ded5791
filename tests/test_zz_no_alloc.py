"""The allocation-free f32 matmul entry point, through the C ABI, on a B200.

oxm_matmul_f32_noalloc serves hosts that must not allocate device memory once
they are running (all of HBM already belongs to their own arena, or an
allocator call's synchronisation and failure modes are unacceptable on their
hot loop).  Its scratch is a fixed array inside the library's device image
that every call shares and that keeps whatever the previous call left in it,
so the check that matters is several calls in a row, of different sizes, each
compared with the ordinary entry point on the same inputs.

Collected last on purpose: a run that stops at the first failure has already
run every other test.  It passes alone in a fresh process as well.
"""
import ctypes as C

import numpy as np
import pytest

import oxmera_b200 as ox
from oxmera_b200 import DType, Tensor, capi
from tests.guard import guarded_matmul
from tests.oracle_lib import ACC_F64, F32

pytestmark = pytest.mark.gpu

TOL = 1e-4  # the f32 tolerance of the parity tests: max |x-y| / max(|y|, rms(Y))


def rel_err(got, ref):
    ref, got = ref.astype(np.float64), got.astype(np.float64)
    rms = float(np.sqrt(np.mean(ref * ref)))
    return float(np.max(np.abs(got - ref) / np.maximum(np.abs(ref), rms)))


def noalloc_into(backend, a: Tensor, b: Tensor, out: Tensor) -> None:
    st = capi.load().oxm_matmul_f32_noalloc(backend._ctx, C.byref(a._view()), C.byref(b._view()), C.byref(out._view()))
    assert st == capi.OK, capi.last_error()


def noalloc(backend, a: Tensor, b: Tensor) -> Tensor:
    out = Tensor.empty((a.shape[0], b.shape[1]), DType.F32, backend)
    noalloc_into(backend, a, b, out)
    return out


def test_back_to_back_calls_match_the_ordinary_entry_point(backend, oracle):
    # Sizes shrink, grow and cross the split-K threshold, so every call finds
    # the previous call's packed operands and partial sums in the scratch.
    cases = [(300, 260, 200), (70, 50, 40), (64, 96, 2100), (129, 257, 65), (300, 260, 200)]
    for i, (m, n, k) in enumerate(cases):
        ha = oracle.fill((m, k), F32, 200 + i, 0, "normal")
        hb = oracle.fill((n, k), F32, 200 + i, 1, "normal")  # B is handed over as a transposed view
        ta = Tensor.from_host(ha, ha.shape, DType.F32, backend)
        tb = Tensor.from_host(hb, hb.shape, DType.F32, backend).permute([1, 0])
        before = backend.launch_counts()
        # the output sits inside guard bands: the entry point writes its result and nothing around it
        got = guarded_matmul(backend, ta, tb, layout="flat" if i % 2 else "window", aligned=i != 3,
                             call=lambda view: noalloc_into(backend, ta, tb, view))
        after = backend.launch_counts()
        assert after["tcgen05"] == before["tcgen05"] + 1
        assert "tf32x3" in backend.last_kernel()
        backend.set_option("kernel", 2)  # the ordinary entry point on the same tensor-core path
        same_path = backend.matmul(ta, tb).to_host()
        backend.set_option("kernel", 0)  # and as a caller would get it by default
        default = backend.matmul(ta, tb).to_host()
        assert rel_err(got, same_path) <= TOL, (m, n, k)
        assert rel_err(got, default) <= TOL, (m, n, k)
        _, ref = oracle.matmul(ha, hb.T, F32, acc=ACC_F64)
        assert rel_err(got, ref) <= TOL, (m, n, k)


def test_warm_calls_allocate_nothing(oracle):
    """The property the entry point exists for.  On a context of its own that
    makes no other call, after one warm-up call (which looks the scratch
    array's address up), calls of several sizes - one of them with split-K
    partial sums - leave the device's memory pool and its free memory exactly
    as they found them."""
    be = ox.B200Backend(0)
    try:
        cases = [(300, 260, 200), (64, 96, 2100), (129, 257, 65), (520, 130, 900)]
        work = []
        for i, (m, n, k) in enumerate(cases):  # every allocation of the test happens here, before the measurement
            ha = oracle.fill((m, k), F32, 300 + i, 0, "normal")
            hb = oracle.fill((k, n), F32, 300 + i, 1, "normal")
            work.append((ha, hb, Tensor.from_host(ha, ha.shape, DType.F32, be), Tensor.from_host(hb, hb.shape, DType.F32, be),
                         Tensor.empty((m, n), DType.F32, be)))
        noalloc_into(be, work[0][2], work[0][3], work[0][4])  # warm-up: resolves the symbol, loads the kernels
        noalloc_into(be, work[1][2], work[1][3], work[1][4])
        be.synchronize()
        before = be.memory_stats()
        for _ in range(2):
            for _, _, ta, tb, out in work:
                noalloc_into(be, ta, tb, out)
        be.synchronize()
        after = be.memory_stats()
        assert after["pool_reserved"] == before["pool_reserved"], (before, after)
        assert after["pool_used"] == before["pool_used"], (before, after)
        assert after["device_free"] == before["device_free"], (before, after)
        # the ordinary entry point, for contrast, takes its workspaces from the pool
        be.set_option("kernel", 2)
        be.matmul(work[3][2], work[3][3])
        be.synchronize()
        assert be.memory_stats()["pool_used"] > after["pool_used"]
        for ha, hb, _, _, out in work:
            _, ref = oracle.matmul(ha, hb, F32, acc=ACC_F64)
            assert rel_err(out.to_host(), ref) <= TOL
    finally:
        be.close()


def test_infinities_and_nans_follow_ieee(backend):
    """An infinity or NaN in an operand reaches exactly the outputs IEEE
    arithmetic gives (inf * 2 = inf, inf * 0 = NaN, inf - inf = NaN): the
    tensor-core path packs such a value so that it meets its partner once."""
    rng = np.random.default_rng(7)
    a = rng.integers(-3, 4, size=(70, 96)).astype(np.float32)   # small integers: several exact zeros, exact in tf32
    b = rng.integers(-3, 4, size=(96, 50)).astype(np.float32)
    a[3, 10], a[5, 20], a[9, 30] = np.inf, -np.inf, np.nan
    b[40, 7], b[41, 8] = np.inf, np.nan
    a[11, 40] = np.inf  # meets b[40, 7] = inf in output (11, 7): inf * inf = inf
    with np.errstate(invalid="ignore"):
        ref = a.astype(np.float64) @ b.astype(np.float64)
    ta, tb = Tensor.from_host(a, a.shape, DType.F32, backend), Tensor.from_host(b, b.shape, DType.F32, backend)
    got = noalloc(backend, ta, tb).to_host()
    backend.set_option("kernel", 1)
    ffma = backend.matmul(ta, tb).to_host()
    backend.set_option("kernel", 0)
    for name, x in (("noalloc", got), ("ffma", ffma)):
        assert np.array_equal(np.isnan(x), np.isnan(ref)), name
        assert np.array_equal(np.isposinf(x), np.isposinf(ref)) and np.array_equal(np.isneginf(x), np.isneginf(ref)), name
        fin = np.isfinite(ref)
        assert np.array_equal(x[fin], ref[fin].astype(np.float32)), name  # small integers: exact


def test_hand_case_and_empty_contraction(backend):
    a = Tensor.from_host(np.array([1, 2, 3, 4], np.float32), (2, 2), DType.F32, backend)
    b = Tensor.from_host(np.array([5, 6, 7, 8], np.float32), (2, 2), DType.F32, backend)
    assert noalloc(backend, a, b).to_host().reshape(-1).tolist() == [19.0, 22.0, 43.0, 50.0]
    e = noalloc(backend, Tensor.from_host(np.ones((2, 0), np.float32), (2, 0), DType.F32, backend),
                Tensor.from_host(np.ones((0, 3), np.float32), (0, 3), DType.F32, backend))
    assert e.shape == (2, 3) and not e.to_host().any()


def test_sizes_beyond_the_scratch_are_refused_with_both_numbers(backend):
    lib = capi.load()
    big = Tensor.empty((4096, 4096), DType.F32, backend)
    out = Tensor.empty((4096, 4096), DType.F32, backend)
    st = lib.oxm_matmul_f32_noalloc(backend._ctx, C.byref(big._view()), C.byref(big._view()), C.byref(out._view()))
    assert st == capi.NOT_IMPLEMENTED
    msg = capi.last_error()
    assert "671088640" in msg and str(32 << 20) in msg, msg  # 2 x 192 MiB packed + 4 x 64 MiB partial sums
    half = Tensor.empty((8, 8), DType.BF16, backend)
    st = lib.oxm_matmul_f32_noalloc(backend._ctx, C.byref(half._view()), C.byref(half._view()), C.byref(half._view()))
    assert st == capi.UNSUPPORTED_DTYPE
    wrong = Tensor.empty((3, 5), DType.F32, backend)
    st = lib.oxm_matmul_f32_noalloc(backend._ctx, C.byref(wrong._view()), C.byref(wrong._view()), C.byref(wrong._view()))
    assert st == capi.SHAPE_MISMATCH
    backend.synchronize()  # the context is still healthy
