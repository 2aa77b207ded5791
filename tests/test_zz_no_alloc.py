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
from tests.oracle_lib import ACC_F64, F32

pytestmark = pytest.mark.gpu

TOL = 1e-4  # the f32 tolerance of the parity tests: max |x-y| / max(|y|, rms(Y))


def rel_err(got, ref):
    ref, got = ref.astype(np.float64), got.astype(np.float64)
    rms = float(np.sqrt(np.mean(ref * ref)))
    return float(np.max(np.abs(got - ref) / np.maximum(np.abs(ref), rms)))


def noalloc(backend, a: Tensor, b: Tensor) -> Tensor:
    out = Tensor.empty((a.shape[0], b.shape[1]), DType.F32, backend)
    st = capi.load().oxm_matmul_f32_noalloc(backend._ctx, C.byref(a._view()), C.byref(b._view()), C.byref(out._view()))
    assert st == capi.OK, capi.last_error()
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
        got = noalloc(backend, ta, tb).to_host()
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
