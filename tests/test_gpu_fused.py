"""The fused epilogue (bias, activation, accumulate) against the oracle's
restatement of the same arithmetic, on every kernel that can finish a product:
the FFMA kernel, the tensor-core kernel with either store path, and the
split-K reduction."""
import numpy as np
import pytest

import oxmera_b200 as ox
from oxmera_b200 import DType, Tensor
from tests.oracle_lib import ACC_F64, ACC_NATIVE
from tests.test_gpu_parity import TAG, TOL, fill, rel_err, set_kernel, to_f64

pytestmark = pytest.mark.gpu

ACT = {"none": 0, "relu": 1, "gelu": 2}
ROUTES = {  # name -> (kernel, split_k, tma_store)
    "ffma": ("simt", -1, 1),
    "tensor": ("tcgen05", 0, 1),
    "tensor-strided-store": ("tcgen05", 0, 0),
    "tensor-split-k": ("tcgen05", 4, 1),
}


@pytest.fixture(autouse=True)
def _reset(backend):
    yield
    set_kernel(backend, "auto")
    backend.set_option("tma_store", 1)


def route(backend, name):
    kernel, split, tma = ROUTES[name]
    set_kernel(backend, kernel)
    backend.set_option("split_k", split)
    backend.set_option("tma_store", tma)


def reference(oracle, a, b, dtype, bias, act, prev):
    acc = ACC_F64 if dtype == DType.F32 else ACC_NATIVE
    prev_f = None if prev is None else to_f64(prev, dtype)
    st, ref = oracle.matmul_fused(a, b, TAG[dtype], bias=bias, act=ACT[act], prev=prev_f, acc=acc)
    assert st == 0
    return ref


@pytest.mark.parametrize("dtype", [DType.F32, DType.BF16, DType.F16], ids=lambda d: d.name)
@pytest.mark.parametrize("name", list(ROUTES))
def test_linear_forward_bias_activation(backend, oracle, name, dtype):
    """Y = act(X . W^T + b): W is a transposed view, the bias a rank-1 tensor."""
    route(backend, name)
    for act in ("none", "relu", "gelu"):
        x = fill(oracle, (200, 2048), dtype, 61, 0, scale=1.0)
        w = fill(oracle, (136, 2048), dtype, 61, 1, scale=0.03)
        bias = fill(oracle, (136,), dtype, 61, 2, scale=0.5)
        tx = Tensor.from_host(x, x.shape, dtype, backend)
        tw = Tensor.from_host(w, w.shape, dtype, backend).permute([1, 0])
        tb = Tensor.from_host(bias, bias.shape, dtype, backend)
        got = backend.matmul_fused(tx, tw, bias=tb, activation=act)
        ref = reference(oracle, x, w.T, dtype, bias, act, None)
        err = rel_err(to_f64(got.to_host(), dtype), ref)
        assert err <= TOL[dtype], (name, act, err, backend.last_kernel())


@pytest.mark.parametrize("dtype", [DType.F32, DType.BF16], ids=lambda d: d.name)
@pytest.mark.parametrize("name", list(ROUTES))
def test_gradient_accumulation(backend, oracle, name, dtype):
    """dW += dY^T . X over two micro-batches: both transposes are views and the
    running sum lives in the output tensor."""
    route(backend, name)
    dw_host = fill(oracle, (160, 264), dtype, 71, 9, scale=0.5)  # what dW held before
    dw = Tensor.from_host(dw_host.copy(), dw_host.shape, dtype, backend)
    expect = to_f64(dw_host, dtype)
    for step in range(2):
        dy = fill(oracle, (2048, 160), dtype, 71 + step, 0, scale=0.05)
        x = fill(oracle, (2048, 264), dtype, 71 + step, 1)
        tdy = Tensor.from_host(dy, dy.shape, dtype, backend).permute([1, 0])
        tx = Tensor.from_host(x, x.shape, dtype, backend)
        prev = dw.to_host()
        backend.matmul_fused(tdy, tx, accumulate_into=dw)
        ref = reference(oracle, dy.T, x, dtype, None, "none", prev)
        err = rel_err(to_f64(dw.to_host(), dtype), ref)
        assert err <= TOL[dtype], (name, step, err, backend.last_kernel())
    assert not np.array_equal(to_f64(dw.to_host(), dtype), expect)


def test_batched_bias_and_accumulate_together(backend, oracle):
    set_kernel(backend, "tcgen05")
    dtype = DType.BF16
    a = fill(oracle, (3, 1, 96, 200), dtype, 81, 0)
    b = fill(oracle, (1, 2, 200, 72), dtype, 81, 1, scale=0.1)
    bias = fill(oracle, (72,), dtype, 81, 2)
    prev = fill(oracle, (3, 2, 96, 72), dtype, 81, 3)
    out = Tensor.from_host(prev.copy(), prev.shape, dtype, backend)
    backend.matmul_fused(Tensor.from_host(a, a.shape, dtype, backend), Tensor.from_host(b, b.shape, dtype, backend),
                         bias=Tensor.from_host(bias, bias.shape, dtype, backend), activation="relu", accumulate_into=out)
    ref = reference(oracle, a, b, dtype, bias, "relu", prev)
    assert rel_err(to_f64(out.to_host(), dtype), ref) <= TOL[dtype]


def test_fused_argument_errors(backend):
    f = lambda shape, dt=DType.BF16: Tensor.empty(shape, dt, backend)
    with pytest.raises(ox.ShapeMismatch) as e:
        backend.matmul_fused(f((4, 8)), f((8, 6)), bias=f((5,)))
    assert "bias" in str(e.value)
    with pytest.raises(ox.ShapeMismatch):
        backend.matmul_fused(f((4, 8)), f((8, 6)), bias=f((1, 6)))  # rank-1 only
    with pytest.raises(ox.DTypeMismatch):
        backend.matmul_fused(f((4, 8)), f((8, 6)), bias=f((6,), DType.F32))
    with pytest.raises(ox.ShapeMismatch):
        backend.matmul_fused(f((4, 8)), f((8, 6)), accumulate_into=f((4, 5)))
    backend.synchronize()
