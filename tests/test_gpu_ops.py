"""UnaryOps, BinaryOps and ReduceOps on the device against the oracle's loops,
through the C ABI: every dtype, strided / transposed / flipped / broadcast
views, every reduction geometry.

Tolerances: results of one arithmetic operation must match the oracle's
correctly rounded value to 2 ulp of the dtype (device exp / log are not
correctly rounded); sums are compared as max |x-y| / max(|y|, rms) against the
f64-accumulated oracle with 1e-5 (f32), 1e-12 (f64), 1e-2 (bf16 / f16);
integer results and max are exact."""
import numpy as np
import pytest

import oxmera_b200 as ox
from oxmera_b200 import DType, Tensor
from tests.oracle_lib import BF16, F16, F32, F64, I32, I64
from tests.test_gpu_parity import rel_err

pytestmark = pytest.mark.gpu

TAGS = {DType.F32: F32, DType.F64: F64, DType.BF16: BF16, DType.F16: F16, DType.I32: I32, DType.I64: I64}
NPDT = {DType.F32: np.float32, DType.F64: np.float64, DType.F16: np.float16, DType.I32: np.int32, DType.I64: np.int64}
EPS = {DType.F32: 2.0 ** -23, DType.F64: 2.0 ** -52, DType.BF16: 2.0 ** -7, DType.F16: 2.0 ** -10}
FLOATS = [DType.F32, DType.F64, DType.BF16, DType.F16]
INTS = [DType.I32, DType.I64]


def host(oracle, shape, dtype, seed, positive=False):
    if dtype in INTS:
        n = int(np.prod(shape)) if len(shape) else 1
        return ((np.arange(n, dtype=np.int64) * 7919 + seed) % 201 - 100).astype(NPDT[dtype]).reshape(shape)
    if dtype == DType.F64:
        x = oracle.fill(shape, F32, seed, 0, "normal").astype(np.float64)
    else:
        x = oracle.fill(shape, TAGS[dtype], seed, 0, "normal")
    if positive:
        x = np.abs(as_f64(x, dtype)) + 0.25
        x = ox.f32_to_bf16_bits(x.astype(np.float32)).reshape(shape) if dtype == DType.BF16 else x.astype(NPDT[dtype])
    return x


def as_f64(x, dtype):
    if dtype == DType.BF16:
        return ox.bf16_bits_to_f32(x).reshape(x.shape).astype(np.float64)
    return x.astype(np.float64)


def assert_close(got, ref, dtype, ulps=2):
    if dtype in INTS:
        assert np.array_equal(got, ref)
        return
    g, r = as_f64(got, dtype), as_f64(ref, dtype)
    assert g.shape == r.shape
    assert np.all(np.abs(g - r) <= ulps * EPS[dtype] * np.maximum(np.abs(r), 1e-30) + 1e-300), float(np.max(np.abs(g - r)))


def views(h, t):
    """The same views on the host array and the device tensor."""
    yield h, t
    if h.ndim >= 2:
        perm = list(range(h.ndim))[::-1]
        yield h.transpose(perm), t.permute(perm)
        yield h[::-1], t.flip(0)
        yield h[:, 1:], t.narrow(1, 1, h.shape[1] - 1)


@pytest.mark.parametrize("dtype", FLOATS + INTS, ids=lambda d: d.name)
def test_unary_ops(backend, oracle, dtype):
    ops = [(0, backend.neg, False), (3, backend.abs, False)]
    if dtype in FLOATS:
        ops += [(1, backend.exp, False), (2, backend.ln, True)]
    for op, fn, positive in ops:
        h = host(oracle, (37, 5, 19), dtype, 10 + op, positive)
        t = Tensor.from_host(h, h.shape, dtype, backend)
        for hv, tv in views(h, t):
            out = fn(tv)
            assert out.shape == hv.shape and out.layout().is_contiguous()
            st, ref = oracle.unary(op, hv, TAGS[dtype])
            assert st == 0
            assert_close(out.to_host(), ref, dtype)
    if dtype in INTS:
        with pytest.raises(ox.UnsupportedDType):
            backend.exp(Tensor.from_host(host(oracle, (4,), dtype, 1), (4,), dtype, backend))


@pytest.mark.parametrize("dtype", FLOATS + INTS, ids=lambda d: d.name)
def test_binary_ops_broadcast(backend, oracle, dtype):
    fns = [backend.add, backend.sub, backend.mul, backend.div]  # the integer test data has no zero divisors: see below
    cases = [((64, 33), (64, 33)), ((2, 3), (3,)), ((2, 1), (1, 3)), ((), (2, 3)), ((4, 1, 5), (3, 1)), ((130, 1, 17), (1, 9, 1)),
             ((2, 0), (1, 1)),
             # long innermost dims: a CTA per row (a bias row, a per-row scalar, an extent that keeps rows off
             # 16-byte boundaries, more rows than CTAs)
             ((300, 136), (136,)), ((300, 136), (300, 1)), ((300, 131), (131,)), ((9600, 136), (136,)), ((9600, 1), (9600, 136))]
    for ls, rs in cases:
        a, b = host(oracle, ls, dtype, 20), host(oracle, rs, dtype, 21, positive=dtype in FLOATS)
        if dtype in INTS:
            b = np.where(b == 0, 7, b).astype(b.dtype)
        ta, tb = Tensor.from_host(a, ls, dtype, backend), Tensor.from_host(b, rs, dtype, backend)
        for op, fn in enumerate(fns):
            out = fn(ta, tb)
            st, ref = oracle.binary(op, a, b, TAGS[dtype])
            assert st == 0 and out.shape == ref.shape
            assert_close(out.to_host(), ref, dtype, ulps=1)
    # views on both sides, through the tensor surface (TensorOps)
    a, b = host(oracle, (24, 40), dtype, 22), host(oracle, (40, 24), dtype, 23)
    ta, tb = Tensor.from_host(a, a.shape, dtype, backend), Tensor.from_host(b, b.shape, dtype, backend)
    got = ta.add(tb.permute([1, 0]).flip(0))
    assert_close(got.to_host(), oracle.binary(0, a, b.T[::-1], TAGS[dtype])[1], dtype, ulps=1)


@pytest.mark.parametrize("dtype", INTS, ids=lambda d: d.name)
def test_integer_division_by_zero_is_a_typed_error(backend, oracle, dtype):
    """BinaryOps::div (crates/oxmera-ops/src/lib.rs:47-49): truncating division;
    a zero divisor anywhere surfaces as DivisionByZero from the call itself, on
    a healthy kernel, and the context keeps working."""
    npdt = NPDT[dtype]
    a = np.array([[7, -7, 9, -9], [0, 100, -100, 5]], npdt)
    b = np.array([2, -2, 4, 3], npdt)
    ta, tb = Tensor.from_host(a, a.shape, dtype, backend), Tensor.from_host(b, b.shape, dtype, backend)
    assert backend.div(ta, tb).to_host().tolist() == [[3, 3, 2, -3], [0, -50, -25, 1]]
    lo = np.iinfo(npdt).min
    edge = Tensor.from_host(np.array([lo, lo + 1], npdt), (2,), dtype, backend)
    minus = Tensor.from_host(np.array([-1, -1], npdt), (2,), dtype, backend)
    assert backend.div(edge, minus).to_host().tolist() == oracle.binary(3, np.array([lo, lo + 1], npdt), np.array([-1, -1], npdt), TAGS[dtype])[1].tolist()
    # a large, strided, broadcast case against the oracle, then the same with one zero planted
    h = host(oracle, (300, 70), dtype, 50)
    d = np.where(host(oracle, (70,), dtype, 51) == 0, 3, host(oracle, (70,), dtype, 51)).astype(npdt)
    th, td = Tensor.from_host(h, h.shape, dtype, backend), Tensor.from_host(d, d.shape, dtype, backend)
    st, ref = oracle.binary(3, h.T[:, ::-1], d[:, None], TAGS[dtype])
    assert st == 0
    assert np.array_equal(backend.div(th.permute([1, 0]).flip(1), td.reshape((70, 1))).to_host(), ref)
    d[41] = 0
    tz = Tensor.from_host(d, d.shape, dtype, backend)
    assert oracle.binary(3, h, d, TAGS[dtype])[0] == 13
    with pytest.raises(ox.DivisionByZero) as e:
        backend.div(th, tz)
    assert "div" in str(e.value)
    backend.synchronize()  # the error was consumed by the failing call; nothing is left pending
    assert backend.div(ta, tb).to_host().tolist() == [[3, 3, 2, -3], [0, -50, -25, 1]]


def test_float_division_follows_ieee(backend):
    a = Tensor.from_host(np.array([1.0, -1.0, 0.0, 6.0], np.float32), (4,), DType.F32, backend)
    z = Tensor.from_host(np.array([0.0, 0.0, 0.0, 3.0], np.float32), (4,), DType.F32, backend)
    got = backend.div(a, z).to_host()
    assert np.isposinf(got[0]) and np.isneginf(got[1]) and np.isnan(got[2]) and got[3] == 2.0


def test_binary_errors(backend):
    f = lambda shape, dt=DType.F32: Tensor.empty(shape, dt, backend)
    with pytest.raises(ox.BroadcastIncompatible):
        backend.add(f((2, 3)), f((2, 4)))
    with pytest.raises(ox.DTypeMismatch):
        backend.mul(f((2, 3)), f((2, 3), DType.F64))
    with pytest.raises(ox.UnsupportedDType):
        backend.add(f((2, 3), DType.U8), f((2, 3), DType.U8))


@pytest.mark.parametrize("dtype", FLOATS + INTS, ids=lambda d: d.name)
def test_reductions(backend, oracle, dtype):
    tol = {DType.F32: 1e-5, DType.F64: 1e-12, DType.BF16: 1e-2, DType.F16: 1e-2}
    shapes = [((6, 7, 50), [[], [0], [2], [0, 2], [1], [0, 1, 2], [1, 2]]),
              ((3, 70000), [[1], [0], []]),       # a long row: one CTA per output
              ((300, 4, 200), [[0], [1], [0, 1]])]  # many outputs over kept inner dims: one thread per output
    for shape, axes_list in shapes:
        h = host(oracle, shape, dtype, 30)
        t = Tensor.from_host(h, shape, dtype, backend)
        pairs = [(h, t)]
        if len(shape) == 3:
            pairs.append((h.transpose(2, 0, 1), t.permute([2, 0, 1])))
        for hv, tv in pairs:
            for axes in axes_list:
                for op, fn in ((0, backend.sum), (1, backend.max)):
                    out = fn(tv, axes)
                    st, ref = oracle.reduce(op, hv, axes, TAGS[dtype])
                    assert st == 0 and out.shape == ref.shape
                    if dtype in INTS or op == 1:
                        assert np.array_equal(out.to_host(), ref), (shape, axes, op)
                    else:
                        exact = as_f64(hv, dtype).sum(axis=tuple(axes) if axes else None)
                        assert rel_err(as_f64(out.to_host(), dtype), np.asarray(exact)) <= tol[dtype], (shape, axes)
    # many short contiguous rows: one warp per row, row starts at every alignment (37 and 36 elements per
    # row), and a sum over everything in enough slices for the CTA-per-output last step
    h = host(oracle, (9600, 37), dtype, 32)
    t = Tensor.from_host(h, (9600, 37), dtype, backend)
    for hv, tv, kernel in ((h, t, "roww_x1"), (h[:, 1:], t.narrow(1, 1, 36), "roww_x1"), (h[::-1], t.flip(0), "roww_x1")):
        for op, fn in ((0, backend.sum), (1, backend.max)):
            out = fn(tv, [1])
            assert backend.last_kernel().endswith(kernel), backend.last_kernel()
            st, ref = oracle.reduce(op, hv, [1], TAGS[dtype])
            assert st == 0 and out.shape == ref.shape
            if dtype in INTS or op == 1:
                assert np.array_equal(out.to_host(), ref), (kernel, op)
            else:
                assert rel_err(as_f64(out.to_host(), dtype), as_f64(hv, dtype).sum(axis=1)) <= tol[dtype]
    h = host(oracle, (2, 600000), dtype, 33)
    t = Tensor.from_host(h, (2, 600000), dtype, backend)
    for op, fn in ((0, backend.sum), (1, backend.max)):
        for hv, tv, axes in ((h, t, []), (h.reshape(4, 300000), t.reshape([4, 300000]), [1])):  # one output; four, each in 37 slices
            out = fn(tv, axes)
            assert int(backend.last_kernel().rsplit("_x", 1)[1]) >= 32, backend.last_kernel()
            st, ref = oracle.reduce(op, hv, axes, TAGS[dtype])
            if dtype in INTS or op == 1:
                assert st == 0 and np.array_equal(out.to_host(), ref)
            else:
                assert rel_err(as_f64(out.to_host(), dtype), np.asarray(as_f64(hv, dtype).sum(axis=tuple(axes) if axes else None))) <= tol[dtype]
    if dtype in FLOATS:
        # max propagates NaN wherever it sits in the slice, through every thread mapping
        for shape, axes in (((5, 3000), [1]), ((3000, 5), [0]), ((40, 4096), [0]), ((64, 64), []), ((9600, 37), [1]), ((2, 600000), [])):
            h = host(oracle, shape, dtype, 31)
            flat = h.reshape(-1)
            for pos in (0, flat.size // 2, flat.size - 1):
                hh = flat.copy()
                hh[pos] = 0x7FC0 if dtype == DType.BF16 else np.nan
                hh = hh.reshape(shape)
                got = as_f64(backend.max(Tensor.from_host(hh, shape, dtype, backend), axes).to_host(), dtype)
                st, ref = oracle.reduce(1, hh, axes, TAGS[dtype])
                ref = as_f64(ref, dtype)
                assert st == 0 and np.array_equal(np.isnan(got), np.isnan(ref)) and np.isnan(ref).sum() == 1, (shape, axes, pos)
                assert np.array_equal(got[~np.isnan(got)], ref[~np.isnan(ref)])
    e = Tensor.from_host(np.zeros((3, 0), np.float32), (3, 0), DType.F32, backend)
    assert backend.sum(e, [1]).to_host().tolist() == [0.0, 0.0, 0.0]
    with pytest.raises(ox.NotImplementedOp):
        backend.max(e, [1])
    with pytest.raises(ox.IndexOutOfBounds):
        backend.sum(e, [2])


@pytest.mark.parametrize("dtype", FLOATS + INTS, ids=lambda d: d.name)
def test_transposed_operands_take_the_tile_kernel(backend, oracle, dtype):
    """Operands whose unit stride is not on the innermost dim (extent >= 32 on
    the unit-stride dim): ragged 32x32 tiles, a batch dim outside and between
    the tile dims, either or both operands turned."""
    shapes = [((70, 45), (1, 0)), ((3, 40, 50), (0, 2, 1)), ((40, 3, 50), (2, 1, 0)), ((33, 2, 2, 65), (3, 1, 2, 0))]
    # extents that are multiples of 4 with aligned rows: 2- and 4-byte elements turn in registers (one tile,
    # several ragged tiles, a batch dim outside and between the tile dims)
    shapes += [((72, 48), (1, 0)), ((200, 136), (1, 0)), ((3, 40, 52), (0, 2, 1)), ((44, 3, 60), (2, 1, 0))]
    for shape, perm in shapes:
        h = host(oracle, shape, dtype, 40)
        t = Tensor.from_host(h, shape, dtype, backend)
        hv, tv = h.transpose(perm), t.permute(list(perm))
        out = backend.neg(tv)
        assert backend.last_kernel() == "unary_neg" and out.layout().is_contiguous()
        assert_close(out.to_host(), oracle.unary(0, hv, TAGS[dtype])[1], dtype)
        assert np.array_equal(tv.contiguous().to_host(), np.ascontiguousarray(hv))
        g = host(oracle, hv.shape, dtype, 41)           # row-major partner
        tg = Tensor.from_host(g, g.shape, dtype, backend)
        assert_close(backend.add(tg, tv).to_host(), oracle.binary(0, g, hv, TAGS[dtype])[1], dtype, ulps=1)
        assert_close(backend.sub(tv, tg).to_host(), oracle.binary(1, hv, g, TAGS[dtype])[1], dtype, ulps=1)
        h2 = host(oracle, shape, dtype, 42)             # both turned the same way
        t2 = Tensor.from_host(h2, shape, dtype, backend)
        assert_close(backend.mul(tv, t2.permute(list(perm))).to_host(), oracle.binary(2, hv, h2.transpose(perm), TAGS[dtype])[1], dtype, ulps=1)
        row = host(oracle, hv.shape[-1:], dtype, 43)    # a broadcast row against a turned operand
        trow = Tensor.from_host(row, row.shape, dtype, backend)
        assert_close(backend.add(tv, trow).to_host(), oracle.binary(0, hv, row, TAGS[dtype])[1], dtype, ulps=1)


@pytest.mark.parametrize("dtype", [DType.U8, DType.Bool, DType.F64, DType.BF16], ids=lambda d: d.name)
def test_contiguous_of_transposed_views(backend, dtype):
    rng = np.random.default_rng(5)
    npdt = {DType.U8: np.uint8, DType.Bool: np.uint8, DType.F64: np.float64, DType.BF16: np.uint16}[dtype]
    for shape, perm in (((130, 77), (1, 0)), ((5, 64, 48), (0, 2, 1)), ((48, 5, 64), (2, 1, 0))):
        h = rng.integers(0, 2 if dtype == DType.Bool else 200, size=shape).astype(npdt)
        t = Tensor.from_host(h, shape, dtype, backend)
        got = t.permute(list(perm)).contiguous()
        assert got.layout().is_contiguous()
        assert np.array_equal(got.to_host(), np.ascontiguousarray(h.transpose(perm)))
        # a window of the transposed view: offset and ragged tiles
        w = t.permute(list(perm)).narrow(len(shape) - 1, 3, 33)
        assert np.array_equal(w.contiguous().to_host(), np.ascontiguousarray(h.transpose(perm)[..., 3:36]))
