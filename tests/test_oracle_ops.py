"""The oracle's elementwise and reduction loops against numpy in float64 /
int64 (CPU only).  These restate UnaryOps, BinaryOps and ReduceOps of
crates/oxmera-ops/src/lib.rs:27-50,61-69, which the reference leaves todo!()."""
import numpy as np
import pytest

from tests.oracle_lib import BF16, F16, F32, F64, I32, I64

UNARY = {0: np.negative, 1: np.exp, 2: np.log, 3: np.abs}
BINARY = {0: np.add, 1: np.subtract, 2: np.multiply, 3: np.divide}


def test_unary_through_views(oracle):
    a = np.abs(oracle.fill((3, 4, 5), F32, 1, 0, "normal")) + 0.1
    for view in (a, a.transpose(2, 0, 1), a[::-1, 1:3, ::2]):
        for op, f in UNARY.items():
            st, c = oracle.unary(op, view, F32)
            assert st == 0
            np.testing.assert_allclose(c, f(view.astype(np.float64)).astype(np.float32), rtol=1e-6)
    i = np.arange(-6, 6, dtype=np.int64).reshape(3, 4)
    assert oracle.unary(0, i, I64)[1].tolist() == (-i).tolist()
    assert oracle.unary(3, i.T, I64)[1].tolist() == np.abs(i.T).tolist()
    assert oracle.unary(1, i, I64)[0] == 4 and oracle.unary(2, i.astype(np.int32), I32)[0] == 4  # UnsupportedDType


def test_binary_broadcasts_like_numpy(oracle):
    cases = [((2, 3), (3,)), ((2, 1), (1, 3)), ((), (2, 3)), ((4, 1, 5), (3, 1)), ((5,), (1,)), ((2, 0), (1, 1))]
    for ls, rs in cases:
        a, b = oracle.fill(ls, F64, 2, 0, "normal"), oracle.fill(rs, F64, 2, 1, "normal") + 3.0
        for op, f in BINARY.items():
            st, c = oracle.binary(op, a, b, F64)
            assert st == 0 and c.shape == np.broadcast_shapes(ls, rs)
            np.testing.assert_array_equal(c, f(a, b))
    assert oracle.binary(0, np.zeros((2, 3)), np.zeros((2, 4)), F64)[0] == 2  # BroadcastIncompatible
    i = np.arange(12, dtype=np.int32).reshape(3, 4)
    assert oracle.binary(2, i, i[:1], I32)[1].tolist() == (i * i[:1]).tolist()


def test_integer_division_and_its_typed_zero_error(oracle):
    # crates/oxmera-ops/src/lib.rs:47-49: "Integer division by zero is a typed error"
    for tag, dt in ((I32, np.int32), (I64, np.int64)):
        a = np.array([[7, -7, 9, -9], [0, 100, -100, 5]], dt)
        b = np.array([2, -2, 4, 3], dt)
        st, c = oracle.binary(3, a, b, tag)
        assert st == 0 and c.tolist() == [[3, 3, 2, -3], [0, -50, -25, 1]]  # truncation toward zero
        lo = np.iinfo(dt).min
        st, c = oracle.binary(3, np.array([lo, lo + 1], dt), np.array([-1, -1], dt), tag)
        assert st == 0 and c.tolist() == [lo, -(lo + 1)]  # the most negative value over -1 wraps
        st, c = oracle.binary(3, a, np.array([2, 0, 4, 3], dt), tag)
        assert st == 13 and c[:, 1].tolist() == [0, 0] and c[:, 0].tolist() == [3, 0]  # DivisionByZero; others still computed
    st, c = oracle.binary(3, np.array([1.0, -1.0, 0.0], np.float32), np.zeros(3, np.float32), F32)
    assert st == 0 and np.isposinf(c[0]) and np.isneginf(c[1]) and np.isnan(c[2])  # float division follows IEEE-754


def test_max_propagates_nan(oracle):
    x = oracle.fill((4, 6), F32, 5, 0, "normal")
    for pos in (0, 3, 5):
        y = x.copy()
        y[1, pos] = np.nan
        st, c = oracle.reduce(1, y, [1], F32)
        assert st == 0 and np.isnan(c[1]) and not np.isnan(c[[0, 2, 3]]).any()
        assert np.array_equal(c[[0, 2, 3]], y[[0, 2, 3]].max(axis=1))
    st, c = oracle.reduce(1, np.full((2, 3), np.nan, np.float32), [], F32)
    assert st == 0 and np.isnan(c)


def test_fill_covers_f64_and_refuses_what_it_cannot_write(oracle):
    x = oracle.fill((1000,), F64, 9, 0, "normal")
    assert x.dtype == np.float64 and np.isfinite(x).all() and 0.8 < x.std() < 1.2
    assert np.array_equal(x.astype(np.float32), oracle.fill((1000,), F32, 9, 0, "normal"))  # the same stream, rounded
    with pytest.raises(AssertionError):
        oracle.fill((4,), I32, 9, 0, "normal")


@pytest.mark.parametrize("tag", [F32, F64, BF16, F16, I32, I64])
def test_reduce_over_axes(oracle, tag):
    if tag in (I32, I64):
        x = np.arange(-60, 60, dtype=np.int32 if tag == I32 else np.int64).reshape(4, 5, 6)
        ref = x.astype(np.int64)
    else:
        x = oracle.fill((4, 5, 6), tag, 3, 0, "normal")
        ref = (x.astype(np.uint32) << 16).view(np.float32).astype(np.float64) if tag == BF16 else x.astype(np.float64)
    for axes in ([], [0], [2], [0, 2], [1], [0, 1, 2]):
        ax = tuple(axes) if axes else None
        st, c = oracle.reduce(0, x, axes, tag)
        assert st == 0
        got = (c.astype(np.uint32) << 16).view(np.float32) if tag == BF16 else c
        tol = {F32: 1e-6, F64: 1e-14, BF16: 1e-2, F16: 2e-3}.get(tag, 0)
        np.testing.assert_allclose(got.astype(np.float64), ref.sum(axis=ax), rtol=tol, atol=tol * 4)
        st, c = oracle.reduce(1, x, axes, tag)
        got = (c.astype(np.uint32) << 16).view(np.float32) if tag == BF16 else c
        np.testing.assert_array_equal(got.astype(np.float64), ref.max(axis=ax))
    assert oracle.reduce(0, x, [3], tag)[0] == 6 and oracle.reduce(0, x, [1, 1], tag)[0] == 6  # IndexOutOfBounds


def test_empty_reductions(oracle):
    e = np.zeros((3, 0), np.float32)
    st, c = oracle.reduce(0, e, [1], F32)
    assert st == 0 and c.tolist() == [0.0, 0.0, 0.0]  # an empty sum is zero
    assert oracle.reduce(1, e, [1], F32)[0] == 9       # an empty max has no identity: refused
