"""The CPU oracle against the reference's own hand-computed constants and laws
(exercises/a4-reference-matmul/tests/spec.rs) and against committed fixtures."""
import json
import os

import numpy as np
import pytest
from hypothesis import given, settings, strategies as st

from tests.oracle_lib import ACC_F64, ACC_NATIVE, BF16, F16, F32, Oracle

GOLD = os.path.join(os.path.dirname(__file__), "golden")
HAND = json.load(open(os.path.join(GOLD, "a4_hand_cases.json")))
FIX = json.load(open(os.path.join(GOLD, "oracle_fixtures.json")))
TAGS = {"f32": F32, "bf16": BF16, "f16": F16}


def close_spec(x, y, tol=1e-4):
    """The reference's own tolerance form (a4 spec.rs:114,128)."""
    return abs(x - y) <= tol * (1.0 + max(abs(x), abs(y)))


@pytest.mark.parametrize("case", HAND["matmul"], ids=lambda c: c["name"])
def test_hand_cases_are_bit_exact(oracle, case):
    a = np.array(case["a"], np.float32).reshape(case["a_shape"])
    b = np.array(case["b"], np.float32).reshape(case["b_shape"])
    if "b_permute" in case:
        b = b.transpose(case["b_permute"])  # a view: strides, not fresh bytes
        assert not b.flags["C_CONTIGUOUS"]
    for acc in (ACC_NATIVE, ACC_F64):
        status, c = oracle.matmul(a, b, F32, acc=acc)
        assert status == 0
        assert list(c.shape) == case["expected_shape"]
        assert c.reshape(-1).tolist() == case["expected"]


def test_inner_dimension_mismatch_is_shape_mismatch(oracle):
    a, b = np.ones((2, 3), np.float32), np.ones((4, 2), np.float32)
    status, _ = oracle.matmul(a, b, F32)
    assert status == 1  # ShapeMismatch


def test_rank_1_operands_are_refused(oracle):
    a = np.ones(6, np.float32)
    status, _ = oracle.matmul(a, a, F32, batched=False)
    assert status != 0


def test_dtype_rules(oracle):
    a, b = np.ones((2, 2), np.float32), np.ones((2, 2), np.uint16)
    from tests.oracle_lib import _view
    import ctypes as C
    va, vb = _view(a, F32), _view(b, BF16)
    assert oracle.lib.orc_check_matmul(C.byref(va), C.byref(vb), None, 0) == 3  # DTypeMismatch
    vi = _view(a, 2)  # I32
    assert oracle.lib.orc_check_matmul(C.byref(vi), C.byref(vi), None, 0) == 4  # UnsupportedDType


mat = lambda r, c: st.lists(st.floats(-8.0, 8.0, width=32), min_size=r * c, max_size=r * c).map(
    lambda d: np.array(d, np.float32).reshape(r, c))


@settings(max_examples=60, deadline=None)
@given(mat(2, 3), mat(3, 2))
def test_transpose_law(a, b):
    o = Oracle()
    _, ab = o.matmul(a, b, F32)
    _, btat = o.matmul(b.T, a.T, F32)  # both operands are transposed views
    for i in range(2):
        for j in range(2):
            assert close_spec(float(ab.T[i, j]), float(btat[i, j]))


@settings(max_examples=60, deadline=None)
@given(mat(3, 3), mat(3, 2), st.integers(0, 1))
def test_columns_are_independent(a, b, j):
    o = Oracle()
    _, full = o.matmul(a, b, F32)
    _, col = o.matmul(a, b[:, j:j + 1], F32)  # narrow(1, j, 1)
    for i in range(3):
        assert close_spec(float(full[i, j]), float(col[i, 0]))


@pytest.mark.parametrize("case", HAND["broadcast_ok"]["cases"], ids=str)
def test_broadcast_hand_cases(oracle, case):
    lhs, rhs, exp = case
    status, got = oracle.broadcast_shapes(lhs, rhs)
    assert status == 0 and list(got) == exp


@pytest.mark.parametrize("case", HAND["broadcast_refuse"]["cases"], ids=str)
def test_broadcast_refusals(oracle, case):
    status, _ = oracle.broadcast_shapes(case[0], case[1])
    assert status == 2  # BroadcastIncompatible


def test_fixture_fill_streams(oracle):
    for f in FIX["fill"]:
        tag = TAGS[f["dtype"]]
        x = oracle.fill((16,), tag, f["seed"], f["stream"], f["dist"], f["scale"])
        bits = x.view(np.uint32 if tag == F32 else np.uint16)
        assert [int(v) for v in bits] == f["bits"], f


def test_fixture_products(oracle):
    for f in FIX["matmul"]:
        tag = TAGS[f["dtype"]]
        a = oracle.fill(tuple(f["a_shape"]), tag, f["seed"], 0, "uniform")
        b = oracle.fill(tuple(f["b_shape"]), tag, f["seed"], 1, "uniform")
        _, c = oracle.matmul(a, b, tag, acc=ACC_F64 if f["acc"] == "f64" else ACC_NATIVE, nthreads=1)
        assert [float(v).hex() for v in c.reshape(-1)] == f["out_hex"], f["dtype"]


def _as_f64(x, tag):
    if tag == BF16:
        return (x.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    return x.astype(np.float64)


@pytest.mark.parametrize("tag", [F32, BF16, F16])
def test_oracle_agrees_with_numpy_float64(oracle, tag):
    a = oracle.fill((2, 1, 17, 33), tag, 5, 0, "normal")
    b = oracle.fill((1, 3, 33, 9), tag, 5, 1, "normal")
    a_view = a.transpose(0, 1, 3, 2).copy().transpose(0, 1, 3, 2)  # M-major storage
    status, c = oracle.matmul(a_view, b, tag, acc=ACC_F64)
    assert status == 0 and c.shape == (2, 3, 17, 9)
    ref = np.matmul(_as_f64(a, tag), _as_f64(b, tag))
    np.testing.assert_allclose(c, ref, rtol=1e-12, atol=1e-12)
    status, c32 = oracle.matmul(a_view, b, tag, acc=ACC_NATIVE)
    np.testing.assert_allclose(c32, ref, rtol=1e-4, atol=1e-4)


def test_threaded_equals_single_thread(oracle):
    a = oracle.fill((3, 40, 50), F32, 9, 0, "normal")
    b = oracle.fill((50, 30), F32, 9, 1, "normal")
    _, c1 = oracle.matmul(a, b, F32, nthreads=1)
    _, c8 = oracle.matmul(a, b, F32, nthreads=8)
    assert np.array_equal(c1, c8)


def test_empty_and_degenerate_shapes(oracle):
    _, c = oracle.matmul(np.zeros((0, 3), np.float32), np.zeros((3, 2), np.float32), F32)
    assert c.shape == (0, 2)
    _, c = oracle.matmul(np.ones((2, 0), np.float32), np.ones((0, 2), np.float32), F32)
    assert c.shape == (2, 2) and not c.any()  # empty contraction sums to zero


def test_negative_strides(oracle):
    a = oracle.fill((4, 6), F32, 3, 0, "uniform")
    b = oracle.fill((6, 5), F32, 3, 1, "uniform")
    _, c = oracle.matmul(a[::-1, ::-1], b[::-1, :], F32, acc=ACC_F64)
    np.testing.assert_allclose(c, a[::-1, ::-1].astype(np.float64) @ b[::-1, :].astype(np.float64), rtol=1e-12)
