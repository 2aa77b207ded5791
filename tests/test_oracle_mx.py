"""The oracle's block-scaled fp8 product (orc_matmul_mx) against hand-computed
cases and a NumPy restatement of the published definition (OCP Microscaling
Formats v1.0: a block of 32 fp8 elements shares one E8M0 scale 2^(e - 127);
e = 255 is NaN).  The reference has no quantised product, so these pins are
this repository's own."""
import numpy as np
import pytest

from tests.oracle_lib import F8E4M3, F8E5M2, Oracle


@pytest.fixture(scope="module")
def oracle():
    return Oracle()


def numpy_mx(oracle, a, sa, b, sb, tag):
    fa = oracle.fp8_to_f32(a, tag).astype(np.float64)
    fb = oracle.fp8_to_f32(b, tag).astype(np.float64)
    scale = lambda e: np.where(e == 255, np.nan, np.ldexp(1.0, e.astype(np.int64) - 127))
    fa = fa * np.repeat(scale(sa), 32, axis=-1)
    fb = fb * np.repeat(scale(sb), 32, axis=-2)
    return fa @ fb


def test_hand_case(oracle):
    # a = all 1.0 (e4m3 0x38), b = all 2.0 (0x40); K = 64 = two blocks
    a = np.full((2, 64), 0x38, np.uint8)
    b = np.full((64, 3), 0x40, np.uint8)
    sa = np.array([[127, 128], [126, 127]], np.uint8)       # row 0: 1, 2; row 1: 1/2, 1
    sb = np.array([[127, 127, 129], [127, 125, 127]], np.uint8)  # block 0: 1, 1, 4; block 1: 1, 1/4, 1
    st, out = oracle.matmul_mx(a, sa, b, sb, F8E4M3)
    assert st == 0
    blk = 32 * 1.0 * 2.0
    want = np.array([[blk * (1 * 1 + 2 * 1), blk * (1 * 1 + 2 * 0.25), blk * (1 * 4 + 2 * 1)],
                     [blk * (0.5 * 1 + 1 * 1), blk * (0.5 * 1 + 1 * 0.25), blk * (0.5 * 4 + 1 * 1)]])
    assert np.array_equal(out, want)


def test_scale_extremes_and_nan(oracle):
    a = np.full((1, 32), 0x38, np.uint8)
    b = np.full((32, 1), 0x38, np.uint8)
    st, out = oracle.matmul_mx(a, np.array([[0]], np.uint8), b, np.array([[254]], np.uint8), F8E4M3)
    assert st == 0 and out[0, 0] == 32.0  # 2^-127 * 2^127
    st, out = oracle.matmul_mx(a, np.array([[255]], np.uint8), b, np.array([[127]], np.uint8), F8E4M3)
    assert st == 0 and np.isnan(out[0, 0])


@pytest.mark.parametrize("tag", [F8E4M3, F8E5M2])
def test_against_numpy_with_views_and_broadcast(oracle, tag):
    rng = np.random.default_rng(7)
    a = oracle.fill((3, 1, 20, 96), tag, 11, 0, "normal")
    bt = oracle.fill((4, 24, 96), tag, 11, 1, "normal")  # B held transposed: a strided view below
    sa = rng.integers(120, 134, size=(3, 1, 20, 3), dtype=np.uint8)
    sbt = rng.integers(120, 134, size=(4, 24, 3), dtype=np.uint8)
    b, sb = np.swapaxes(bt, -1, -2), np.swapaxes(sbt, -1, -2)
    st, out = oracle.matmul_mx(a, sa, b, sb, tag)
    assert st == 0 and out.shape == (3, 4, 20, 24)
    want = numpy_mx(oracle, a, sa, b, sb, tag)
    assert np.allclose(out, want, rtol=1e-12, atol=0)


def test_refusals(oracle):
    a = np.zeros((4, 48), np.uint8)
    b = np.zeros((48, 4), np.uint8)
    st, _ = oracle.matmul_mx(a, np.zeros((4, 1), np.uint8), b, np.zeros((1, 4), np.uint8), F8E4M3)
    assert st == 1  # ShapeMismatch: K = 48 is not a multiple of 32
    a, b = np.zeros((4, 64), np.uint8), np.zeros((64, 4), np.uint8)
    st, _ = oracle.matmul_mx(a, np.zeros((4, 3), np.uint8), b, np.zeros((2, 4), np.uint8), F8E4M3)
    assert st == 1
