"""Parity of the CUDA path with the CPU oracle, through the C ABI, on a B200.

Tolerances (stated once, used everywhere below):
  f32            max |x-y| / max(|y|, rms(Y)) <= 1e-4 against the f64-accumulated oracle
  bf16 / f16     same measure <= 1e-2 against the oracle's f32 result on the same rounded inputs
Small-integer products (the reference's hand cases) must be bit-exact.
"""
import json
import os

import numpy as np
import pytest

import oxmera_b200 as ox
from oxmera_b200 import DType, Tensor
from tests.guard import Guarded, guarded_matmul
from tests.oracle_lib import ACC_F64, ACC_NATIVE, BF16, F16, F32

pytestmark = pytest.mark.gpu

HAND = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "a4_hand_cases.json")))
TAG = {DType.F32: F32, DType.BF16: BF16, DType.F16: F16}
TOL = {DType.F32: 1e-4, DType.BF16: 1e-2, DType.F16: 1e-2}
KERNELS = {"auto": 0, "simt": 1, "tcgen05": 2}


def to_f64(x, dtype):
    if dtype == DType.BF16:
        return ox.bf16_bits_to_f32(x).reshape(x.shape).astype(np.float64)
    return x.astype(np.float64)


def rel_err(got, ref):
    ref = ref.astype(np.float64)
    got = got.astype(np.float64)
    rms = float(np.sqrt(np.mean(ref * ref))) if ref.size else 0.0
    if rms == 0.0:
        return 0.0 if np.array_equal(got, ref) else float("inf")
    return float(np.max(np.abs(got - ref) / np.maximum(np.abs(ref), rms)))


def oracle_ref(oracle, a, b, dtype):
    """The reference result the tolerance is stated against."""
    acc = ACC_F64 if dtype == DType.F32 else ACC_NATIVE
    st, ref = oracle.matmul(a, b, TAG[dtype], acc=acc)
    assert st == 0
    return ref


def fill(oracle, shape, dtype, seed, stream, dist="normal", scale=1.0):
    return oracle.fill(shape, TAG[dtype], seed, stream, dist, scale)


def set_kernel(backend, name, tile_n=0, pair=-1):
    backend.set_option("kernel", KERNELS[name])
    backend.set_option("tile_n", tile_n)
    backend.set_option("cta_pair", pair)
    backend.set_option("split_k", -1)
    backend.set_option("stream_k", -1)


@pytest.fixture(autouse=True)
def _reset_options(backend):
    yield
    set_kernel(backend, "auto")


# ---------------------------------------------------------------------------
# the reference's own spec (exercises/a4-reference-matmul/tests/spec.rs)
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("kernel", list(KERNELS))
@pytest.mark.parametrize("case", HAND["matmul"], ids=lambda c: c["name"])
def test_hand_cases_are_bit_exact(backend, kernel, case):
    set_kernel(backend, kernel)
    a = Tensor.from_host(np.array(case["a"], np.float32), case["a_shape"], DType.F32, backend)
    b = Tensor.from_host(np.array(case["b"], np.float32), case["b_shape"], DType.F32, backend)
    if "b_permute" in case:
        b = b.permute(case["b_permute"])
    c = a.matmul(b)  # TensorOps -> backend_for(device) -> MatmulOps::matmul
    assert list(c.shape) == case["expected_shape"]
    assert c.layout().is_contiguous()
    assert c.to_host().reshape(-1).tolist() == case["expected"]
    idx = [s - 1 for s in case["expected_shape"]]
    assert c.get_f32(idx) == case["expected"][-1]


def test_typed_errors(backend):
    f = lambda shape, dt=DType.F32: Tensor.empty(shape, dt, backend)
    with pytest.raises(ox.ShapeMismatch) as e:
        backend.matmul(f((2, 3)), f((4, 2)))
    assert "matmul" in str(e.value)
    with pytest.raises(ox.OxmeraError):
        backend.matmul(f((6,)), f((6,)))  # rank-1 operands must refuse
    with pytest.raises(ox.ShapeMismatch):
        backend.matmul(f((2, 2, 3)), f((3, 2)))  # rank-2 only for matmul
    with pytest.raises(ox.DTypeMismatch):
        backend.matmul(f((2, 3)), f((3, 2), DType.BF16))
    with pytest.raises(ox.UnsupportedDType):
        backend.matmul(f((2, 3), DType.I32), f((3, 2), DType.I32))
    with pytest.raises(ox.BroadcastIncompatible):
        backend.batched_matmul(f((2, 4, 3)), f((3, 3, 5)))
    with pytest.raises(ox.ShapeMismatch):
        backend.matmul_into(f((2, 3)), f((3, 2)), f((2, 3)), batched=False)  # wrong output shape
    # the context is still healthy
    c = backend.matmul(Tensor.from_host(np.eye(2, dtype=np.float32), (2, 2), DType.F32, backend),
                       Tensor.from_host(np.array([1, 2, 3, 4], np.float32), (2, 2), DType.F32, backend))
    assert c.to_host().reshape(-1).tolist() == [1.0, 2.0, 3.0, 4.0]


def test_unregistered_device_is_backend_unavailable(backend):
    with pytest.raises(ox.BackendUnavailable):
        ox.backend_for(ox.Device.cuda(63))
    with pytest.raises(ox.BackendUnavailable):
        ox.B200Backend(63)
    assert ox.backend_for(ox.Device.cuda(0)) is backend
    assert backend.name() == "b200-tcgen05"


@pytest.mark.parametrize("kernel", ["simt", "tcgen05"])
def test_transpose_law_and_column_independence(backend, oracle, kernel):
    set_kernel(backend, kernel)
    spec_close = lambda x, y: np.all(np.abs(x - y) <= 1e-4 * (1 + np.maximum(np.abs(x), np.abs(y))))
    rng = np.random.default_rng(4)
    for _ in range(8):
        a = Tensor.from_host(rng.uniform(-8, 8, 6).astype(np.float32), (2, 3), DType.F32, backend)
        b = Tensor.from_host(rng.uniform(-8, 8, 6).astype(np.float32), (3, 2), DType.F32, backend)
        ab_t = a.matmul(b).permute([1, 0]).to_host()
        bt_at = b.permute([1, 0]).matmul(a.permute([1, 0])).to_host()
        assert spec_close(ab_t, bt_at)
        a3 = Tensor.from_host(rng.uniform(-8, 8, 9).astype(np.float32), (3, 3), DType.F32, backend)
        full = a3.matmul(b).to_host()
        for j in range(2):
            col = a3.matmul(b.narrow(1, j, 1)).to_host()
            assert spec_close(full[:, j], col[:, 0])


# ---------------------------------------------------------------------------
# shapes, dtypes and kernels
# ---------------------------------------------------------------------------
SHAPES = [(1, 1, 1), (2, 3, 4), (7, 5, 3), (64, 64, 64), (128, 256, 64), (129, 257, 65), (130, 70, 520),
          (300, 520, 200), (77, 33, 1000), (256, 384, 512), (1, 300, 40), (300, 1, 40), (33, 65, 1)]


@pytest.mark.parametrize("dtype", [DType.F32, DType.BF16, DType.F16], ids=lambda d: d.name)
@pytest.mark.parametrize("kernel", ["simt", "tcgen05"])
def test_shape_sweep(backend, oracle, kernel, dtype):
    set_kernel(backend, kernel)
    for i, (m, n, k) in enumerate(SHAPES):
        a = fill(oracle, (m, k), dtype, 100 + i, 0)
        b = fill(oracle, (k, n), dtype, 100 + i, 1)
        ta, tb = Tensor.from_host(a, a.shape, dtype, backend), Tensor.from_host(b, b.shape, dtype, backend)
        got = backend.matmul(ta, tb).to_host()
        err = rel_err(to_f64(got, dtype), oracle_ref(oracle, a, b, dtype))
        assert err <= TOL[dtype], (kernel, dtype.name, (m, n, k), err, backend.last_kernel())
        # the same product into outputs with guard bands: nothing outside the output may be written,
        # whichever epilogue the output's alignment selects, and not a bit of the result may change
        for layout, aligned in (("flat", True), ("window", True), ("window", False)):
            assert np.array_equal(guarded_matmul(backend, ta, tb, layout=layout, aligned=aligned), got), (kernel, (m, n, k), layout, aligned)


@pytest.mark.parametrize("dtype", [DType.BF16, DType.F16, DType.F32], ids=lambda d: d.name)
@pytest.mark.parametrize("dims", [(256, 384, 320), (250, 130, 99), (512, 256, 1024), (304, 1544, 136)], ids=str)
@pytest.mark.parametrize("a_t,b_t", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_transposed_operands_need_no_copy(backend, oracle, dims, a_t, b_t, dtype):
    """All four (A, B) major combinations: K-major and MN-major operands reach
    the tensor cores as views.  Aligned extents take the direct TMA path,
    unaligned ones the pack path."""
    set_kernel(backend, "tcgen05", tile_n=512 if dims[1] > 1024 else 0)  # the widest case runs 256 x 512 pair tiles
    m, n, k = dims
    ha = fill(oracle, (k, m) if a_t else (m, k), dtype, 7, 0)
    hb = fill(oracle, (n, k) if b_t else (k, n), dtype, 7, 1)
    ta = Tensor.from_host(ha, ha.shape, dtype, backend)
    tb = Tensor.from_host(hb, hb.shape, dtype, backend)
    if a_t:
        ha, ta = ha.T, ta.permute([1, 0])
    if b_t:
        hb, tb = hb.T, tb.permute([1, 0])
    before = backend.launch_counts()
    got = backend.matmul(ta, tb)
    after = backend.launch_counts()
    assert after["tcgen05"] == before["tcgen05"] + 1
    if dtype != DType.F32 and dims != (250, 130, 99):
        assert after["pack"] == before["pack"], "aligned 16-bit views must be read in place"
    err = rel_err(to_f64(got.to_host(), dtype), oracle_ref(oracle, ha, hb, dtype))
    assert err <= TOL[dtype], (dims, a_t, b_t, err, backend.last_kernel())


@pytest.mark.parametrize("kernel", ["simt", "tcgen05"])
@pytest.mark.parametrize("dtype", [DType.F32, DType.BF16], ids=lambda d: d.name)
def test_narrowed_and_flipped_views(backend, oracle, kernel, dtype):
    set_kernel(backend, kernel)
    ha = fill(oracle, (90, 150), dtype, 21, 0)
    hb = fill(oracle, (160, 70), dtype, 21, 1)
    ta = Tensor.from_host(ha, ha.shape, dtype, backend)
    tb = Tensor.from_host(hb, hb.shape, dtype, backend)
    # odd windows: offsets that are not 16-byte aligned
    va, vta = ha[3:80, 5:133], ta.narrow(0, 3, 77).narrow(1, 5, 128)
    vb, vtb = hb[17:145, 1:66], tb.narrow(0, 17, 128).narrow(1, 1, 65)
    err = rel_err(to_f64(backend.matmul(vta, vtb).to_host(), dtype), oracle_ref(oracle, va, vb, dtype))
    assert err <= TOL[dtype]
    # negative strides
    fa, fta = va[::-1, ::-1], vta.flip(0).flip(1)
    fb, ftb = vb[::-1, :], vtb.flip(0)
    err = rel_err(to_f64(backend.matmul(fta, ftb).to_host(), dtype), oracle_ref(oracle, fa, fb, dtype))
    assert err <= TOL[dtype]


@pytest.mark.parametrize("kernel", ["simt", "tcgen05"])
@pytest.mark.parametrize("dtype", [DType.F32, DType.BF16, DType.F16], ids=lambda d: d.name)
def test_broadcast_batch_dims(backend, oracle, kernel, dtype):
    set_kernel(backend, kernel)
    cases = [
        ((3, 1, 24, 40), True, (1, 5, 24, 56)),   # the strided-view config in miniature: A is a transposed view
        ((2, 3, 40, 24), False, (2, 3, 24, 56)),  # equal batch dims
        ((4, 64, 32), False, (32, 48)),           # shared B: folds into one tall product
        ((64, 32), False, (5, 32, 48)),           # shared A
        ((2, 1, 3, 16, 8), False, (4, 1, 8, 24)), # interleaved broadcast dims
    ]
    for i, (ashape, a_t, bshape) in enumerate(cases):
        ha = fill(oracle, ashape, dtype, 50 + i, 0)
        hb = fill(oracle, bshape, dtype, 50 + i, 1)
        ta = Tensor.from_host(ha, ashape, dtype, backend)
        tb = Tensor.from_host(hb, bshape, dtype, backend)
        if a_t:
            perm = list(range(len(ashape) - 2)) + [len(ashape) - 1, len(ashape) - 2]
            ha, ta = ha.transpose(perm), ta.permute(perm)
        got = backend.batched_matmul(ta, tb)
        ref = oracle_ref(oracle, ha, hb, dtype)
        assert got.shape == ref.shape
        err = rel_err(to_f64(got.to_host(), dtype), ref)
        assert err <= TOL[dtype], (ashape, bshape, err, backend.last_kernel())


@pytest.mark.parametrize("dtype", [DType.F32, DType.BF16, DType.F16], ids=lambda d: d.name)
def test_seeded_random_products_under_the_default_planner(backend, oracle, dtype):
    """Whatever the planner picks by itself (FFMA or tensor cores, packed or in
    place, split or not, the order it walks the batch dims in): random extents,
    random broadcast batch dims, either operand transposed, windowed or both."""
    rng = np.random.default_rng({DType.F32: 11, DType.BF16: 12, DType.F16: 13}[dtype])
    kernels = set()
    for case in range(36):
        m, n, k = (int(x) for x in rng.integers(1, 330, size=3))
        if case % 6 == 0:
            k = int(rng.integers(400, 2200))  # long contractions: the split paths
        nb = int(rng.integers(0, 3))
        batch = [int(x) for x in rng.integers(1, 4, size=nb)]
        a_batch = [1 if rng.random() < 0.3 else d for d in batch]
        b_batch = [1 if rng.random() < 0.3 else d for d in batch]
        if rng.random() < 0.3:
            b_batch = b_batch[1:]  # B with fewer batch dims than A
        a_t, b_t, win = rng.random() < 0.4, rng.random() < 0.4, rng.random() < 0.3
        pad = 3 if win else 0
        ashape = tuple(a_batch) + ((k + pad, m + pad) if a_t else (m + pad, k + pad))
        bshape = tuple(b_batch) + ((n, k) if b_t else (k, n))
        ha, hb = fill(oracle, ashape, dtype, 900 + case, 0), fill(oracle, bshape, dtype, 900 + case, 1)
        ta, tb = Tensor.from_host(ha, ashape, dtype, backend), Tensor.from_host(hb, bshape, dtype, backend)
        if a_t:
            perm = list(range(len(ashape) - 2)) + [len(ashape) - 1, len(ashape) - 2]
            ha, ta = ha.transpose(perm), ta.permute(perm)
        if b_t:
            perm = list(range(len(bshape) - 2)) + [len(bshape) - 1, len(bshape) - 2]
            hb, tb = hb.transpose(perm), tb.permute(perm)
        if win:  # an odd window of A: offsets and strides that are not 16-byte multiples
            ha = ha[..., 1:m + 1, 2:k + 2]
            ta = ta.narrow(len(ashape) - 2, 1, m).narrow(len(ashape) - 1, 2, k)
        got = backend.batched_matmul(ta, tb)
        kernels.add(backend.last_kernel().split("_bn")[0].split("_w")[0])
        ref = oracle_ref(oracle, ha, hb, dtype)
        assert got.shape == ref.shape, (case, ashape, bshape)
        err = rel_err(to_f64(got.to_host(), dtype), ref)
        assert err <= TOL[dtype], (case, ashape, bshape, a_t, b_t, win, err, backend.last_kernel())
    assert len(kernels) >= 2, kernels  # the sweep reached more than one kernel family


@pytest.mark.parametrize("tile_n", [64, 96, 128, 160, 224, 256, 288, 320, 384, 416, 448, 480, 512])
@pytest.mark.parametrize("dtype", [DType.BF16, DType.F32], ids=lambda d: d.name)
def test_tile_widths(backend, oracle, tile_n, dtype):
    """Every kernel instance at its full width and at narrower widths (any
    multiple of 32 columns), with a B operand of either major, ragged edges in
    M and N, and guard bands around the output."""
    m, n, k = 384, 1100, 448
    cls = 512 if tile_n > 256 else 256 if tile_n > 128 else 128 if tile_n > 64 else 64
    a = fill(oracle, (m, k), dtype, 31, 0)
    ta = Tensor.from_host(a, a.shape, dtype, backend)
    for b_t in (0, 1):
        set_kernel(backend, "tcgen05", tile_n=tile_n)
        backend.set_option("split_k", 0)  # one chain per element at every width, so that widths can be compared bit for bit
        hb = fill(oracle, (n, k) if b_t else (k, n), dtype, 31, 1)
        b = hb.T if b_t else hb
        tb = Tensor.from_host(hb, hb.shape, dtype, backend)
        tb = tb.permute([1, 0]) if b_t else tb
        got = backend.matmul(ta, tb).to_host()
        name = backend.last_kernel()
        assert f"bn{cls}_" in name and (tile_n == cls or name.endswith(f"_w{tile_n}")), name
        assert rel_err(to_f64(got, dtype), oracle_ref(oracle, a, b, dtype)) <= TOL[dtype], (tile_n, b_t, name)
        for aligned in (True, False):
            assert np.array_equal(guarded_matmul(backend, ta, tb, aligned=aligned), got), (tile_n, b_t, aligned)
        # the width changes which tile an element falls in, never the chain of products behind it
        set_kernel(backend, "tcgen05", tile_n=cls)
        backend.set_option("split_k", 0)
        assert np.array_equal(backend.matmul(ta, tb).to_host(), got), (tile_n, b_t)


def test_long_f32_contractions_keep_their_accuracy(backend, oracle):
    """The tensor core adds into its fp32 accumulator with truncation, so the
    f32 path cuts contractions longer than 1024 into chains and adds the
    partial sums in round-to-nearest: the error must not grow with K."""
    set_kernel(backend, "tcgen05")
    cases = [((130, 8192), (8192, 260)), ((64, 5000), (5000, 100)), ((3, 64, 4096), (4096, 96)),
             ((2, 1, 64, 3000), (1, 2, 3000, 72))]
    for i, (ashape, bshape) in enumerate(cases):
        a, b = fill(oracle, ashape, DType.F32, 90 + i, 0), fill(oracle, bshape, DType.F32, 90 + i, 1)
        before = backend.launch_counts()
        got = backend.batched_matmul(Tensor.from_host(a, ashape, DType.F32, backend),
                                     Tensor.from_host(b, bshape, DType.F32, backend))
        after = backend.launch_counts()
        assert after["pack"] - before["pack"] == 3, "two operand packs and one partial-sum reduction"
        err = rel_err(got.to_host(), oracle_ref(oracle, a, b, DType.F32))
        print(f"f32 K={ashape[-1]}: error {err:.3e}")
        assert err <= 5e-5, (ashape, bshape, err)


@pytest.mark.parametrize("kernel", ["simt", "tcgen05", "auto"])
def test_f32_infinities_and_nans_follow_ieee_on_every_path(backend, kernel):
    """inf * 2 = inf, inf * 0 = NaN, inf - inf = NaN, NaN poisons its row and
    column, whichever kernel computes the product: the FFMA kernel does this by
    construction; the 3xTF32 split has to keep an infinity from meeting a
    correction term (inf * 0).  Small-integer data, so finite outputs are exact."""
    set_kernel(backend, kernel)
    rng = np.random.default_rng(17)
    for (m, n, k), at, bt in (((70, 50, 96), 0, 0), ((260, 300, 1500), 1, 1), ((512, 768, 2048), 1, 0)):
        a = rng.integers(-3, 4, size=(m, k)).astype(np.float32)
        b = rng.integers(-3, 4, size=(k, n)).astype(np.float32)
        a[3, 10], a[5, 20], a[9, 30], a[m - 1, k - 1] = np.inf, -np.inf, np.nan, -np.inf
        b[40, 7], b[41, 8], b[k - 1, n - 1] = np.inf, np.nan, np.inf
        a[11, 40] = np.inf  # meets b[40, 7] = inf in output (11, 7): inf * inf = inf
        with np.errstate(invalid="ignore"):
            ref = a.astype(np.float64) @ b.astype(np.float64)
        sa = np.ascontiguousarray(a.T) if at else a
        sb = np.ascontiguousarray(b.T) if bt else b
        ta, tb = Tensor.from_host(sa, sa.shape, DType.F32, backend), Tensor.from_host(sb, sb.shape, DType.F32, backend)
        ta = ta.permute([1, 0]) if at else ta
        tb = tb.permute([1, 0]) if bt else tb
        x = backend.matmul(ta, tb).to_host()
        where = (kernel, (m, n, k), backend.last_kernel())
        assert np.array_equal(np.isnan(x), np.isnan(ref)), where
        assert np.array_equal(np.isposinf(x), np.isposinf(ref)) and np.array_equal(np.isneginf(x), np.isneginf(ref)), where
        fin = np.isfinite(ref)
        assert np.array_equal(x[fin], ref[fin].astype(np.float32)), where


@pytest.mark.parametrize("dtype", [DType.BF16, DType.F16], ids=lambda d: d.name)
@pytest.mark.parametrize("a_t,b_t", [(0, 1), (1, 0)])
def test_split_k_fills_small_grids(backend, oracle, dtype, a_t, b_t):
    """A small output with a long contraction (the weight gradient of one
    shard) is cut along K into chains whose fp32 partial sums are reduced."""
    set_kernel(backend, "tcgen05")
    m, n, k = 256, 520, 8192
    ha = fill(oracle, (k, m) if a_t else (m, k), dtype, 17, 0)
    hb = fill(oracle, (n, k) if b_t else (k, n), dtype, 17, 1)
    ta, tb = Tensor.from_host(ha, ha.shape, dtype, backend), Tensor.from_host(hb, hb.shape, dtype, backend)
    if a_t:
        ha, ta = ha.T, ta.permute([1, 0])
    if b_t:
        hb, tb = hb.T, tb.permute([1, 0])
    ref = oracle_ref(oracle, ha, hb, dtype)
    for split in (-1, 0, 3, 8):
        backend.set_option("split_k", split)
        before = backend.launch_counts()
        got = backend.matmul(ta, tb)
        after = backend.launch_counts()
        if split > 0:
            assert after["pack"] == before["pack"] + 1, "one reduction pass"
        if split == 0:
            assert after["pack"] == before["pack"]
        err = rel_err(to_f64(got.to_host(), dtype), ref)
        assert err <= TOL[dtype], (split, err, backend.last_kernel())
    backend.set_option("split_k", -1)
    # the auto choice splits here: 3 column tiles cannot fill the SMs
    before = backend.launch_counts()
    backend.matmul(ta, tb)
    assert backend.launch_counts()["pack"] == before["pack"] + 1


@pytest.mark.parametrize("dtype", [DType.BF16, DType.F32], ids=lambda d: d.name)
@pytest.mark.parametrize("b_t", [0, 1])
def test_skinny_products(backend, oracle, dtype, b_t):
    """One row of tiles over a long weight matrix (a decode step): A's box
    holds just its rows, and the automatic choice splits the contraction so
    that every SM streams part of B.  Also the mirror case (one column of
    tiles) and an output width that is not a multiple of four (scalar
    reduction path)."""
    set_kernel(backend, "auto")
    for (m, n, k) in ((1, 1024, 4096), (8, 1024, 4096), (17, 1030, 4096), (100, 1024, 2048), (2048, 40, 4096)):
        ha = fill(oracle, (m, k), dtype, 31, 0)
        hb = fill(oracle, (n, k) if b_t else (k, n), dtype, 31, 1)
        ta, tb = Tensor.from_host(ha, ha.shape, dtype, backend), Tensor.from_host(hb, hb.shape, dtype, backend)
        if b_t:
            hb, tb = hb.T, tb.permute([1, 0])
        got = backend.matmul(ta, tb)
        if 2 * m * n * k >= (2e8 if dtype == DType.F32 else 8e6):  # where the FFMA kernel hands over to the tensor cores
            assert "tcgen05" in backend.last_kernel(), backend.last_kernel()
        err = rel_err(to_f64(got.to_host(), dtype), oracle_ref(oracle, ha, hb, dtype))
        assert err <= TOL[dtype], ((m, n, k), err, backend.last_kernel())


@pytest.mark.parametrize("dtype", [DType.BF16, DType.F32], ids=lambda d: d.name)
def test_stream_k_shares_the_last_tiles_out_by_contraction_block(backend, oracle, dtype):
    """Tile counts that do not divide by the SM count: the remainder (plus a
    wave when it is small) is cut into equal runs of contraction blocks; runs
    that start inside a tile hand their partial sums to the run that holds the
    tile's first block.  Forced on here for every tile shape, with ragged
    edges, and twice in a row (the hand-over flags carry a launch counter)."""
    cases = [(64, 0, (1280, 650, 1024)),     # 110 tiles on 148 CTAs: all of them shared out
             (128, 0, (1536, 1800, 1100)),   # 180 tiles: one wave and 32 more -> 180 shared out
             (256, 1, (1536, 2048, 1024)),   # 48 pair tiles on 74 pairs
             (512, 1, (2000, 3072, 1024)),   # 48 pair tiles of 256 x 512, one accumulator
             (480, 1, (2000, 3072, 1024)),   # 56 pair tiles of 256 x 480: the same instance, narrower
             (256, 0, (1024, 5120, 2048))]   # 160 tiles, 1-CTA 128 x 256
    for tile_n, pair, (m, n, k) in cases:
        if dtype == DType.F32 and k > 1024:
            k = 1024  # longer f32 contractions are split into chains, which excludes stream-K
        a, b = fill(oracle, (m, k), dtype, 61, 0), fill(oracle, (k, n), dtype, 61, 1)
        ta, tb = Tensor.from_host(a, a.shape, dtype, backend), Tensor.from_host(b, b.shape, dtype, backend)
        ref = oracle_ref(oracle, a, b, dtype)
        set_kernel(backend, "tcgen05", tile_n=tile_n, pair=pair)
        backend.set_option("stream_k", 0)
        whole = backend.matmul(ta, tb).to_host()
        backend.set_option("stream_k", 1)
        try:
            for rep in range(2):
                got = guarded_matmul(backend, ta, tb, layout="flat" if rep else "window")
                err = rel_err(to_f64(got, dtype), ref)
                assert err <= TOL[dtype], (tile_n, pair, (m, n, k), err, backend.last_kernel())
            # the two schedules differ only in where the fp32 chains are cut
            assert rel_err(to_f64(got, dtype), to_f64(whole, dtype)) <= (5e-5 if dtype == DType.F32 else 1e-2)
            backend.set_option("tma_store", 0)  # the strided-store epilogue takes the same hand-over
            got2 = backend.matmul(ta, tb).to_host()
            assert np.array_equal(got, got2)
        finally:
            backend.set_option("tma_store", 1)
            backend.set_option("stream_k", 0)


def test_expired_device_wait_is_reported_and_survivable(backend):
    """Failure detection without a fault: a wait nothing satisfies runs out
    after its bound, the kernel returns, the host reads OXM_TIMEOUT, and the
    same context multiplies correctly afterwards."""
    from oxmera_b200 import capi
    lib = capi.load()
    st = lib.oxm_selftest_bounded_wait(backend._ctx, 20)
    assert st == capi.TIMEOUT, capi.last_error()
    assert "bounded device-side wait expired" in capi.last_error()
    backend.synchronize()  # the status word was cleared: no stale error
    a = Tensor.from_host(np.array([1, 2, 3, 4], np.float32), (2, 2), DType.F32, backend)
    b = Tensor.from_host(np.array([5, 6, 7, 8], np.float32), (2, 2), DType.F32, backend)
    for kernel in ("simt", "tcgen05"):
        set_kernel(backend, kernel)
        assert backend.matmul(a, b).to_host().reshape(-1).tolist() == [19.0, 22.0, 43.0, 50.0]


@pytest.mark.parametrize("dtype", [DType.BF16, DType.F32], ids=lambda d: d.name)
def test_strided_store_epilogue_matches_the_bulk_store_epilogue(backend, oracle, dtype):
    set_kernel(backend, "tcgen05")
    for tile_n, (m, n, k) in ((0, (300, 520, 200)), (512, (520, 1100, 136)), (128, (77, 130, 72))):
        backend.set_option("tile_n", tile_n)
        a, b = fill(oracle, (3, m, k), dtype, 41, 0), fill(oracle, (3, k, n), dtype, 41, 1)
        ta, tb = Tensor.from_host(a, a.shape, dtype, backend), Tensor.from_host(b, b.shape, dtype, backend)
        outs = []
        for flag in (1, 0):
            backend.set_option("tma_store", flag)
            outs.append(backend.batched_matmul(ta, tb).to_host())
        backend.set_option("tma_store", 1)
        assert np.array_equal(outs[0], outs[1]), (tile_n, m, n, k)
        assert rel_err(to_f64(outs[0], dtype), oracle_ref(oracle, a, b, dtype)) <= TOL[dtype]


def test_empty_and_degenerate(backend):
    z = lambda shape: Tensor.from_host(np.zeros(shape, np.float32), shape, DType.F32, backend)
    assert backend.matmul(z((0, 3)), z((3, 2))).shape == (0, 2)
    c = backend.matmul(Tensor.from_host(np.ones((2, 0), np.float32), (2, 0), DType.F32, backend), z((0, 2)))
    assert c.shape == (2, 2) and not c.to_host().any()  # an empty contraction sums to zero
    assert backend.batched_matmul(z((0, 2, 3)), z((3, 2))).shape == (0, 2, 2)


def test_output_written_through_its_own_strides(backend, oracle):
    """A shard writes its rows into a window of the parent output."""
    a, b = fill(oracle, (192, 96), DType.BF16, 61, 0), fill(oracle, (96, 160), DType.BF16, 61, 1)
    ta, tb = Tensor.from_host(a, a.shape, DType.BF16, backend), Tensor.from_host(b, b.shape, DType.BF16, backend)
    for kernel in ("simt", "tcgen05"):
        set_kernel(backend, kernel)
        for aligned in (True, False):
            g = Guarded(backend, (192, 160), DType.BF16, "window", aligned)  # the parent, itself inside guard bands
            for r0, r1 in ((0, 64), (64, 192)):
                backend.matmul_into(ta.narrow(0, r0, r1 - r0), tb, g.view.narrow(0, r0, r1 - r0), batched=False)
            assert rel_err(to_f64(g.result(), DType.BF16), oracle_ref(oracle, a, b, DType.BF16)) <= 1e-2
        # a transposed output view (column stride != 1)
        g = Guarded(backend, (160, 192), DType.BF16, "window")
        backend.matmul_into(ta, tb, g.view.permute([1, 0]), batched=False)
        assert rel_err(to_f64(g.result().T, DType.BF16), oracle_ref(oracle, a, b, DType.BF16)) <= 1e-2


def test_host_entry_point(backend, oracle):
    a = fill(oracle, (3, 1, 130, 70), DType.F32, 71, 0)
    b = fill(oracle, (1, 2, 70, 90), DType.F32, 71, 1)
    av = a.transpose(0, 1, 3, 2).copy().transpose(0, 1, 3, 2)  # M-major host view
    got = backend.matmul_host(av, b, DType.F32)
    assert rel_err(got, oracle_ref(oracle, av, b, DType.F32)) <= 1e-4
    a16, b16 = fill(oracle, (200, 136), DType.BF16, 72, 0), fill(oracle, (136, 264), DType.BF16, 72, 1)
    got = backend.matmul_host(a16, b16, DType.BF16)
    assert rel_err(to_f64(got, DType.BF16), oracle_ref(oracle, a16, b16, DType.BF16)) <= 1e-2


def test_host_entry_point_pipeline_matches_the_single_shot(backend, oracle):
    """Outputs of 16 MiB or more go through the sliced copy/compute pipeline;
    slicing must not change a bit, for rank-2 and for batched products, with
    K-major, M-major and broadcast operands."""
    cases = [((4096, 1040), False, (1040, 2064)),          # rank 2, rows sliced
             ((1040, 4096), True, (1040, 2064)),           # A is M-major: copied whole, still sliced as a view
             ((6, 640, 520), False, (520, 2304)),          # batch sliced, B shared
             ((5, 1, 640, 520), False, (1, 3, 520, 776))]  # leading batch dim sliced, B broadcast over it
    for i, (ashape, a_t, bshape) in enumerate(cases):
        a, b = fill(oracle, ashape, DType.BF16, 300 + i, 0), fill(oracle, bshape, DType.BF16, 300 + i, 1)
        av = a.T if a_t else a
        outs = []
        for chunks in (1, 0, 3):
            backend.set_option("host_chunks", chunks)
            outs.append(backend.matmul_host(av, b, DType.BF16))
        backend.set_option("host_chunks", 0)
        assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[0], outs[2]), (ashape, bshape)
        sample = (slice(0, 40),) if len(outs[0].shape) == 2 else (0,) * (len(outs[0].shape) - 2)
        a_s = av[:40] if len(outs[0].shape) == 2 else av[(0,) * (av.ndim - 2)]
        b_s = b if b.ndim == 2 else b[(0,) * (b.ndim - 2)]
        assert rel_err(to_f64(outs[0][sample], DType.BF16), oracle_ref(oracle, a_s, b_s, DType.BF16)) <= 1e-2


def test_concurrent_callers_share_one_context(backend, oracle):
    """`Backend: Send + Sync`: eight host threads issue products of different
    shapes, dtypes and kernels through the same context at once."""
    import threading
    shapes = [(300, 200, 520), (64, 64, 64), (129, 257, 2100), (520, 1100, 136), (77, 33, 1000), (256, 384, 512),
              (1, 300, 40), (130, 70, 520)]
    errors, results = [], {}

    def work(i):
        try:
            m, k, n = shapes[i]
            dtype = (DType.BF16, DType.F32, DType.F16)[i % 3]
            a, b = fill(oracle, (m, k), dtype, 400 + i, 0), fill(oracle, (n, k), dtype, 400 + i, 1)
            ta = Tensor.from_host(a, a.shape, dtype, backend)
            tb = Tensor.from_host(b, b.shape, dtype, backend).permute([1, 0])
            for _ in range(5):
                got = backend.matmul(ta, tb).to_host()
            results[i] = rel_err(to_f64(got, dtype), oracle_ref(oracle, a, b.T, dtype)) <= TOL[dtype]
        except BaseException as e:
            errors.append(e)

    threads = [threading.Thread(target=work, args=(i,)) for i in range(len(shapes))]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    assert all(results.get(i) for i in range(len(shapes))), results


def test_sharded_host_matmul_across_devices(backend, oracle):
    """One backend per visible GPU, one host thread each (needs two or more GPUs)."""
    import ctypes as C
    from oxmera_b200 import capi
    n = C.c_int(0)
    capi.load().oxm_device_count(C.byref(n))
    if n.value < 2:
        pytest.skip("one GPU visible")
    world = min(n.value, 4)
    backends = [backend] + [ox.B200Backend(i) for i in range(1, world)]
    try:
        a = fill(oracle, (world * 2, 300, 264), DType.BF16, 83, 0)
        b = fill(oracle, (264, 520), DType.BF16, 83, 1)
        assert np.array_equal(ox.sharded_matmul_host(backends, a, b, DType.BF16), backend.matmul_host(a, b, DType.BF16))
        rows = fill(oracle, (1024, 264), DType.BF16, 84, 0)
        assert np.array_equal(ox.sharded_matmul_host(backends, rows, b, DType.BF16), backend.matmul_host(rows, b, DType.BF16))
    finally:
        for be in backends[1:]:
            be.close()


def test_sharded_host_matmul_matches_single_device(backend, oracle):
    """The collective-free sharding driver, with two shards on one device.
    Bit equality of shards and whole is promised for one accumulation chain
    per output element ("split_k" 0): products this small run on the FFMA
    kernel, which otherwise cuts the contraction over a cluster whose size
    follows the tile count, i.e. the shard's size."""
    a = fill(oracle, (4, 96, 64), DType.BF16, 81, 0)
    b = fill(oracle, (64, 80), DType.BF16, 81, 1)
    backend.set_option("split_k", 0)
    try:
        whole = backend.matmul_host(a, b, DType.BF16)
        parts = ox.sharded_matmul_host([backend, backend], a, b, DType.BF16)
        assert np.array_equal(whole, parts)
        rows = ox.sharded_matmul_host([backend, backend], a[0], b, DType.BF16)
        assert np.array_equal(whole[0], rows)
    finally:
        backend.set_option("split_k", -1)
    # with the automatic split the two may differ in the last place, no more
    auto = ox.sharded_matmul_host([backend, backend], a, b, DType.BF16)
    assert rel_err(to_f64(auto, DType.BF16), to_f64(whole, DType.BF16)) <= 2.0 ** -7
