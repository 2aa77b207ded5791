"""The host-side planner (oxm_plan_matmul): which kernel, tile width, CTA
pairing, split-K factor and operand staging a product gets on a 148-SM GPU.
Runs without a GPU: the views only carry shapes, strides and an aligned dummy
address."""
import ctypes as C

import pytest

from oxmera_b200 import DType, capi
from oxmera_b200.core import contiguous_strides

BASE = 0x10000000  # 256-byte aligned, never dereferenced
FFMA, TCGEN05 = 1, 2


def view(dtype, shape, strides=None, offset=0):
    return capi.make_view(int(dtype), shape, strides or contiguous_strides(shape), offset, BASE, 0)


def t(v):
    """The view with its last two dims swapped."""
    n = v.ndim
    shape, strides = list(v.shape[:n]), list(v.strides[:n])
    shape[-1], shape[-2] = shape[-2], shape[-1]
    strides[-1], strides[-2] = strides[-2], strides[-1]
    return capi.make_view(v.dtype, shape, strides, v.offset, BASE, 0)


def plan(a, b, out_dtype=None, sms=148):
    lead = []
    la, lb = list(a.shape[:a.ndim - 2]), list(b.shape[:b.ndim - 2])
    for i in range(max(len(la), len(lb))):
        x = la[len(la) - 1 - i] if i < len(la) else 1
        y = lb[len(lb) - 1 - i] if i < len(lb) else 1
        lead.insert(0, max(x, y))
    out = view(out_dtype if out_dtype is not None else a.dtype, lead + [a.shape[a.ndim - 2], b.shape[b.ndim - 1]])
    res = (C.c_int32 * 8)()
    st = capi.load().oxm_plan_matmul(C.byref(a), C.byref(b), C.byref(out), sms, res)
    return st, dict(kernel=res[0], tile_n=res[1], pair=res[2], splits=res[3], pack_a=res[4], pack_b=res[5], stream_k=res[6])


def test_the_five_configurations():
    bf, f32 = DType.BF16, DType.F32
    # c3: square, B column-major -> the widest pair tile (512 tiles = 6.92 waves of 74 pairs), operands read in place
    st, p = plan(view(bf, [8192, 8192]), t(view(bf, [8192, 8192])))
    assert st == 0 and {k: p[k] for k in ('kernel', 'tile_n', 'pair', 'splits', 'pack_a', 'pack_b')} == dict(kernel=TCGEN05, tile_n=512, pair=1, splits=1, pack_a=0, pack_b=0)
    # c4: 32 x [2048, 4096] . [4096, 11008]: 11008 is 43 tiles of 256 but 21.5 of 512, and W is N-major, so no
    # narrower width of the wide tile would load less: 256 x 256 pairs
    st, p = plan(view(bf, [32, 2048, 4096]), view(bf, [4096, 11008]))
    assert st == 0 and (p["kernel"], p["tile_n"], p["pair"], p["splits"], p["pack_a"], p["pack_b"]) == (TCGEN05, 256, 1, 1, 0, 0)
    # c5: forward and input gradient are 512 wide tiles; the weight gradient dY^T . X has both operands
    # M- / N-major views and 128 tiles: the wide tile, the last tiles shared out by contraction block
    st, p = plan(view(bf, [16384, 4096]), t(view(bf, [4096, 4096])))
    assert st == 0 and (p["tile_n"], p["pair"], p["stream_k"]) == (512, 1, 0)
    st, p = plan(t(view(bf, [16384, 4096])), view(bf, [16384, 4096]))
    assert st == 0 and p["kernel"] == TCGEN05 and (p["tile_n"], p["pair"], p["splits"]) == (512, 1, 1) and p["pack_a"] == p["pack_b"] == 0
    # c2: f32 goes through the TF32 split, which always packs; K = 1024 is one accumulation chain
    st, p = plan(t(view(f32, [8, 1, 1024, 512])), view(f32, [1, 16, 1024, 768]))
    assert st == 0 and {k: p[k] for k in ('kernel', 'pair', 'splits', 'pack_a', 'pack_b')} == dict(kernel=TCGEN05, pair=1, splits=1, pack_a=1, pack_b=1)
    assert p["tile_n"] == 384  # 768 columns are two tiles of 384: no half-empty tile as with 512
    # c1: a small f32 product: one launch of the FFMA kernel (its contraction split over a cluster)
    st, p = plan(view(f32, [256, 512]), view(f32, [512, 384]))
    assert st == 0 and p["kernel"] == FFMA


def test_the_shards_of_an_8_gpu_run():
    """The M-row shards of c3 and the batch shards of c4: tile widths that are
    not powers of two fit the 74 CTA pairs where 512 columns leave a tenth of
    them idle."""
    bf = DType.BF16
    b = t(view(bf, [8192, 8192]))
    # 1024 rows: 4 x 16 tiles of 512 use 64 of 74 pairs; 4 x 18 tiles of 480 use 72, each 6 % shorter
    st, p = plan(view(bf, [1024, 8192]), b)
    assert st == 0 and (p["tile_n"], p["pair"], p["splits"], p["stream_k"]) == (480, 1, 1, 0)
    # 2048 rows: 8 x 18 = 144 tiles of 480 are two nearly full waves
    st, p = plan(view(bf, [2048, 8192]), b)
    assert st == 0 and (p["tile_n"], p["pair"], p["splits"]) == (480, 1, 1)
    # 4096 rows: 512 tiles of 256 x 256 are 6.92 waves, as for the whole product with the wide tile
    st, p = plan(view(bf, [4096, 8192]), b)
    assert st == 0 and (p["tile_n"], p["pair"], p["splits"]) == (256, 1, 1)
    # c4 on 8 GPUs: 4 batch entries per GPU
    st, p = plan(view(bf, [4, 2048, 4096]), view(bf, [4096, 11008]))
    assert st == 0 and (p["tile_n"], p["pair"], p["splits"]) == (256, 1, 1)
    # any multiple of 32 columns can be forced; an N-major B never gets a narrowed wide tile on its own
    for n in (2048, 3000, 11008):
        st, p = plan(view(bf, [4096, 4096]), view(bf, [4096, n]))
        assert st == 0 and p["tile_n"] in (64, 128, 256, 512), (n, p)


def test_long_f32_contractions_are_cut_into_chains():
    st, p = plan(view(DType.F32, [2048, 8192]), view(DType.F32, [8192, 2048]))
    assert st == 0 and p["splits"] >= 8  # at most 1024 elements of K per fp32 accumulation chain


def test_skinny_and_short_products():
    bf = DType.BF16
    # a decode step: one row of tiles over a long weight matrix -> wide tiles, contraction split to fill the SMs
    for m in (1, 16, 128):
        st, p = plan(view(bf, [m, 8192]), t(view(bf, [8192, 8192])))
        assert st == 0 and p["kernel"] == TCGEN05 and p["pair"] == 0 and p["splits"] > 1, (m, p)
        assert p["tile_n"] >= 128 and p["tile_n"] * p["splits"] >= 256, (m, p)
    # a tiny output with a huge contraction
    st, p = plan(view(bf, [128, 262144]), t(view(bf, [128, 262144])))
    assert st == 0 and p["splits"] >= 32
    # two contraction blocks per tile: the epilogue decides; one CTA per tile drains fastest
    st, p = plan(view(bf, [8192, 128]), t(view(bf, [8192, 128])))
    assert st == 0 and (p["tile_n"], p["pair"], p["splits"]) == (256, 0, 1)
    # under the crossover: the FFMA kernel
    st, p = plan(view(bf, [64, 64]), view(bf, [64, 64]))
    assert st == 0 and p["kernel"] == FFMA
    st, p = plan(view(DType.F32, [128, 128]), view(DType.F32, [128, 128]))
    assert st == 0 and p["kernel"] == FFMA


def test_staging_decisions():
    bf = DType.BF16
    # a window whose rows start on odd addresses cannot be described to the TMA engine
    a = capi.make_view(int(bf), [512, 1024], [1027, 1], 3, BASE, 0)
    st, p = plan(a, view(bf, [1024, 512]))
    assert st == 0 and p["pack_a"] == 1 and p["pack_b"] == 0
    # inner stride 2 on both dims of B
    b = capi.make_view(int(bf), [1024, 512], [1024, 2], 0, BASE, 0)
    st, p = plan(view(bf, [512, 1024]), b)
    assert st == 0 and p["pack_b"] == 1
    # an N-major fp8 B is staged in boxes of 128 columns: no tile narrower than that
    f8 = DType.F8E4M3
    st, p = plan(view(f8, [256, 4096]), view(f8, [4096, 192]), out_dtype=DType.BF16)
    assert st == 0 and p["kernel"] == TCGEN05 and (p["tile_n"] // (2 if p["pair"] else 1)) >= 128


def test_planner_validates_like_the_product():
    bf = DType.BF16
    st, _ = plan(view(bf, [4, 5]), view(bf, [6, 7]))
    assert st == capi.SHAPE_MISMATCH if hasattr(capi, "SHAPE_MISMATCH") else st == 1
    st, _ = plan(view(bf, [4, 5]), view(DType.F16, [5, 7]))
    assert st == 3  # DTypeMismatch
    st, p = plan(view(bf, [0, 5]), view(bf, [5, 7]))
    assert st == 0 and p["kernel"] == 0
    res = (C.c_int32 * 8)()
    a = view(bf, [4, 4])
    assert capi.load().oxm_plan_matmul(C.byref(a), C.byref(a), C.byref(a), 1, res) == 12  # InvalidArgument


def test_stream_k_only_beside_whole_waves():
    bf = DType.BF16
    # 512 tiles on 74 pairs = 6.92 waves: too little to gain
    _, p = plan(view(bf, [8192, 8192]), t(view(bf, [8192, 8192])))
    assert p["stream_k"] == 0
    # the 8-GPU shard of the same product: all of its tiles would be shared out
    _, p = plan(view(bf, [1024, 8192]), t(view(bf, [8192, 8192])))
    assert p["stream_k"] == 0
    # the linear layer's weight gradient: 128 tiles of 256 x 512 = one wave and 54 more
    _, p = plan(t(view(bf, [16384, 4096])), view(bf, [16384, 4096]))
    assert (p["tile_n"], p["stream_k"]) == (512, 54)
    # long f32 contractions are cut into chains instead
    _, p = plan(view(DType.F32, [4096, 4096]), view(DType.F32, [4096, 4096]))
    assert p["splits"] > 1 and p["stream_k"] == 0
