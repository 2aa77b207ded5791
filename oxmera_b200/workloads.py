"""The five benchmark configurations of the matmul path, as data.

Each workload names its base tensors (shape, distribution, seed stream), the
products formed from VIEWS of them (transposes are permutes, never copies), the
flop and algorithmic-byte counts, and how it splits across the GPUs of one box
with no exchange step.  Inputs are seeded synthetic data; whoever runs the
workload supplies the generator (the tests fill on the host with the oracle's
generator so both sides see identical bits, the benchmark fills on the device).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

from .core import DType, broadcast_shapes, numel
from .tensor import Tensor


@dataclass(frozen=True)
class TensorSpec:
    name: str
    shape: Tuple[int, ...]
    dist: str      # "uniform" = U(-1,1), "normal" = N(0,1) * scale
    scale: float
    stream: int    # tensors are drawn in stream order from the workload's seed


@dataclass(frozen=True)
class GemmSpec:
    name: str
    a: str                      # base tensor name
    a_perm: Optional[Tuple[int, ...]]
    b: str
    b_perm: Optional[Tuple[int, ...]]
    # The dim of A's BASE tensor (before a_perm) that shards across GPUs: a
    # batch dim, or the dim that becomes the M rows.  K never shards.  When A
    # has extent 1 there (it broadcasts over that batch dim) only B is cut.
    shard_dim: int
    shard_b_dim: Optional[int] = None  # B's matching base dim when B carries the same batch dim


@dataclass(frozen=True)
class Workload:
    key: str
    title: str
    dtype: DType
    seed: int
    tensors: Tuple[TensorSpec, ...]
    gemms: Tuple[GemmSpec, ...]
    out_dtype: Optional[DType] = None  # fp8 products may be kept wider than their operands
    mx: bool = False  # block-scaled: every base tensor (contraction dim last) comes with E8M0 scales, one per 32 of K

    @property
    def result_dtype(self) -> DType:
        return self.dtype if self.out_dtype is None else self.out_dtype

    def spec(self, name: str) -> TensorSpec:
        return next(t for t in self.tensors if t.name == name)

    def _view_shape(self, name: str, perm) -> Tuple[int, ...]:
        s = self.spec(name).shape
        return tuple(s[p] for p in perm) if perm else s

    def gemm_shapes(self, g: GemmSpec):
        a, b = self._view_shape(g.a, g.a_perm), self._view_shape(g.b, g.b_perm)
        lead = broadcast_shapes(a[:-2], b[:-2])
        return a, b, tuple(lead) + (a[-2], b[-1])

    def flops(self) -> int:
        total = 0
        for g in self.gemms:
            a, b, o = self.gemm_shapes(g)
            total += 2 * numel(o) * a[-1]
        return total

    def algorithmic_bytes(self) -> int:
        """Every unique operand element read once, every output element written once."""
        esz, osz = self.dtype.size_in_bytes(), self.result_dtype.size_in_bytes()
        total = 0
        for g in self.gemms:
            a, b, o = self.gemm_shapes(g)
            total += (numel(a) + numel(b)) * esz + numel(o) * osz
        return total


def _t(name, shape, dist, scale, stream):
    return TensorSpec(name, tuple(shape), dist, scale, stream)


WORKLOADS: Dict[str, Workload] = {
    "c1": Workload(
        "c1", "f32 256x512 . 512x384, row-major, U(-1,1), seed 0", DType.F32, 0,
        (_t("A", (256, 512), "uniform", 1.0, 0), _t("B", (512, 384), "uniform", 1.0, 1)),
        (GemmSpec("C", "A", None, "B", None, 0),)),
    "c2": Workload(
        "c2", "f32 broadcast-batched: [8,1,1024,512] transposed view . [1,16,1024,768] -> [8,16,512,768], N(0,1)/32, seed 1",
        DType.F32, 1,
        (_t("T", (8, 1, 1024, 512), "normal", 1.0 / 32.0, 0), _t("B", (1, 16, 1024, 768), "normal", 1.0 / 32.0, 1)),
        # of the two batch dims the second is cut: every GPU then needs all of T (16 MiB) and 1/N of B
        # (48 MiB in all) rather than 1/N of T and all of B
        (GemmSpec("C", "T", (0, 1, 3, 2), "B", None, 1, 1),)),
    "c3": Workload(
        "c3", "bf16 8192^3, A row-major, B column-major, N(0,1)/sqrt(8192), fp32 accumulate, bf16 out, seed 2",
        DType.BF16, 2,
        (_t("A", (8192, 8192), "normal", 8192 ** -0.5, 0), _t("Bt", (8192, 8192), "normal", 8192 ** -0.5, 1)),
        (GemmSpec("C", "A", None, "Bt", (1, 0), 0),)),
    "c4": Workload(
        "c4", "bf16 MLP up-projection: 32 x [2048x4096] . [4096x11008], X~N(0,1), W~N(0,0.02^2) shared, seed 3",
        DType.BF16, 3,
        (_t("X", (32, 2048, 4096), "normal", 1.0, 0), _t("W", (4096, 11008), "normal", 0.02, 1)),
        (GemmSpec("Y", "X", None, "W", None, 0),)),
    "c5": Workload(
        "c5", "bf16 linear forward+backward, tokens 16384, d_in = d_out = 4096, transposes as views, seed 4",
        DType.BF16, 4,
        (_t("X", (16384, 4096), "normal", 1.0, 0), _t("W", (4096, 4096), "normal", 0.02, 1),
         _t("dY", (16384, 4096), "normal", 1.0, 2)),
        (GemmSpec("Y", "X", None, "W", (1, 0), 0),          # Y  = X . W^T
         GemmSpec("dX", "dY", None, "W", None, 0),          # dX = dY . W
         GemmSpec("dW", "dY", (1, 0), "X", None, 1))),      # dW = dY^T . X   (rows of dY^T = columns of dY)
    # beyond the reference's configurations: the same square product at the next tensor-core rate
    "c3f8": Workload(
        "c3f8", "fp8 e4m3 8192^3, A row-major, B column-major, N(0,1), fp32 accumulate, bf16 out, seed 2",
        DType.F8E4M3, 2,
        (_t("A", (8192, 8192), "normal", 1.0, 0), _t("Bt", (8192, 8192), "normal", 1.0, 1)),
        (GemmSpec("C", "A", None, "Bt", (1, 0), 0),), DType.BF16),
}


WORKLOADS["c3mx"] = Workload(
    "c3mx", "MXFP8: fp8 e4m3 8192^3 with one E8M0 scale per 32 of K (exponents 124..130), A row-major, B column-major, "
            "N(0,1), fp32 accumulate, bf16 out, seed 2",
    DType.F8E4M3, 2,
    (_t("A", (8192, 8192), "normal", 1.0, 0), _t("Bt", (8192, 8192), "normal", 1.0, 1)),
    (GemmSpec("C", "A", None, "Bt", (1, 0), 0),), DType.BF16, mx=True)


def mx_scales(w: Workload, backend) -> Dict[str, Tensor]:
    """The E8M0 scale tensor of every base tensor of a block-scaled workload
    (shape: the tensor's with its last dim / 32), seeded, generated on the
    host: exponents 124..130, i.e. scales 1/8 .. 8."""
    import numpy as np
    out = {}
    for t in w.tensors:
        shape = tuple(t.shape[:-1]) + (t.shape[-1] // 32,)
        host = np.random.default_rng(1000 * w.seed + t.stream).integers(124, 131, size=shape, dtype=np.uint8)
        out[t.name] = Tensor.from_host(host, shape, DType.U8, backend)
    return out


def scaled(w: Workload, factor: int) -> Workload:
    """The same workload with every extent above 64 divided by `factor`
    (tests: oracle-sized versions of the large configurations)."""
    shr = lambda s: tuple(max(64, d // factor) if d > 64 else d for d in s)
    return Workload(w.key + f"/{factor}", w.title + f" (extents / {factor})", w.dtype, w.seed,
                    tuple(TensorSpec(t.name, shr(t.shape), t.dist, t.scale, t.stream) for t in w.tensors), w.gemms,
                    w.out_dtype, w.mx)


Fill = Callable[[TensorSpec, DType, int], Tensor]


def device_fill(backend) -> Fill:
    """Generate on the device (benchmarks)."""
    return lambda spec, dtype, seed: backend.synthetic(spec.shape, dtype, seed, spec.stream, spec.dist, spec.scale)


def materialise(w: Workload, fill: Fill) -> Dict[str, Tensor]:
    return {t.name: fill(t, w.dtype, w.seed) for t in w.tensors}


def gemm_views(w: Workload, g: GemmSpec, tensors: Dict[str, Tensor], rank: int = 0, world: int = 1):
    """The (A, B) views of product `g` that rank `rank` of `world` multiplies.
    Returns (a_view, b_view, row_or_batch_range)."""
    from .backend import shard_ranges
    a, b = tensors[g.a], tensors[g.b]
    total = shard_extent(g, a.shape, b.shape)
    rg = range(0, total)
    if world > 1:
        rg = shard_ranges(total, world)[rank]
        if a.shape[g.shard_dim] != 1:
            a = a.narrow(g.shard_dim, rg.start, len(rg))
        if g.shard_b_dim is not None and b.shape[g.shard_b_dim] != 1:
            b = b.narrow(g.shard_b_dim, rg.start, len(rg))
    if g.a_perm:
        a = a.permute(g.a_perm)
    if g.b_perm:
        b = b.permute(g.b_perm)
    return a, b, rg


def shard_extent(g: GemmSpec, a_shape: Sequence[int], b_shape: Sequence[int]) -> int:
    """How many units (batch entries or rows) product `g` shards over: the
    extent of the sharded dim in whichever base tensor carries it."""
    n = a_shape[g.shard_dim]
    if g.shard_b_dim is not None:
        n = max(n, b_shape[g.shard_b_dim])
    return n


def shard_axis(w: Workload, g: GemmSpec) -> int:
    """The axis of product `g`'s output along which the ranks' shards lie side by side."""
    a_shape, b_shape, o_shape = w.gemm_shapes(g)
    a_base = w.spec(g.a).shape
    if a_base[g.shard_dim] != 1 or g.shard_b_dim is None:
        pos = list(g.a_perm).index(g.shard_dim) if g.a_perm else g.shard_dim
        return pos + (len(o_shape) - len(a_shape))
    pos = list(g.b_perm).index(g.shard_b_dim) if g.b_perm else g.shard_b_dim
    return pos + (len(o_shape) - len(b_shape))


def shard_flops(w: Workload, rank: int, world: int) -> int:
    from .backend import shard_ranges
    total = 0
    for g in w.gemms:
        a, b, o = w.gemm_shapes(g)
        full = shard_extent(g, w.spec(g.a).shape, w.spec(g.b).shape)
        part = len(shard_ranges(full, world)[rank])
        total += 2 * numel(o) * a[-1] * part // full
    return total
