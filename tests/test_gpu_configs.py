"""The five benchmark configurations at their full sizes, on a B200.

At these sizes the CPU oracle cannot produce the whole result in seconds, so
each product is checked three ways:
  1. sampled output rows (tile corners, tile boundaries, random rows) against
     the oracle on the same inputs, to the stated tolerance;
  2. two size-independent checksums over the WHOLE output: C.1 against
     A.(B.1) and 1^T.C against (1^T.A).B, evaluated in float64 — any tile that
     was skipped, misplaced or filled with the wrong operand shows up here;
  3. scaled-down versions of the same workloads against the full oracle result.
Inputs come from the oracle's seeded generator, so both sides see identical bits.
"""
import itertools

import numpy as np
import pytest

import oxmera_b200 as ox
from oxmera_b200 import DType, Tensor
from oxmera_b200.workloads import WORKLOADS, gemm_views, materialise, scaled, shard_axis
from tests.test_gpu_parity import TAG, TOL, oracle_ref, rel_err, to_f64

pytestmark = pytest.mark.gpu


def host_fill(oracle, backend, host_store):
    def fill(spec, dtype, seed):
        h = oracle.fill(spec.shape, TAG[dtype], seed, spec.stream, spec.dist, spec.scale)
        host_store[spec.name] = h
        return Tensor.from_host(h, spec.shape, dtype, backend)
    return fill


def host_view(host, name, perm):
    h = host[name]
    return h.transpose(perm) if perm else h


def sample_rows(m, count, tile=128, seed=0):
    rows = {0, m - 1}
    for edge in (tile - 1, tile, 2 * tile - 1, 2 * tile, m - tile, m - tile - 1, m // 2):
        if 0 <= edge < m:
            rows.add(edge)
    rng = np.random.default_rng(seed)
    while len(rows) < min(count, m):
        rows.add(int(rng.integers(0, m)))
    return sorted(rows)


def check_product(backend, oracle, w, g, host, dev, rows_per_batch, max_batches):
    dtype, tol = w.dtype, TOL[w.dtype]
    a, b, _ = gemm_views(w, g, dev)
    out = backend.batched_matmul(a, b) if len(a.shape) > 2 or len(b.shape) > 2 else backend.matmul(a, b)
    ha, hb = host_view(host, g.a, g.a_perm), host_view(host, g.b, g.b_perm)
    ho = out.to_host()
    lead = ho.shape[:-2]
    m, n, k = ho.shape[-2], ho.shape[-1], ha.shape[-1]
    bidx_all = list(itertools.product(*[range(d) for d in lead])) or [()]

    def pick(full, bi):
        """Index of `full`'s own batch entry for output batch index `bi` (broadcast dims -> 0)."""
        nb = full.ndim - 2
        return tuple(0 if full.shape[j] == 1 else bi[len(lead) - nb + j] for j in range(nb))

    # 1. sampled rows against the oracle
    rng = np.random.default_rng(w.seed)
    chosen = bidx_all if len(bidx_all) <= max_batches else [bidx_all[i] for i in sorted(
        {0, len(bidx_all) - 1, *rng.choice(len(bidx_all), max_batches - 2, replace=False).tolist()})]
    worst = 0.0
    for bi in chosen:
        rows = sample_rows(m, rows_per_batch, seed=sum(bi))
        a_rows = np.ascontiguousarray(ha[pick(ha, bi)][rows])
        ref = oracle_ref(oracle, a_rows, hb[pick(hb, bi)], dtype)
        worst = max(worst, rel_err(to_f64(ho[bi][rows], dtype), ref))
    assert worst <= tol, (w.key, g.name, "sampled rows", worst, backend.last_kernel())
    print(f"parity {w.key}/{g.name}: sampled-row error {worst:.3e} (tolerance {tol:g}) {backend.last_kernel()}")
    # 2. whole-output checksums in float64.  bf16/f16 results carry an unbiased
    # rounding of 2^-9 per stored element, which sums like sqrt(n).  The f32
    # tensor-core path accumulates with truncation, a bias that sums like n;
    # allow a tenth of the elementwise tolerance per element.
    def budget(count, rms):
        if dtype == DType.F32:
            return 1e-5 * rms * count + 1e-9
        return 6 * 2.0 ** -8 * rms * np.sqrt(count) + 1e-9

    b_cache = {}
    for bi in bidx_all:
        pb = pick(hb, bi)
        if pb not in b_cache:
            b_cache.clear()
            b_cache[pb] = to_f64(hb[pb], dtype)
        A, B, Cm = to_f64(ha[pick(ha, bi)], dtype), b_cache[pb], to_f64(ho[bi], dtype)
        rms = float(np.sqrt(np.mean(Cm * Cm)))
        row_sum, row_ref = Cm.sum(axis=1), A @ B.sum(axis=1)
        col_sum, col_ref = Cm.sum(axis=0), A.sum(axis=0) @ B
        assert np.max(np.abs(row_sum - row_ref)) <= budget(n, rms), (w.key, g.name, bi, "C.1")
        assert np.max(np.abs(col_sum - col_ref)) <= budget(m, rms), (w.key, g.name, bi, "1^T.C")
    return out


@pytest.mark.parametrize("key", ["c1", "c2", "c3", "c4", "c5"])
def test_config_at_full_size(backend, oracle, key):
    w = WORKLOADS[key]
    host = {}
    dev = materialise(w, host_fill(oracle, backend, host))
    for g in w.gemms:
        out = check_product(backend, oracle, w, g, host, dev, rows_per_batch=24 if key != "c1" else 256,
                            max_batches=6)
        if key == "c1":
            # small enough for the whole result
            ref = oracle_ref(oracle, host["A"], host["B"], w.dtype)
            assert rel_err(out.to_host(), ref) <= TOL[w.dtype]
        else:
            assert "tcgen05" in backend.last_kernel()
        del out


@pytest.mark.parametrize("key,factor", [("c2", 4), ("c3", 16), ("c4", 16), ("c5", 16)])
@pytest.mark.parametrize("pair", [0, 1])
def test_scaled_configs_against_the_full_oracle_result(backend, oracle, key, factor, pair):
    w = scaled(WORKLOADS[key], factor)
    backend.set_option("kernel", 2)
    backend.set_option("cta_pair", pair)
    try:
        host = {}
        dev = materialise(w, host_fill(oracle, backend, host))
        for g in w.gemms:
            a, b, _ = gemm_views(w, g, dev)
            out = backend.batched_matmul(a, b)
            ref = oracle_ref(oracle, host_view(host, g.a, g.a_perm), host_view(host, g.b, g.b_perm), w.dtype)
            err = rel_err(to_f64(out.to_host(), w.dtype), ref)
            assert err <= TOL[w.dtype], (w.key, g.name, err, backend.last_kernel())
    finally:
        backend.set_option("kernel", 0)
        backend.set_option("cta_pair", -1)


@pytest.mark.parametrize("key", ["c3", "c4", "c5", "c2"])
def test_shards_reassemble_to_the_whole(backend, oracle, key):
    """Collective-free sharding: the shards of each product, computed as the
    ranks of a 1/2/4-GPU run would, tile the unsharded result bit for bit."""
    w = scaled(WORKLOADS[key], 8)
    host = {}
    dev = materialise(w, host_fill(oracle, backend, host))
    backend.set_option("kernel", 2)
    backend.set_option("split_k", 0)  # one accumulation chain per element, whatever the shard's shape
    try:
        for g in w.gemms:
            a, b, _ = gemm_views(w, g, dev)
            whole = backend.batched_matmul(a, b).to_host()
            for world in (2, 4):
                parts = []
                for rank in range(world):
                    sa, sb, rg = gemm_views(w, g, dev, rank, world)
                    parts.append(backend.batched_matmul(sa, sb).to_host())
                assert np.array_equal(np.concatenate(parts, axis=shard_axis(w, g)), whole), (w.key, g.name, world)
    finally:
        backend.set_option("kernel", 0)
        backend.set_option("split_k", -1)
