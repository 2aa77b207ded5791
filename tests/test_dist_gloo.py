"""The N > 1 path on CPU: two gloo ranks shard each workload the way
`bench.py --gpus 2` does, multiply their shards (the CPU oracle stands in for
the device), and the shards tile the unsharded result; the step time reported
for the job is the slowest rank's."""
import os
import socket
import sys

import numpy as np
import pytest
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import oxmera_b200 as ox
    from oxmera_b200.dist import init_from_env
    from oxmera_b200.workloads import WORKLOADS, gemm_views, materialise, scaled, shard_flops
    from tests.oracle_lib import ACC_F64, Oracle
    from tests.test_gpu_parity import TAG
    from tests.test_host_mirror import HostStandIn

    grp = init_from_env("gloo")
    assert (grp.rank, grp.world) == (rank, world)
    oracle, be = Oracle(), HostStandIn()
    grp.barrier()
    # the job's step time is the slowest rank's
    assert grp.max_over_ranks(10.0 + rank) == 10.0 + world - 1
    assert grp.min_over_ranks(10.0 + rank) == 10.0
    for key, factor in (("c3", 32), ("c4", 32), ("c5", 32), ("c2", 8)):
        w = scaled(WORKLOADS[key], factor)
        fill = lambda spec, dtype, seed: ox.Tensor.from_host(
            oracle.fill(spec.shape, TAG[dtype], seed, spec.stream, spec.dist, spec.scale), spec.shape, dtype, be)
        tensors = materialise(w, fill)  # every rank draws the same seeded inputs
        total = 0
        for gi, g in enumerate(w.gemms):
            a, b, rg = gemm_views(w, g, tensors, rank, world)
            st, part = oracle.matmul(a.to_host(), b.to_host(), TAG[w.dtype], acc=ACC_F64, nthreads=1)
            assert st == 0
            np.save(os.path.join(out_dir, f"{key}_{gi}_rank{rank}.npy"), part)
            if rank == 0:
                fa, fb, _ = gemm_views(w, g, tensors)
                st, whole = oracle.matmul(fa.to_host(), fb.to_host(), TAG[w.dtype], acc=ACC_F64, nthreads=1)
                np.save(os.path.join(out_dir, f"{key}_{gi}_whole.npy"), whole)
        # the ranks' flop shares add up to the workload's
        share = shard_flops(w, rank, world)
        import torch
        import torch.distributed as dist
        t = torch.tensor([float(share)], dtype=torch.float64)
        dist.all_reduce(t)
        assert int(t.item()) == w.flops(), (key, int(t.item()), w.flops())
    grp.barrier()
    grp.close()


@pytest.mark.timeout(300)
def test_two_gloo_ranks_tile_the_unsharded_result(tmp_path):
    world = 2
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    from oxmera_b200.workloads import WORKLOADS, shard_axis
    for key in ("c3", "c4", "c5", "c2"):
        for gi, g in enumerate(WORKLOADS[key].gemms):
            whole = np.load(tmp_path / f"{key}_{gi}_whole.npy")
            parts = [np.load(tmp_path / f"{key}_{gi}_rank{r}.npy") for r in range(world)]
            assert np.array_equal(np.concatenate(parts, axis=shard_axis(WORKLOADS[key], g)), whole), (key, g.name)


def test_shard_ranges_and_plan():
    import oxmera_b200 as ox
    assert [len(r) for r in ox.shard_ranges(10, 4)] == [3, 3, 2, 2]
    assert [r.start for r in ox.shard_ranges(8192, 8)] == [i * 1024 for i in range(8)]
    assert ox.shard_ranges(3, 4)[-1] == range(3, 3)  # more ranks than units: the last rank idles
    assert ox.shard_plan((32, 2048, 4096), (4096, 11008), 8)[0] == "batch"
    assert ox.shard_plan((8192, 8192), (8192, 8192), 8)[0] == "rows"
    assert ox.shard_plan((2, 64, 32), (32, 48), 4)[0] == "rows"  # fewer batch entries than ranks


def test_a_failing_shard_surfaces_as_the_callers_error():
    """One host thread per device; a shard that fails (here: a device whose
    backend raises) must end the whole call with that typed error, not a hang
    and not a partial result."""
    import numpy as np
    import oxmera_b200 as ox

    class Healthy:
        def matmul_host(self, a, b, dtype, out=None):
            return np.matmul(a.astype(np.float32), b.astype(np.float32))

    class Broken:
        def matmul_host(self, a, b, dtype, out=None):
            raise ox.BackendFault(10, "matmul: CudaError: injected on the host")

    a, b = np.ones((4, 8, 16), np.float32), np.ones((16, 8), np.float32)
    got = ox.sharded_matmul_host([Healthy(), Healthy()], a, b, ox.DType.F32)
    assert got.shape == (4, 8, 8) and np.all(got == 16.0)
    with pytest.raises(ox.BackendFault) as e:
        ox.sharded_matmul_host([Healthy(), Broken(), Healthy()], a, b, ox.DType.F32)
    assert "injected" in str(e.value)
    with pytest.raises(ox.BroadcastIncompatible):  # a typed error raised before any shard starts
        ox.sharded_matmul_host([Healthy()], np.ones((2, 3, 4, 5), np.float32), np.ones((3, 1, 5, 6), np.float32), ox.DType.F32)
