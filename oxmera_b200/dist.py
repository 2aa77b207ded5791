"""Process-group plumbing for the one-process-per-GPU benchmark.

The matmul path shards with no exchange step, so the only things ranks ever
say to each other are "everyone is ready" and "how long did the slowest of us
take".  `torch.distributed` carries both: NCCL on GPUs, gloo in CPU tests.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional


@dataclass
class Group:
    rank: int = 0
    world: int = 1
    local_rank: int = 0
    backend: Optional[str] = None  # None: single process, nothing initialised

    def _tensor(self, value: float):
        import torch
        dev = f"cuda:{self.local_rank}" if self.backend == "nccl" else "cpu"
        return torch.tensor([value], dtype=torch.float64, device=dev)

    def barrier(self) -> None:
        """All ranks have reached this point (and, on GPUs, their queued work
        up to the all-reduce has drained)."""
        if self.backend is None:
            return
        import torch
        import torch.distributed as dist
        t = self._tensor(0.0)
        dist.all_reduce(t)
        if self.backend == "nccl":
            torch.cuda.synchronize(self.local_rank)

    def max_over_ranks(self, value: float) -> float:
        if self.backend is None:
            return value
        import torch.distributed as dist
        t = self._tensor(value)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def min_over_ranks(self, value: float) -> float:
        return -self.max_over_ranks(-value)

    def close(self) -> None:
        if self.backend is not None:
            import torch.distributed as dist
            dist.destroy_process_group()
            self.backend = None


def init_from_env(backend: str = "nccl") -> Group:
    """Join the group the launcher described in RANK / LOCAL_RANK / WORLD_SIZE /
    MASTER_ADDR / MASTER_PORT; a lone process gets a trivial group."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world <= 1:
        return Group()
    import torch
    import torch.distributed as dist
    rank = int(os.environ["RANK"])
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if backend == "nccl":
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        dist.init_process_group(backend)
    return Group(rank, world, local, backend)
