"""Replica plumbing for multi-GPU runs: one process per GPU, no data-path collective.

The path does not exchange data between GPUs (the reference shards whole tasks over GPUs by
process, scripts/bench_parallel.py:2432-2444); the only things ranks agree on are *when* the timed
region starts and ends and *how long the slowest of them took*. ``ReplicaGroup`` wraps exactly
that on top of ``torch.distributed``: NCCL on GPUs, gloo for CPU tests.
"""
from __future__ import annotations

import os


def dist_env():
    """(rank, local_rank, world_size) from the launcher's environment; (0, 0, 1) outside one."""
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")),
            int(os.environ.get("WORLD_SIZE", "1")))


class ReplicaGroup:
    """Barrier and max-over-ranks for N independent replicas.

    With world_size 1 nothing is initialised and every operation is local. ``device`` is the
    torch device the reductions run on (the rank's GPU under NCCL, the CPU under gloo).
    """

    def __init__(self, backend: str | None = None, device=None):
        import torch
        self.rank, self.local_rank, self.world = dist_env()
        self.device = device if device is not None else torch.device("cpu")
        self._dist = None
        if self.world > 1:
            import torch.distributed as dist
            backend = backend or ("nccl" if self.device.type == "cuda" else "gloo")
            if not dist.is_initialized():
                kwargs = {"device_id": self.device} if backend == "nccl" else {}
                dist.init_process_group(backend, **kwargs)
            self._dist = dist

    def barrier(self) -> None:
        if self._dist is not None:
            self._dist.barrier()

    def max_over_ranks(self, value: float) -> float:
        """The largest ``value`` any rank holds (a duration: the job is as slow as its slowest rank)."""
        if self._dist is None:
            return float(value)
        import torch
        t = torch.tensor([float(value)], dtype=torch.float64, device=self.device)
        self._dist.all_reduce(t, op=self._dist.ReduceOp.MAX)
        return float(t.item())

    def job_throughput(self, units_per_rank: float, seconds_this_rank: float) -> float:
        """Whole-job units per second: what all ranks processed divided by the slowest rank's time."""
        slowest = self.max_over_ranks(seconds_this_rank)
        return units_per_rank * self.world / slowest

    def is_reporter(self) -> bool:
        return self.rank == 0

    def close(self) -> None:
        if self._dist is not None and self._dist.is_initialized():
            self._dist.barrier()
            self._dist.destroy_process_group()
            self._dist = None
