"""One process per GPU, independent replicas of the recipe: the only cross-rank traffic is timing.

A batch-1 action chunk (or one prefill) is not sharded: every rank holds the whole package and serves its
own episodes, as N copies of the reference runtime would.  This module is the host-side plumbing for that
mode: rank discovery from the launcher's environment, "rank 0 first" sections (in-tree builds write files
all ranks share), barriers, and the max-over-ranks reduction that turns per-rank device times into one
whole-job rate.  ``backend`` is ``nccl`` on GPUs and ``gloo`` in the CPU tests.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Callable, Sequence, TypeVar

T = TypeVar("T")


@dataclass
class ReplicaGroup:
    world: int = 1
    rank: int = 0
    local_rank: int = 0
    backend: str | None = None

    @classmethod
    def from_env(cls, backend: str = "nccl") -> "ReplicaGroup":
        """Join the process group the launcher described (RANK / LOCAL_RANK / WORLD_SIZE / MASTER_*);
        a single process needs no group."""
        world = int(os.environ.get("WORLD_SIZE", "1"))
        group = cls(world, int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")), None)
        if world > 1:
            import torch
            import torch.distributed as dist
            kwargs = {}
            if backend == "nccl":
                kwargs["device_id"] = torch.device("cuda", group.local_rank)
            dist.init_process_group(backend, **kwargs)
            group.backend = backend
        return group

    def barrier(self) -> None:
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()

    def rank0_first(self, fn: Callable[[], T]) -> T:
        """Run ``fn`` on rank 0, then on everyone else (for steps that write shared files once)."""
        if self.rank == 0:
            out = fn()
            self.barrier()
            return out
        self.barrier()
        return fn()

    def max_over_ranks(self, values: Sequence[float]) -> list[float]:
        """Element-wise maximum over ranks (the slowest rank defines the job's time)."""
        if self.world == 1:
            return [float(v) for v in values]
        import torch
        import torch.distributed as dist
        device = "cuda" if self.backend == "nccl" else "cpu"
        t = torch.tensor(list(values), dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    def whole_job_rate(self, units_per_rank: int, milliseconds: float) -> float:
        """Units per second over all replicas, given the max-over-ranks time for ``units_per_rank`` each."""
        return self.world * units_per_rank / (milliseconds / 1000.0)

    def close(self) -> None:
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
            dist.destroy_process_group()
