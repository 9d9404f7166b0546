"""One process per GPU: the host-side plumbing for running several replicas of the path.

The decode path does not shard across GPUs at the benchmark's shape (the FFN width of
5632 is 22 super-blocks of 256 and does not split evenly beyond two ways), so N GPUs
run N independent replicas, each with its own weights, KV cache and token stream: no
data-path collective. `torch.distributed` is used only to line the ranks up around a
timed region and to take the slowest rank's time.

`backend="nccl"` on GPUs; `backend="gloo"` lets the same code run as CPU processes.
"""
from __future__ import annotations

import os
from dataclasses import dataclass


@dataclass
class RankInfo:
    rank: int
    world: int
    local_rank: int

    @staticmethod
    def from_env(env=None) -> "RankInfo":
        e = os.environ if env is None else env
        return RankInfo(int(e.get("RANK", "0")), int(e.get("WORLD_SIZE", "1")), int(e.get("LOCAL_RANK", "0")))


def shard_units(n_units: int, rank: int, world: int) -> range:
    """Contiguous, near-even split of independent units (sequences, requests) over ranks:
    the first `n_units % world` ranks take one more. Every unit goes to exactly one rank."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    base, rem = divmod(n_units, world)
    start = rank * base + min(rank, rem)
    return range(start, start + base + (1 if rank < rem else 0))


class Ranks:
    """Barrier and max-over-ranks for the timed region. With world == 1 nothing is set up."""

    def __init__(self, info: RankInfo, backend: str = "nccl"):
        self.info = info
        self.backend = backend
        self._dist = None
        self._device = None
        if info.world > 1:
            import torch
            import torch.distributed as dist
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            if backend == "nccl":
                torch.cuda.set_device(info.local_rank)
                self._device = torch.device("cuda", info.local_rank)
                dist.init_process_group("nccl", rank=info.rank, world_size=info.world, device_id=self._device)
            else:
                self._device = torch.device("cpu")
                dist.init_process_group(backend, rank=info.rank, world_size=info.world)
            self._dist = dist

    @property
    def is_root(self) -> bool:
        return self.info.rank == 0

    def barrier(self) -> None:
        if self._dist:
            self._dist.barrier()

    def max_over_ranks(self, v: float) -> float:
        if not self._dist:
            return float(v)
        import torch
        t = torch.tensor([float(v)], dtype=torch.float64, device=self._device)
        self._dist.all_reduce(t, op=self._dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(self, v: float) -> float:
        if not self._dist:
            return float(v)
        import torch
        t = torch.tensor([float(v)], dtype=torch.float64, device=self._device)
        self._dist.all_reduce(t, op=self._dist.ReduceOp.SUM)
        return float(t.item())

    def close(self) -> None:
        if self._dist:
            self._dist.destroy_process_group()
            self._dist = None


def whole_job_rate(units_all_ranks: float, seconds_slowest_rank: float) -> float:
    """Units every rank processed divided by the slowest rank's time."""
    return units_all_ranks / seconds_slowest_rank
