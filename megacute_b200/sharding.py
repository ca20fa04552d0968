"""Batch sharding across the GPUs of one node: one process per GPU, weights replicated, every rank
decodes its own sequences with its own launch.  Nothing crosses GPUs on the data path (sequences of
a decode batch never interact), so the only collectives are the ones a measurement needs: a
barrier around the timed region and a MAX over the ranks' device times.

The reference has no multi-GPU path; this mirrors how its single-GPU loop
(``examples/llama/llama1b.py:103-121``) is replicated per device.
"""

from __future__ import annotations

import torch


def shard_range(total: int, world: int, rank: int) -> tuple[int, int]:
    """(first sequence, count) of `rank`'s contiguous share of `total` sequences; shares differ by at
    most one and the first ``total % world`` ranks take the extra sequence."""
    if world <= 0 or not 0 <= rank < world or total < 0:
        raise ValueError(f"bad shard request: total={total}, world={world}, rank={rank}")
    base, extra = divmod(total, world)
    count = base + (1 if rank < extra else 0)
    start = rank * base + min(rank, extra)
    return start, count


def max_over_ranks(value: float, device="cpu") -> float:
    """MAX of a per-rank scalar over the default process group (identity without one)."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


def job_throughput(units_per_rank: int, ms_per_step: float, device="cpu") -> float:
    """Whole-job units per second: the units all ranks processed in a step divided by the slowest
    rank's step time."""
    import torch.distributed as dist
    total = float(units_per_rank)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        t = torch.tensor([total], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        total = float(t[0])
    return total * 1e3 / max_over_ranks(ms_per_step, device)
