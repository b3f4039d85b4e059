"""Host-side logic of batch-sharded inference: which images a rank owns, how per-rank timings and results are combined.

Inference over independent images needs no exchange on the data path (the reference's CDistributedInference splits
the batch across replicas the same way, NeoML/src/Dnn/DnnDistributed.cpp:551-607); the only communication is the
timing barrier, the max-over-ranks reduction of the measured time and, when a caller wants one result tensor, the
gather of the per-rank outputs in rank order.  Works on any torch.distributed backend (NCCL on GPUs, gloo on CPU).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def image_slice(total: int, world: int, rank: int) -> tuple[int, int]:
    """(first image, image count) of `rank` when `total` images are split into contiguous slices; the first
    total % world ranks take one image more, so slices differ by at most one and cover [0, total) exactly."""
    if world <= 0 or not 0 <= rank < world or total < 0:
        raise ValueError(f"bad split: total={total} world={world} rank={rank}")
    base, extra = divmod(total, world)
    count = base + (1 if rank < extra else 0)
    start = rank * base + min(rank, extra)
    return start, count


def world_and_rank() -> tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size(), dist.get_rank()
    return 1, 0


def max_over_ranks(values: list[float], device="cpu") -> list[float]:
    """Element-wise maximum over all ranks (a step is as slow as its slowest rank)."""
    t = torch.tensor(values, dtype=torch.float64, device=device)
    world, _ = world_and_rank()
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t]


def sum_over_ranks(values: list[float], device="cpu") -> list[float]:
    t = torch.tensor(values, dtype=torch.float64, device=device)
    world, _ = world_and_rank()
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return [float(v) for v in t]


def gather_by_rank(local: torch.Tensor, counts: list[int]) -> torch.Tensor:
    """Concatenation of every rank's rows in rank order (rows of rank r = counts[r]); identical on all ranks."""
    world, _ = world_and_rank()
    if world == 1:
        return local
    width = max(counts)
    padded = torch.zeros((width, *local.shape[1:]), dtype=local.dtype, device=local.device)
    padded[: local.shape[0]] = local
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded)
    return torch.cat([p[:c] for p, c in zip(parts, counts)], dim=0)


def whole_job_throughput(units_all_ranks: float, ms_max_over_ranks: float) -> float:
    """Units per second of the whole job: everything all ranks processed over the slowest rank's time."""
    return units_all_ranks / (ms_max_over_ranks * 1e-3)
