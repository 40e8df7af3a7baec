"""Request-sharded replicas: the multi-GPU form of the verify path for models that fit one GPU.

The reference runs one engine per worker process and shards REQUESTS across workers at its gateway; sequences never
exchange data inside a step. The same holds here: rank r owns its own model copy, KV pool, engine and requests, and
there is no collective on the data path. The only cross-rank traffic is the reduction of the measurements below.
"""
from __future__ import annotations

from dataclasses import dataclass


def rank_seed(base: int, rank: int) -> int:
    """Seed of rank `rank`'s synthetic requests: distinct per rank, reproducible per (base, rank)."""
    return base + rank


def shard_requests(n_requests: int, rank: int, world: int) -> range:
    """Indices of the requests rank `rank` serves when `n_requests` arrive at a front end: contiguous, sizes differ
    by at most one, every request served exactly once."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world {world}")
    base, extra = divmod(n_requests, world)
    lo = rank * base + min(rank, extra)
    return range(lo, lo + base + (1 if rank < extra else 0))


@dataclass
class Totals:
    device_ms: float      # max over ranks: the job is as slow as its slowest replica
    wall_ms: float        # max over ranks
    tokens: float         # sum over ranks: whole-job units of work
    all_identical: bool   # every rank's speculation-on output equalled its speculation-off output


def combine_over_ranks(dist, device, device_ms: float, wall_ms: float, tokens: float, identical: bool, world: int) -> Totals:
    """All ranks call this with their own measurements; all get the job totals. `dist` is torch.distributed with an
    initialised default group (nccl on GPUs, gloo on CPU), or None for a single process."""
    if dist is None or world == 1:
        return Totals(device_ms, wall_ms, tokens, bool(identical))
    import torch
    t = torch.tensor([device_ms, wall_ms], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    c = torch.tensor([float(tokens), 1.0 if identical else 0.0], dtype=torch.float64, device=device)
    dist.all_reduce(c, op=dist.ReduceOp.SUM)
    return Totals(float(t[0]), float(t[1]), float(c[0]), float(c[1]) == world)
