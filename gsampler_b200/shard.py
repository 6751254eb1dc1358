"""Replica data-parallelism for the sampling path: the graph is replicated per GPU, the seed
list is split, every rank samples its own super-batches; no collective is needed for the data.
``gather_counts`` (one int64 per rank, for reporting) is the only communication.

Host-side logic only: works with any ``torch.distributed`` backend (NCCL on GPUs, gloo in the
CPU tests)."""
from __future__ import annotations

from typing import List, Tuple

import torch


def shard_bounds(n: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous, balanced split of ``n`` items: the first ``n % world`` ranks get one more."""
    if not (0 <= rank < world):
        raise ValueError("rank %d outside world of %d" % (rank, world))
    base, rem = divmod(n, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def shard_seeds(seeds: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    lo, hi = shard_bounds(seeds.numel(), rank, world)
    return seeds[lo:hi]


def super_batches(seeds: torch.Tensor, batch: int, per_step: int) -> List[Tuple[torch.Tensor, torch.Tensor]]:
    """Cuts ``seeds`` into super-batches of ``per_step`` minibatches of ``batch`` seeds.  Every
    pointer has ``per_step + 1`` entries; minibatches past the end of the data are empty."""
    out = []
    step = batch * per_step
    for s0 in range(0, seeds.numel(), step):
        chunk = seeds[s0:s0 + step]
        ptr = (torch.arange(per_step + 1, dtype=torch.int64) * batch).clamp_max(chunk.numel())
        out.append((chunk.contiguous(), ptr.to(seeds.device)))
    return out


def gather_counts(local_count: int, device=None, group=None) -> List[int]:
    """All ranks' counts (reporting only).  Without an initialised process group returns
    ``[local_count]``."""
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()):
        return [int(local_count)]
    t = torch.tensor([int(local_count)], dtype=torch.int64, device=device)
    outs = [torch.zeros_like(t) for _ in range(dist.get_world_size(group))]
    dist.all_gather(outs, t, group=group)
    return [int(o.item()) for o in outs]


def reduce_timing(elapsed_ms: float, units: int, device=None, group=None) -> Tuple[float, int]:
    """(slowest rank's time, summed units): the aggregation the benchmark reports."""
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()):
        return float(elapsed_ms), int(units)
    t = torch.tensor([float(elapsed_ms)], dtype=torch.float64, device=device)
    n = torch.tensor([int(units)], dtype=torch.int64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    dist.all_reduce(n, op=dist.ReduceOp.SUM, group=group)
    return float(t.item()), int(n.item())
