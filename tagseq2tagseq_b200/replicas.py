"""Data-parallel plumbing shared by the benchmarks: which packs a rank owns and how per-rank measurements combine.

The attention path has no exchange step: each rank owns whole packed sequences (the reference's only parallelism is
DDP with one pack per rank per micro-batch and per-rank sampler seeds, main.py:167-168, 404-415).  So a multi-GPU
attention run is a set of independent replicas; the only collective on the path is the gradient all-reduce of the
training step, which torch DDP issues over NCCL.
"""
from __future__ import annotations

from typing import Sequence, Tuple

import torch
import torch.distributed as dist


def rank_seed(base: int, rank: int, item: int = 0) -> int:
    """Seed of item `item` owned by `rank`: disjoint streams per rank, as the reference offsets its sampler seed by rank."""
    return base + 1000 * rank + item


def aggregate(elapsed_ms: Sequence[float], work: Sequence[float], device=None) -> Tuple[list, list]:
    """Whole-job figures from per-rank ones: elapsed times combine by MAX (the slowest rank ends the step),
    work (FLOPs, tokens) by SUM.  Works on any initialised backend; without a process group it is the identity."""
    t = torch.tensor(list(elapsed_ms), dtype=torch.float64, device=device)
    w = torch.tensor(list(work), dtype=torch.float64, device=device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(w, op=dist.ReduceOp.SUM)
    return t.tolist(), w.tolist()
