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


def tile_cost(doc_ids: torch.Tensor, link_bits=None, q_row_ids=None, kv_col_ids=None) -> int:
    """Attention cost of one packed sequence as the pre-pass sees it: the number of non-skipped 128 x 128 tiles
    (partial + full), read back once from the device.  This is what a real data pipeline can know about a pack before
    it trains on it -- the mask inputs, not the generator's document lengths."""
    from .mask_spec import build_block_map
    bm = build_block_map(doc_ids, link_bits, q_row_ids, kv_col_ids, with_lists=True)
    return int((bm.q_cnt.sum() + bm.full_q_cnt.sum()).item())


def schedule_packs(costs: Sequence[float], world: int) -> list:
    """Density-aware pack -> (step, rank) schedule.

    With one packed sequence per rank per step, a DDP step lasts as long as its most expensive pack, and attention
    cost varies several-fold between packs (the reference reports backward times of 2-6 s across ranks,
    configs/stack_100m_32k_baseline.yaml:39-41, and lists balancing as an open item, README.md:151).  Given the
    cost of every pack in a pool of ``steps * world`` packs (e.g. non-skipped tiles from the block-map pre-pass, or
    the exact number of unmasked pairs), packs of similar cost are put into the same step: sort by cost and cut into
    consecutive groups of ``world``.  Within a step the ranks are rotated so that no rank always gets the largest.
    Every rank computes the same schedule from the same costs, so no communication is needed.

    Returns ``schedule[step][rank] = pack index``; packs beyond a multiple of ``world`` are dropped."""
    order = sorted(range(len(costs)), key=lambda i: (-costs[i], i))
    steps = len(order) // world
    sched = []
    for s in range(steps):
        group = order[s * world:(s + 1) * world]
        rot = s % world
        sched.append(group[rot:] + group[:rot])
    return sched


def step_time_model(costs: Sequence[float], schedule: Sequence[Sequence[int]]) -> float:
    """Sum over steps of the most expensive pack in the step (what the slowest rank makes every other rank wait for)."""
    return float(sum(max(costs[i] for i in step) for step in schedule))
