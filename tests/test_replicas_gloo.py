"""Multi-rank host logic on CPU: two gloo ranks own different packs and their measurements combine as max / sum."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from tagseq2tagseq_b200 import synth
        from tagseq2tagseq_b200.replicas import aggregate, rank_seed
        pack = synth.make_pack(rank_seed(1003, rank), 4096, 150, 16, 1024, p_link=0.1)
        pairs = pack.unmasked_pairs()
        ms, work = aggregate([10.0 + 5.0 * rank, 1.0], [float(pairs), 1.0])
        gathered = [None] * world
        dist.all_gather_object(gathered, (int(pack.doc_ids.sum()), pairs))
        if rank == 0:
            out.put((ms, work, gathered))
    finally:
        dist.destroy_process_group()


def test_two_ranks_own_different_packs_and_aggregate():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    ms, work, gathered = out.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert ms == [15.0, 1.0]                      # max over ranks
    assert gathered[0] != gathered[1]             # per-rank seeds give different packs
    assert work == [float(gathered[0][1] + gathered[1][1]), 2.0]   # sum over ranks


def test_aggregate_without_process_group_is_identity():
    from tagseq2tagseq_b200.replicas import aggregate, rank_seed
    assert aggregate([3.0], [7.0]) == ([3.0], [7.0])
    assert rank_seed(1003, 2, 1) == 3004


def test_density_aware_schedule_reduces_the_slowest_rank_stall():
    from tagseq2tagseq_b200 import synth
    from tagseq2tagseq_b200.replicas import schedule_packs, step_time_model
    world, steps = 8, 6
    costs = [float(synth.make_pack(500 + i, 8192, 150, 16, 4096, p_link=0.15, heavy_frac=0.05, heavy_lo=2048, heavy_hi=4096).unmasked_pairs())
             for i in range(world * steps)]
    naive = [list(range(s * world, (s + 1) * world)) for s in range(steps)]
    sched = schedule_packs(costs, world)
    assert sorted(i for st in sched for i in st) == list(range(world * steps))      # every pack used exactly once
    assert all(len(st) == world for st in sched)
    assert step_time_model(costs, sched) <= step_time_model(costs, naive)
    assert step_time_model(costs, sched) < 0.9 * step_time_model(costs, naive)       # heavy-tailed packs: a clear gain
    lower_bound = sum(costs) / world
    assert step_time_model(costs, sched) >= lower_bound
