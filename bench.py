#!/usr/bin/env python
"""Benchmark of the masked flash-attention hot path (block-map pre-pass + forward + backward).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload = the 32k configuration the headline metric is quoted on: B=2, T=32768, H=16, D=128, bf16, swept over
three masks (doc_causal, cross_doc_link with p=0.05 and p=0.3) on seeded synthetic packs (median 150 tokens,
5 % of documents of 4k-8k tokens).  One step = for each mask: pre-pass, forward, backward.  The metric counts
only unmasked FLOPs: 14 * D * H * N with N the exact number of allowed (q, kv) pairs.

Prints ONE JSON line on rank 0.  Under torchrun every rank runs a replica of the same masks on its own q, k, v, dO
(weak scaling: exactly the same work per GPU at every N); there is no collective on this path, so the multi-GPU
number is the aggregate over independent replicas, timed as the max over ranks.
"""
from __future__ import annotations

import argparse
import ctypes
import gc
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

B, T, H, D = 2, 32768, 16, 128
MASKS = ["doc_causal", "link_p05", "link_p30"]
SEED = 1003
WORKLOAD = "attn_fwd_bwd_32k_mask_sweep"
METRIC = "masked attn fwd+bwd TFLOP/s (unmasked FLOPs) at 32k"


def measured_traffic():
    """DRAM bytes per launch of the two main kernels as one ncu capture measured them, per (batch x head x token) so that
    they scale to other sizes of the same kernels.  The capture and the commit it was taken at are recorded in the
    JSON file beside the ncu summary; None when that file is absent."""
    path = os.path.join(ROOT, "profiles", "attn_kernels_dram_traffic.json")
    if not os.path.exists(path):
        return None
    with open(path) as f:
        d = json.load(f)
    units = float(d["B"] * d["H"] * d["T"])
    return {"bwd_bytes_per_bht": (d["bwd"]["dram_read_bytes"] + d["bwd"]["dram_write_bytes"]) / units,
            "fwd_bytes_per_bht": (d["fwd"]["dram_read_bytes"] + d["fwd"]["dram_write_bytes"]) / units,
            "source": f"ncu capture of {d['workload']} at commit {d['commit']}"}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d["bf16_tflops"], d["hbm_gbs"], "measured"
    return 1590.0, 6650.0, "fallback"


def sustained_peak():
    """Dense bf16 rate of a seconds-long GEMM loop under the power cap (the ruler for a kernel timed inside a long loop)."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f).get("bf16_tflops_sustained")
    return 1400.0


class ClockSampler:
    """SM clock and throttle reasons sampled every 50 ms while the timed region runs, read-only through NVML in a
    background thread (spawning nvidia-smi inside the timed region was measured to stall the GPU for tens of
    milliseconds per poll); falls back to one nvidia-smi query after the region when NVML is unavailable."""
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown"}

    def __init__(self, index: int):
        self.index = index
        self.result = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        self._stop = False
        self._thread = None
        self._sm, self._reasons, self._max = [], set(), None

    def _physical_index(self) -> int:
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [x.strip() for x in vis.split(",") if x.strip()]
            if self.index < len(ids) and ids[self.index].isdigit():
                return int(ids[self.index])
        return self.index

    def _loop(self, nv, handle):
        while not self._stop:
            try:
                self._sm.append(float(nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(handle))
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self._reasons.add(name)
            except Exception:  # noqa: BLE001 - sampling must never disturb the measurement
                break
            time.sleep(0.05)

    def __enter__(self):
        try:
            import pynvml as nv
            import threading
            nv.nvmlInit()
            handle = nv.nvmlDeviceGetHandleByIndex(self._physical_index())
            self._max = float(nv.nvmlDeviceGetMaxClockInfo(handle, nv.NVML_CLOCK_SM))
            self._thread = threading.Thread(target=self._loop, args=(nv, handle), daemon=True)
            self._thread.start()
        except Exception:  # noqa: BLE001
            self._thread = None
        return self

    def __exit__(self, *exc):
        self._stop = True
        if self._thread is not None:
            self._thread.join(timeout=2)
        if self._sm:
            self.result = {"sm_mhz": statistics.median(self._sm), "sm_max_mhz": self._max, "reasons": sorted(self._reasons),
                           "samples": len(self._sm), "source": "nvml"}
            return
        try:  # fallback: a single query after the region
            out = subprocess.run(["nvidia-smi", "--query-gpu=clocks.sm,clocks.max.sm", "--format=csv,noheader,nounits", "-i", str(self.index)],
                                 capture_output=True, text=True, timeout=20).stdout.strip().split(",")
            self.result = {"sm_mhz": float(out[0]), "sm_max_mhz": float(out[1]), "reasons": [], "samples": 1, "source": "nvidia-smi after the region"}
        except Exception:  # noqa: BLE001
            pass


def make_workload(rank: int, device):
    from tagseq2tagseq_b200 import synth
    masks = []
    for mi, name in enumerate(MASKS):
        if WORKLOAD == "attn_fwd_bwd_16k_cross_doc_link":
            packs = [synth.config2_pack(SEED + b) for b in range(B)]
        else:
            packs = [synth.config3_pack(SEED + 10 * mi + b, name) for b in range(B)]
        doc_np, link_np = synth.stack_packs(packs)
        n_pairs = sum(p.unmasked_pairs() for p in packs)
        masks.append({"name": name, "doc": torch.from_numpy(doc_np).to(device),
                      "link": None if link_np is None else torch.from_numpy(link_np).to(device),
                      "doc_host": torch.from_numpy(doc_np).pin_memory(),
                      "link_host": None if link_np is None else torch.from_numpy(link_np).pin_memory(),
                      "pairs": n_pairs, "density": n_pairs / (B * T * T), "docs": [int(p.lengths.size) for p in packs], "packs": packs})
    return masks


def flops_of(pairs: int) -> float:
    return 14.0 * D * H * pairs


def run_ours(args, rank, world, device):
    from tagseq2tagseq_b200 import _lib
    from tagseq2tagseq_b200.attention import _attn_bwd, _attn_fwd
    from tagseq2tagseq_b200.mask_spec import build_block_map, read_status

    L = _lib.lib()
    torch.manual_seed(SEED + rank)
    masks = make_workload(rank, device)
    q, k, v, do = (torch.randn(B, H, T, D, device=device, dtype=torch.float32).bfloat16() for _ in range(4))
    scale = 1.0 / D ** 0.5
    launches = [0]

    def step_device():
        for m in masks:
            bm = build_block_map(m["doc"], m["link"])
            out, lse = _attn_fwd(q, k, v, m["doc"], m["link"], None, None, bm.plan, scale)
            _attn_bwd(q, k, v, out, do, lse, m["doc"], m["link"], None, None, bm.plan, scale)
            # pre-pass (runs, state, lists, pair counts, orders; + transposed links), forward, backward (prep, main, convert)
            launches[0] += 5 + (1 if m["link"] is not None else 0) + 1 + 3
        return bm

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize(device)

    for _ in range(max(3, args.warmup)):
        bm = step_device()
    barrier()
    if read_status(bm.plan) != 0:
        raise RuntimeError("a kernel reported a bounded-wait timeout during warm-up")
    launches[0] = 0
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(device.index) as clocks:
        barrier()
        ev0.record()
        for _ in range(args.steps):
            step_device()
        ev1.record()
        barrier()
    ms = ev0.elapsed_time(ev1)
    total_flops = sum(flops_of(m["pairs"]) for m in masks) * args.steps
    n_launch = launches[0]

    # ---- per-kernel timing (main forward / backward kernels) for the roofline, same inputs, after the timed region
    L.ts2ts_profile_enable(1)
    per_mask = []
    fms, bms = ctypes.c_float(0), ctypes.c_float(0)
    for m in masks:
        bml = build_block_map(m["doc"], m["link"], with_lists=True)
        m["tiles"] = int((bml.q_cnt.sum() + bml.full_q_cnt.sum()).item())  # non-skipped 128 x 128 tiles
        del bml
        f_list, b_list, pp_list = [], [], []
        for _ in range(max(3, min(args.steps, 5))):
            pe0, pe1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            pe0.record()
            bm = build_block_map(m["doc"], m["link"])
            pe1.record()
            out, lse = _attn_fwd(q, k, v, m["doc"], m["link"], None, None, bm.plan, scale)
            _attn_bwd(q, k, v, out, do, lse, m["doc"], m["link"], None, None, bm.plan, scale)
            L.ts2ts_profile_last_ms(0, ctypes.byref(fms)); L.ts2ts_profile_last_ms(1, ctypes.byref(bms))
            f_list.append(fms.value); b_list.append(bms.value); pp_list.append(pe0.elapsed_time(pe1))
        per_mask.append({"mask": m["name"], "density": round(m["density"], 4), "tiles": m["tiles"],
                         "executed_over_algorithmic": m["tiles"] * 16384.0 / m["pairs"], "fwd_ms": statistics.mean(f_list),
                         "bwd_ms": statistics.mean(b_list), "prepass_ms": statistics.median(pp_list), "fwd_tflops": 4.0 * D * H * m["pairs"] / statistics.mean(f_list) / 1e9,
                         "bwd_tflops": 10.0 * D * H * m["pairs"] / statistics.mean(b_list) / 1e9})
    L.ts2ts_profile_enable(0)
    bwd_flops = sum(10.0 * D * H * m["pairs"] for m in masks) / len(masks)
    bwd_ms = statistics.mean(p["bwd_ms"] for p in per_mask)
    peak_tf, peak_hbm, peak_kind = measured_peaks()
    achieved = sum(10.0 * D * H * m["pairs"] for m in masks) / sum(p["bwd_ms"] for p in per_mask) / 1e9

    # ---- end to end: pinned host buffers in, results back to host, through the same entry points
    hq, hk, hv, hdo = (x.cpu().pin_memory() for x in (q, k, v, do))
    h_out, h_dq, h_dk, h_dv = (torch.empty((B, H, T, D), dtype=torch.bfloat16).pin_memory() for _ in range(4))
    h_lse = torch.empty((B, H, T), dtype=torch.float32).pin_memory()
    # Three streams, two input slots: the host->device copy of the next call, the kernels of the current one and the
    # device->host copy of the previous one overlap.  Every call still moves all of its inputs in and all of its
    # results out inside the timed region.
    s_in, s_comp, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device), torch.cuda.Stream(device)
    slots = [{"t": [torch.empty_like(q) for _ in range(4)], "ev_in": torch.cuda.Event(), "ev_comp": torch.cuda.Event()} for _ in range(2)]
    dq_ = dk_ = dv_ = do_ = None

    def run_e2e(n_steps):
        items = [m for _ in range(n_steps) for m in masks]
        ev_start, ev_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for s_ in (s_in, s_comp, s_out):
            s_.wait_stream(torch.cuda.current_stream(device))
        ev_start.record(s_in)
        for t, m in enumerate(items):
            sl = slots[t % 2]
            with torch.cuda.stream(s_in):
                if t >= 2:
                    s_in.wait_event(sl["ev_comp"])  # the kernels that read this slot two calls ago are done
                for dst, src in zip(sl["t"], (hq, hk, hv, hdo)):
                    dst.copy_(src, non_blocking=True)
                doc = m["doc_host"].to(device, non_blocking=True)
                link = None if m["link_host"] is None else m["link_host"].to(device, non_blocking=True)
                sl["ev_in"].record(s_in)
            with torch.cuda.stream(s_comp):
                s_comp.wait_event(sl["ev_in"])
                doc.record_stream(s_comp)
                if link is not None:
                    link.record_stream(s_comp)
                dq_i, dk_i, dv_i, do_i = sl["t"]
                bm = build_block_map(doc, link)
                out, lse = _attn_fwd(dq_i, dk_i, dv_i, doc, link, None, None, bm.plan, scale)
                gq, gk, gv = _attn_bwd(dq_i, dk_i, dv_i, out, do_i, lse, doc, link, None, None, bm.plan, scale)
                sl["ev_comp"].record(s_comp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(sl["ev_comp"])
                for dst, src in zip((h_out, h_lse, h_dq, h_dk, h_dv), (out, lse, gq, gk, gv)):
                    src.record_stream(s_out)
                    dst.copy_(src, non_blocking=True)
        s_comp.wait_stream(s_in)
        s_comp.wait_stream(s_out)
        ev_end.record(s_comp)
        torch.cuda.current_stream(device).wait_stream(s_comp)
        return ev_start, ev_end

    e2e_steps = max(1, min(args.steps, 5))
    run_e2e(1)
    barrier()
    e0, e1 = run_e2e(e2e_steps)
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    tens = B * H * T * D * 2
    mask_bytes = sum(m["doc_host"].numel() * 4 + (0 if m["link_host"] is None else m["link_host"].numel() * 8) for m in masks)
    h2d = 4 * tens * len(masks) + mask_bytes
    d2h = (4 * tens + B * H * T * 4) * len(masks)

    ref_mask = ref_format = mask_create = decode = None
    if world == 1 and WORKLOAD == "attn_fwd_bwd_32k_mask_sweep":
        ref_mask = reference_block_mask_time(masks[0]["packs"][0], device)
        ref_format = reference_format_mask_time(masks[2]["packs"][0], q, k, v, do, device)
        mask_create = mask_create_time(device)
        decode = decode_step_bench(masks, q, k, v, device, per_mask[2]["fwd_ms"])

    train = None
    if WORKLOAD == "attn_fwd_bwd_32k_mask_sweep" and not args.no_train:
        del hq, hk, hv, hdo, h_out, h_dq, h_dk, h_dv, slots, q, k, v, do
        torch.cuda.empty_cache()
        train = run_train(args, rank, world, device, "train4", steps=max(2, min(args.steps, 5)), warmup=3)
        torch.cuda.empty_cache()
        train5 = run_train(args, rank, world, device, "train5", steps=max(2, min(args.steps, 3)), warmup=3, both_schedules=False)
        if train is not None and train5 is not None:
            train["config5"] = train5

    t_ms = torch.tensor([ms, e2e_ms], device=device, dtype=torch.float64)
    fl = torch.tensor([total_flops, sum(flops_of(m["pairs"]) for m in masks) * e2e_steps], device=device, dtype=torch.float64)
    rates = torch.zeros(world, device=device, dtype=torch.float64)  # every rank's own TFLOP/s over its own timed region
    rates[rank] = total_flops / (ms * 1e-3) / 1e12
    if world > 1:
        torch.distributed.all_reduce(t_ms, op=torch.distributed.ReduceOp.MAX)
        torch.distributed.all_reduce(fl, op=torch.distributed.ReduceOp.SUM)
        torch.distributed.all_reduce(rates, op=torch.distributed.ReduceOp.SUM)
    if rank != 0:
        return
    rate_list = sorted(rates.tolist())
    traffic = measured_traffic()
    value = fl[0].item() / (t_ms[0].item() * 1e-3) / 1e12
    e2e_value = fl[1].item() / (t_ms[1].item() * 1e-3) / 1e12
    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
        "ms_per_step": t_ms[0].item() / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "B": B, "T": T, "H": H, "head_dim": D, "masks": MASKS,
                   "replicas": "every rank runs the same masks on its own q,k,v,dO (equal work per GPU)",
                   "doc_lengths": ("lognormal median 150 sigma 1.0 clip [16,4096], 5% uniform [4096,8192]" if T == 32768 else
                                   "lognormal median 200 sigma 1.0 clip [32,2048]"),
                   "l2": "inputs_exceed_l2 (q,k,v,dO = 1.07 GB per call)", "per_mask": per_mask,
                   "step": "per mask: block-map pre-pass + forward + backward", "seed": SEED},
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                "ms_per_step": t_ms[1].item() / e2e_steps,
                # both directions run concurrently with the kernels; each figure is that direction's bytes over the whole region
                "h2d_gbs_per_gpu": h2d * e2e_steps / (e2e_ms * 1e-3) / 1e9, "d2h_gbs_per_gpu": d2h * e2e_steps / (e2e_ms * 1e-3) / 1e9,
                "how": "pinned host q,k,v,dout + mask in, out,lse,dq,dk,dv back to pinned host for every call; copies and kernels on three streams"},
        "per_rank_tflops": {"min": rate_list[0], "median": statistics.median(rate_list), "max": rate_list[-1]},
        "gpu_launches": n_launch,
        "clocks": clocks.result,
        "roofline": {"bound": "tensor", "kernel": "attn_bwd_kernel<128>", "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s",
                     "frac": achieved / peak_tf, "peak_kind": peak_kind + " (burst)", "avg_launch_ms": bwd_ms,
                     # the launches are timed inside the seconds-long loop, at the clock the power cap leaves
                     "peak_sustained": sustained_peak(), "frac_of_sustained": achieved / sustained_peak(),
                     "algorithmic_flops_per_launch": bwd_flops,
                     # dram read + write bytes per launch from the recorded ncu capture, scaled by B*H*T to this workload
                     "traffic": None if traffic is None else traffic["bwd_bytes_per_bht"] * (B * H * T),
                     "traffic_source": None if traffic is None else traffic["source"],
                     "fwd": {"achieved": sum(4.0 * D * H * m["pairs"] for m in masks) / sum(p["fwd_ms"] for p in per_mask) / 1e9,
                             "frac": sum(4.0 * D * H * m["pairs"] for m in masks) / sum(p["fwd_ms"] for p in per_mask) / 1e9 / peak_tf,
                             "avg_launch_ms": statistics.mean(p["fwd_ms"] for p in per_mask),
                             "traffic": None if traffic is None else traffic["fwd_bytes_per_bht"] * (B * H * T)},
                     # executed = every element of a non-skipped 128 x 128 tile counted, masked or not
                     "executed_over_algorithmic_flops": sum(m["tiles"] for m in masks) * 16384.0 / sum(m["pairs"] for m in masks)},
    }
    if world == 1:
        line["cpu_baseline"] = cpu_baseline(steps=5)
    if train is not None:
        line["train_step"] = train
    if world == 1:
        line["link_scan"] = link_scan_bench(device)
    if ref_mask is not None:
        line["block_map_vs_reference"] = ref_mask
    if ref_format is not None:
        line["reference_format_mask"] = ref_format
    if mask_create is not None:
        line["mask_create"] = mask_create
    if decode is not None:
        line["decode_step"] = decode
    emit(line)


def decode_step_bench(masks, q, k, v, device, fwd_ms_full):
    """One decoding step with KV reuse (ts2ts_attn_decode) at the workload's size: the newest token of each of the B
    sequences against the cached K / V of all T tokens under the link_p30 mask, beside the time of the full forward
    that the reference would recompute for that token.  HBM-bound: every allowed key's K and V row is read once."""
    from tagseq2tagseq_b200.attention import masked_attn_decode
    _, hbm_gbs, peak_kind = measured_peaks()
    m = masks[2]
    q1 = q[:, :, -1:].contiguous()
    for _ in range(3):
        out, lse = masked_attn_decode(q1, k, v, m["doc"], m["link"])
    torch.cuda.synchronize(device)
    reps = 50
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        out, lse = masked_attn_decode(q1, k, v, m["doc"], m["link"])
    e1.record()
    torch.cuda.synchronize(device)
    us = e0.elapsed_time(e1) * 1e3 / reps
    allowed = 0
    for pk in m["packs"]:  # keys the last token may read: its own document and the documents it links to
        last = len(pk.lengths) - 1
        allowed += int(pk.lengths[last]) + sum(int(pk.lengths[b_]) for a, b_ in pk.links if a == last)
    bytes_alg = allowed * 4.0 * D * H
    return {"B": B, "H": H, "Tk": T, "head_dim": D, "mask": m["name"], "allowed_keys": allowed, "us_per_call": us, "gpu_launches_per_call": 2,
            "full_forward_ms_recomputed_by_the_reference": fwd_ms_full, "speedup_over_full_forward": fwd_ms_full * 1e3 / us,
            "roofline": {"bound": "hbm", "achieved": bytes_alg / us / 1e3, "peak": hbm_gbs, "unit": "GB/s", "frac": bytes_alg / us / 1e3 / hbm_gbs,
                         "peak_kind": peak_kind, "note": "K and V rows of the allowed keys, once; a call this short is bound by its two launches"}}


def reference_block_mask_time(pack, device):
    """The mask build the reference does once per micro-batch, timed beside this package's pre-pass on the same pack:
    torch's create_block_mask with the reference's doc_causal mask_mod and arguments (B=None, H=None, eager, as in
    model/graph_traversal/block_mask_creator.py:121-139), which materialises the dense T x T mask on the GPU."""
    from torch.nn.attention.flex_attention import create_block_mask
    from tagseq2tagseq_b200.mask_spec import build_block_map
    doc_np = pack.doc_ids
    t = int(doc_np.shape[0])
    document_ids = torch.from_numpy(doc_np).to(device)

    def doc_causal_mod(b, h, q_idx, kv_idx):
        return (q_idx >= kv_idx) & (document_ids[q_idx] == document_ids[kv_idx])

    def timed(fn, warm, reps):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize(device)
        out = []
        for _ in range(reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); fn(); e1.record()
            torch.cuda.synchronize(device)
            out.append(e0.elapsed_time(e1))
        return statistics.median(out)

    try:
        ref_ms = timed(lambda: create_block_mask(doc_causal_mod, B=None, H=None, Q_LEN=t, KV_LEN=t, device=device), 3, 5)
    except Exception as exc:  # noqa: BLE001 - a torch-side failure must not cost the whole line
        return {"unavailable": str(exc).splitlines()[0][:200]}
    doc1 = document_ids[None].contiguous()
    ours_ms = timed(lambda: build_block_map(doc1, None), 3, 5)
    torch.cuda.empty_cache()
    return {"mask": "doc_causal pack 0, B=1, T=%d" % t, "reference_create_block_mask_ms": ref_ms, "prepass_ms": ours_ms,
            "how": "3 warm-ups, median of 5, CUDA events; torch.nn.attention.flex_attention.create_block_mask (eager) with the reference's mask_mod"}


def reference_format_mask_time(pack, q, k, v, do, device):
    """Forward / backward on a mask in the reference's own grant format: every link of the pack starts in the middle of
    its source document (link_end_pos), so documents split into several row classes, and at most 256 grants are kept
    (the reference's largest max_grants).  Built through the host adapter from_reference; same q, k, v, dO (batch 0)."""
    from types import SimpleNamespace
    from tagseq2tagseq_b200 import _lib
    from tagseq2tagseq_b200.attention import _attn_bwd, _attn_fwd
    from tagseq2tagseq_b200.mask_spec import from_reference, ordered_grants
    L = _lib.lib()
    lengths = pack.lengths
    starts = np.concatenate([[0], np.cumsum(lengths)[:-1]])
    spans = [SimpleNamespace(doc_id=i, start=int(starts[i]), end=int(starts[i] + lengths[i])) for i in range(len(lengths))]
    link_to_target = {}
    for a, b_ in pack.links:
        pos = int(starts[a] + max(1, lengths[a] // 2))
        link_to_target.setdefault(pos, []).append(int(b_))
    t = int(pack.doc_ids.shape[0])
    spec = from_reference(spans, link_to_target, t, max_grants_cap=256, device=device)
    grants = ordered_grants(t, spans, link_to_target, 256)
    pairs = int(sum(int(n) * (int(n) + 1) // 2 for n in lengths))
    covered = set()
    for q0, q1, k0, k1 in grants:  # grants may overlap: count every (source rows, target document) block once
        covered.add((q0, q1, k0, k1))
    pairs += sum((q1 - q0) * (k1 - k0) for q0, q1, k0, k1 in covered)
    q1_, k1_, v1_, do1_ = (x[:1] for x in (q, k, v, do))
    scale = 1.0 / D ** 0.5
    L.ts2ts_profile_enable(1)
    fms, bms = ctypes.c_float(0), ctypes.c_float(0)
    f_list, b_list = [], []
    for _ in range(4):
        out, lse = _attn_fwd(q1_, k1_, v1_, spec.doc_ids, spec.link_bits, spec.q_row_ids, spec.kv_col_ids, spec.plan, scale)
        _attn_bwd(q1_, k1_, v1_, out, do1_, lse, spec.doc_ids, spec.link_bits, spec.q_row_ids, spec.kv_col_ids, spec.plan, scale)
        L.ts2ts_profile_last_ms(0, ctypes.byref(fms)); L.ts2ts_profile_last_ms(1, ctypes.byref(bms))
        f_list.append(fms.value); b_list.append(bms.value)
    L.ts2ts_profile_enable(0)
    f_ms, b_ms = statistics.median(f_list[1:]), statistics.median(b_list[1:])
    return {"mask": "link_p30 pack 0 as reference grants from mid-document link positions, cap 256", "grants": len(grants),
            "row_classes": int(spec.link_bits.shape[1]), "B": 1, "fwd_ms": f_ms, "bwd_ms": b_ms,
            "fwd_tflops": 4.0 * D * H * pairs / f_ms / 1e9, "bwd_tflops": 10.0 * D * H * pairs / b_ms / 1e9,
            "note": "overlapping grants are counted once per distinct (row range, target) block; an upper bound when blocks overlap"}


def link_scan_bench(device):
    """Device-side markdown link scan (ts2ts_detect_links) on synthetic GPT-2-sized token streams: uniform random ids
    with a '](' planted every ~200 tokens behind a '[' and in front of a closing token.  The real GPT-2 table of
    tokens that contain ')' needs the BPE files, so a synthetic table stands in for it (every 97th id closes a link).
    Reports the scan at the 32k sequence length of the workload (latency-bound) and on a 1 Mi-token stream against the
    measured HBM copy bandwidth, with the oracle's pure-Python scan of the 32k stream timed beside it."""
    from tagseq2tagseq_b200 import _lib
    from oracle import link_detect as old
    L = _lib.lib()
    _, hbm_gbs, peak_kind = measured_peaks()
    vocab, mid, starts = 50257, 16151, [58, 685]
    rng = np.random.default_rng(77)
    flags_np = (np.arange(vocab) % 97 == 0).astype(np.uint8)
    closers = np.nonzero(flags_np)[0]
    out = {"vocab": vocab, "note": "synthetic close-token table (every 97th id)"}
    for name, n_tok in (("32k", 32768), ("1Mi", 1 << 20)):
        toks = rng.integers(1000, vocab, size=n_tok, dtype=np.int64)
        toks[np.isin(toks, [mid] + starts)] = 1000
        for pos in range(50, n_tok - 60, 200):
            toks[pos] = starts[pos // 200 % 2]
            toks[pos + 5] = mid
            toks[pos + 5 + 1 + (pos // 200) % 9] = closers[(pos // 200) % len(closers)]
        tok_d = torch.from_numpy(toks).to(device)
        flags_d = torch.from_numpy(flags_np).to(device)
        scratch = torch.empty(L.ts2ts_detect_links_scratch_bytes(n_tok), dtype=torch.uint8, device=device)
        max_links = n_tok // 64
        links = torch.empty((max_links, 3), dtype=torch.int32, device=device)
        count = torch.zeros(1, dtype=torch.int32, device=device)
        start_arr = (ctypes.c_int64 * 2)(*starts)
        stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)

        def call():
            rc = L.ts2ts_detect_links(tok_d.data_ptr(), 8, n_tok, mid, start_arr, 2, flags_d.data_ptr(), vocab, 100, 50,
                                      scratch.data_ptr(), scratch.numel(), links.data_ptr(), max_links, count.data_ptr(), stream)
            if rc != 0:
                raise RuntimeError(L.ts2ts_last_error_string().decode())
        for _ in range(3):
            call()
        torch.cuda.synchronize(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 50
        e0.record()
        for _ in range(reps):
            call()
        e1.record()
        torch.cuda.synchronize(device)
        us = e0.elapsed_time(e1) * 1e3 / reps
        res = {"tokens": n_tok, "links": int(count.item()), "us_per_call": us, "gpu_launches_per_call": 3,
               "token_gbs": n_tok * 8 / us / 1e3}
        if name == "1Mi":
            # algorithmic bytes: tokens read once (8 B) + dense marks written and read once (2 x 8 B)
            res["roofline"] = {"bound": "hbm", "achieved": n_tok * 24 / us / 1e3, "peak": hbm_gbs, "unit": "GB/s",
                               "frac": n_tok * 24 / us / 1e3 / hbm_gbs, "peak_kind": peak_kind}
        else:
            decode = lambda ids: "".join(")" if flags_np[i] else "a" for i in ids)
            t0 = time.perf_counter()
            want = old.candidates(toks.tolist(), decode, mid_id=mid, start_ids=starts, window=50)
            res["cpu_port_us"] = (time.perf_counter() - t0) * 1e6
            got = links[:int(count.item())].cpu().tolist()
            res["matches_oracle"] = [tuple(g) for g in got] == want
        out[name] = res
    return out


def run_train(args, rank, world, device, which: str, steps: int, warmup: int, both_schedules: bool = True):
    """Training step of the 12-layer (train4) or 24-layer (train5) decoder LM, one packed sequence per rank, DDP.

    Packs come from a pool of world * n_packs seeded packs that every rank derives identically.  Two schedules are
    timed: the density-aware one (packs of similar attention cost share a step; the cost of a pack is its number of
    non-skipped tiles, read from the block-map pre-pass) and plain seed order, which is what the reference does."""
    from tagseq2tagseq_b200 import synth
    from tagseq2tagseq_b200.mask_spec import MaskSpec
    from tagseq2tagseq_b200.replicas import aggregate, rank_seed, schedule_packs, tile_cost
    from tagseq2tagseq_b200.train_step import TrainStep, config4, config5, train_flops_per_step
    cfg, t_len, base = (config4(), 16384, 1004) if which == "train4" else (config5(), 32768, 1005)
    ts = TrainStep(cfg, device, world, bucket_cap_mb=args.bucket_mb, bf16_grads=not args.fp32_buckets)
    n_packs = 4  # steps in the pool
    make = (lambda sd: synth.config2_pack(sd)) if which == "train4" else (lambda sd: synth.config5_pack(sd))
    pool = [make(rank_seed(base, r, i)) for i in range(n_packs) for r in range(world)]

    def to_spec(pk):
        doc_np, link_np = synth.stack_packs([pk])
        return MaskSpec(doc_ids=torch.from_numpy(doc_np).to(device), link_bits=torch.from_numpy(link_np).to(device))

    costs = None
    if world > 1 and not args.no_balance:
        costs = []
        for pk in pool:
            sp = to_spec(pk)
            costs.append(float(tile_cost(sp.doc_ids, sp.link_bits)))
        del sp
        torch.cuda.empty_cache()  # the block maps with explicit lists leave odd-sized cached blocks behind
    peak_tf, _, kind = measured_peaks()

    def measure(schedule_name):
        if schedule_name == "seed order" or costs is None:
            mine = [i * world + rank for i in range(n_packs)]
        else:
            sched = schedule_packs(costs, world)
            mine = [sched[i][rank] for i in range(n_packs)]
        g = torch.Generator().manual_seed(rank_seed(base, rank))
        batches = []
        for i in mine:
            batches.append((torch.randint(0, cfg.vocab, (1, t_len + 1), generator=g).to(device), to_spec(pool[i]), pool[i].unmasked_pairs()))
        for i in range(max(warmup, n_packs)):  # every batch of the schedule once before the clock starts
            tok, spec, _ = batches[i % n_packs]
            spec._block_map = None
            loss = ts.step(tok, spec)
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize(device)
        # The step is 30 ms of kernels behind 15-20 ms of host work per rank: a full Python garbage collection in the
        # middle of the timed steps (tens of ms with this many live objects) would be billed to the GPU.
        gc.collect()
        gc.disable()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        flops = 0.0
        for i in range(steps):
            tok, spec, pairs = batches[i % n_packs]
            spec._block_map = None  # the pre-pass is part of every step, as in the reference (one mask build per micro-batch)
            loss = ts.step(tok, spec)
            flops += train_flops_per_step(cfg, t_len, pairs)
        ev1.record()
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize(device)
        gc.enable()
        my_ms = ev0.elapsed_time(ev1)
        (ms,), (tot_flops, tot_tokens) = aggregate([my_ms], [flops, float(t_len * steps)], device)
        res = {"value": tot_tokens / (ms * 1e-3), "ms_per_step": ms / steps,
               "model_tflops": tot_flops / (ms * 1e-3) / 1e12, "frac_of_peak": tot_flops / (ms * 1e-3) / 1e12 / (peak_tf * world),
               "loss": float(loss)}
        if world > 1:
            # What the collective and the slowest rank cost: forward + backward of every pack of the schedule with and
            # without the gradient all-reduce (DDP no_sync), timed per rank without barriers in between.
            def fb_ms(sync):
                torch.cuda.synchronize(device)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for tok, spec, _ in batches:
                    ts.forward_backward(tok, spec, sync=sync)
                e1.record()
                torch.cuda.synchronize(device)
                return e0.elapsed_time(e1) / len(batches)
            local = fb_ms(False)
            torch.distributed.barrier()
            synced = fb_ms(True)
            v = torch.tensor([local, -local, synced], device=device, dtype=torch.float64)
            torch.distributed.all_reduce(v, op=torch.distributed.ReduceOp.MAX)
            res["fwd_bwd_ms_without_allreduce"] = {"max_over_ranks": v[0].item(), "min_over_ranks": -v[1].item()}
            res["fwd_bwd_ms_with_allreduce_max"] = v[2].item()
        return res

    first = "seed order" if (args.no_balance or world == 1) else "density-aware (similar-cost packs share a step; cost = non-skipped tiles from the pre-pass)"
    main = measure(first)
    out = {"metric": "train tokens/s", "unit": "tokens/s", "steps": steps,
           "model": f"{cfg.n_layers}L d{cfg.d_model} {cfg.n_heads}h hd{cfg.head_dim} swiglu{cfg.mlp_hidden} V{cfg.vocab}",
           "seq_len": t_len, "global_batch_tokens": t_len * world, "parallelism": f"ddp{world}", "pack_schedule": first,
           "optimizer": "fused AdamW (fp32 params, bf16 autocast)",
           "gradient_allreduce": "none (1 GPU)" if world == 1 else f"NCCL, {'bf16-compressed' if ts.bf16_grads else 'fp32'} buckets of {args.bucket_mb} MB (fp32 size), {ts.grad_bytes_per_step / 1e9:.2f} GB per rank per step",
           "peak_kind": kind}
    out.update(main)
    if both_schedules and world > 1 and not args.no_balance:
        out["seed_order_schedule"] = measure("seed order")
    return out


def cpu_sample():
    """Bounded sample of the workload for the CPU arm: the first 8192 tokens of the doc_causal pack, 4 heads."""
    from tagseq2tagseq_b200 import synth
    from oracle import masks as om
    pack = synth.config3_pack(SEED, "doc_causal")
    t = 8192
    doc = pack.doc_ids[:t]
    dense = om.class_mask_dense(doc, None, None, None)
    pairs = int(dense.sum())
    g = torch.Generator().manual_seed(SEED)
    heads = 4
    q, k, v, do = (torch.randn(1, heads, t, D, generator=g) for _ in range(4))
    return torch.from_numpy(dense), q, k, v, do, pairs, heads, t


def load_reference_mask_modules():
    """The reference's link_detector.py and cross_doc_mask.py loaded by path from baseline/_ref (bare `model` packages:
    model/__init__ needs tunalab, which is absent).  None when baseline/_ref is absent or does not import."""
    import importlib.util
    import types
    ref = os.path.join(ROOT, "baseline", "_ref")
    path = os.path.join(ref, "model", "graph_traversal", "cross_doc_mask.py")
    if not os.path.exists(path):
        return None
    try:
        for name in ("model", "model.graph_traversal"):
            if name not in sys.modules:
                m = types.ModuleType(name)
                m.__path__ = []
                sys.modules[name] = m
        mods = {}
        for name, rel in (("model.graph_traversal.link_detector", "link_detector.py"), ("model.graph_traversal.cross_doc_mask", "cross_doc_mask.py")):
            if name in sys.modules and hasattr(sys.modules[name], "__file__"):
                mods[name] = sys.modules[name]
                continue
            spec = importlib.util.spec_from_file_location(name, os.path.join(ref, "model", "graph_traversal", rel))
            mod = importlib.util.module_from_spec(spec)
            sys.modules[name] = mod
            spec.loader.exec_module(mod)
            mods[name] = mod
        return mods["model.graph_traversal.link_detector"], mods["model.graph_traversal.cross_doc_mask"]
    except Exception:  # noqa: BLE001
        return None


def mask_create_time(device):
    """One micro-batch's mask creation, CrossDocLinkMaskCreator.__call__ to a usable mask object, timed on the same
    document spans and detected links (T = 16384, the config-2 pack, every link placed in the middle of its source
    document, max_grants = 256): this package's creator (host matching and segment classes, per-token ids and block-map
    pre-pass on the device) and, when baseline/_ref is present, the reference's own creator
    (model/graph_traversal/cross_doc_mask.py:302-369: per-grant slice writes + torch create_block_mask on the GPU).
    Wall clock around a device synchronisation, 2 warm-ups, median of 5."""
    from types import SimpleNamespace
    from tagseq2tagseq_b200 import mask_spec as ms
    from tagseq2tagseq_b200 import synth
    pack = synth.config2_pack()
    lengths = pack.lengths
    starts = np.concatenate([[0], np.cumsum(lengths)[:-1]])
    t = int(pack.doc_ids.shape[0])
    spans = [SimpleNamespace(doc_id=i, start=int(starts[i]), end=int(starts[i] + lengths[i]), raw_identifier=f"doc{i}") for i in range(len(lengths))]
    found = [(int(starts[a] + max(1, lengths[a] // 2)), f"doc{b_}") for a, b_ in pack.links]
    tokens = torch.zeros((1, t), dtype=torch.int64, device=device)

    def detector(link_cls):
        class Det:
            def detect_links(self, ids):
                return [link_cls(p_, s_) for p_, s_ in found]

            def index_doc_span(self, span):
                return span.raw_identifier
        return Det()

    def timed(fn):
        for _ in range(2):
            fn()
        torch.cuda.synchronize(device)
        out = []
        for _ in range(5):
            t0 = time.perf_counter()
            fn()
            torch.cuda.synchronize(device)
            out.append((time.perf_counter() - t0) * 1e3)
        return statistics.median(out)

    ours = ms.CrossDocLinkMaskCreator(detector(ms.LinkInfo), max_grants=256)
    res = {"T": t, "docs": len(spans), "links": len(found), "max_grants": 256,
           "ours_ms": timed(lambda: ours(tokens, spans).plan)}
    mods = load_reference_mask_modules()
    if mods is None:
        res["reference_ms"] = None
        res["reference"] = "baseline/_ref absent"
        return res
    ld, cdm = mods
    try:
        theirs = cdm.CrossDocLinkMaskCreator(link_detector=detector(ld.LinkInfo), max_grants=256)
        res["reference_ms"] = timed(lambda: theirs(tokens, spans))
        res["reference"] = "CrossDocLinkMaskCreator.__call__ of baseline/_ref on the same GPU"
    except Exception as exc:  # noqa: BLE001 - the reference's eager mask build may not fit or trace on this box
        res["reference_ms"] = None
        res["reference"] = "failed: " + str(exc).splitlines()[0][:160]
    torch.cuda.empty_cache()
    return res


def reference_mask_and_step():
    """The reference's own CPU code for this path, when its sources are present under baseline/_ref: dense mask from
    CrossDocLinkMaskCreator.build_dense_mask_for_visualization (model/graph_traversal/cross_doc_mask.py:371-409),
    attention = fp32 F.scaled_dot_product_attention + autograd (FlexAttention has no CPU backward).
    Returns None when baseline/_ref is absent, so that the oracle port is used instead."""
    from types import SimpleNamespace
    mods = load_reference_mask_modules()
    if mods is None:
        return None
    cdm = mods[1]

    class NoLinks:
        def detect_links(self, ids):
            return []

        def index_doc_span(self, span):
            return span.raw_identifier

    def dense_for(doc_ids):
        spans, start = [], 0
        t = len(doc_ids)
        for i in range(1, t + 1):
            if i == t or doc_ids[i] != doc_ids[start]:
                spans.append(SimpleNamespace(doc_id=int(doc_ids[start]), start=start, end=i, raw_identifier=f"d{int(doc_ids[start])}"))
                start = i
        creator = cdm.CrossDocLinkMaskCreator(link_detector=NoLinks())
        return creator.build_dense_mask_for_visualization(torch.zeros((1, t), dtype=torch.int64), spans)

    def step(q, k, v, dense, do):
        qa, ka, va = (x.clone().requires_grad_(True) for x in (q, k, v))
        out = torch.nn.functional.scaled_dot_product_attention(qa, ka, va, attn_mask=dense)
        out.backward(do)
        return out

    return dense_for, step


def cpu_baseline(steps: int):
    """The oracle (fp32 dense-masked attention forward + backward, the reference's CPU path restated) on host cores."""
    from oracle import attention as oattn
    torch.set_num_threads(os.cpu_count() or 1)
    dense, q, k, v, do, pairs, heads, t = cpu_sample()
    for _ in range(3):  # warm-ups
        oattn.forward_backward(q, k, v, dense, do)
    times = []
    for _ in range(max(5, steps)):
        t0 = time.perf_counter()
        oattn.forward_backward(q, k, v, dense, do)
        times.append(time.perf_counter() - t0)
    sec = statistics.median(times)
    return {"value": 14.0 * D * heads * pairs / sec / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"doc_causal pack, first {t} tokens, {heads} heads, fp32 dense-masked attention fwd+bwd, unmasked FLOPs credited",
            "sec_per_sample": sec, "timing": f"3 warm-ups, median of {len(times)}"}


def run_reference(args, rank, world):
    if rank != 0:
        return
    from oracle import attention as oattn
    torch.set_num_threads(os.cpu_count() or 1)
    dense, q, k, v, do, pairs, heads, t = cpu_sample()
    ref = reference_mask_and_step()
    kind = "port"
    run = lambda: oattn.forward_backward(q, k, v, dense, do)
    if ref is not None:
        from tagseq2tagseq_b200 import synth
        dense_for, step = ref
        ref_dense = dense_for(synth.config3_pack(SEED, "doc_causal").doc_ids[:t])
        if torch.equal(ref_dense, dense):  # the reference's own mask construction agrees with the port's
            kind = "reference"
            run = lambda: step(q, k, v, ref_dense, do)
    for _ in range(min(args.warmup, 2)):
        run()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        run()
    sec = time.perf_counter() - t0
    value = 14.0 * D * heads * pairs * args.steps / sec / 1e12
    base = {"value": value, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": kind,
            "sample": f"doc_causal pack, first {t} tokens, {heads} heads per step, fp32 dense-masked attention fwd+bwd"
                      + (" (reference mask code from baseline/_ref + torch SDPA autograd)" if kind == "reference" else " (oracle port)")}
    emit({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "attn_fwd_bwd_32k_mask_sweep", "B": B, "T": T, "H": H, "head_dim": D, "masks": MASKS,
                   "note": "CPU restatement of the reference's dense-masked attention, timed on a bounded sample of the workload"},
        "cpu_baseline": base, "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0})


def run_flex_gpu(args, rank, world, device):
    """The reference's GPU attention path on the same inputs, for comparison: torch.compile(flex_attention)
    (Inductor's Triton templates, reached from model/modules/layer.py:33) with a BlockMask from create_block_mask and
    a mask_mod equal to the reference's (cross_doc_mask.py:348-357) expressed over (doc ids, link bits).
    Library code only; none of this package's kernels run in this mode."""
    from torch.nn.attention.flex_attention import create_block_mask, flex_attention
    masks = make_workload(rank, device)
    torch.manual_seed(SEED + rank)
    q, k, v, do = (torch.randn(B, H, T, D, device=device, dtype=torch.float32).bfloat16() for _ in range(4))
    q.requires_grad_(True); k.requires_grad_(True); v.requires_grad_(True)
    compiled = torch.compile(flex_attention, dynamic=False)
    # The stock template configuration can exceed the 227 KB of shared memory at head_dim 128; smaller tiles are tried
    # in turn and the options that worked are reported.
    option_sets = [None, {"num_stages": 2}, {"BLOCK_M": 64, "BLOCK_N": 64, "BLOCK_M1": 32, "BLOCK_N1": 64, "BLOCK_M2": 64, "BLOCK_N2": 32},
                   {"BLOCK_M": 64, "BLOCK_N": 32, "BLOCK_M1": 32, "BLOCK_N1": 32, "BLOCK_M2": 32, "BLOCK_N2": 32, "num_stages": 1}]
    used_options = "unset"
    per_mask, tot_ms, tot_flops = [], 0.0, 0.0
    for m in masks:
        doc, link = m["doc"], m["link"]
        if link is None:
            def mask_mod(b, h, qi, ki, doc=doc):
                return (qi >= ki) & (doc[b, qi] == doc[b, ki])
        else:
            def mask_mod(b, h, qi, ki, doc=doc, link=link):
                dq_, dk_ = doc[b, qi], doc[b, ki]
                word = link[b, dq_, dk_ >> 6]
                return (qi >= ki) & ((dq_ == dk_) | (((word >> (dk_ & 63)) & 1) != 0))
        t0 = time.perf_counter()
        bm = create_block_mask(mask_mod, B, None, T, T, device=device, _compile=True)
        torch.cuda.synchronize(device)
        mask_s = time.perf_counter() - t0
        used_options = "unset"  # searched per mask: a mask_mod that captures more tensors needs more resources
        if used_options == "unset":
            errors = []
            for opts in option_sets:
                try:
                    torch._dynamo.reset()
                    out = compiled(q, k, v, block_mask=bm, kernel_options=opts)
                    out.backward(do)
                    torch.cuda.synchronize(device)
                    used_options = opts
                    break
                except Exception as exc:  # noqa: BLE001 - report and try the next configuration
                    errors.append(f"{opts}: {str(exc).splitlines()[0][:160]}")
            if used_options == "unset":
                emit({"impl": "flex_gpu", "unavailable": "no FlexAttention template configuration compiled: " + " | ".join(errors)})
                return
        for _ in range(3):
            out = compiled(q, k, v, block_mask=bm, kernel_options=used_options)
            out.backward(do)
        torch.cuda.synchronize(device)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(args.steps):
            out = compiled(q, k, v, block_mask=bm, kernel_options=used_options)
            out.backward(do)
        ev1.record()
        torch.cuda.synchronize(device)
        ms = ev0.elapsed_time(ev1) / args.steps
        per_mask.append({"mask": m["name"], "fwd_bwd_ms": ms, "tflops": flops_of(m["pairs"]) / ms / 1e9, "first_block_mask_s": mask_s,
                         "kernel_options": used_options})
        tot_ms += ms
        tot_flops += flops_of(m["pairs"])
    emit({"impl": "flex_gpu", "metric": METRIC, "value": tot_flops / tot_ms / 1e9, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
          "ms_per_step": tot_ms, "dtype": "bf16", "data": "synthetic", "higher_is_better": True,
          "config": {"workload": WORKLOAD, "B": B, "T": T, "H": H, "head_dim": D, "per_mask": per_mask,
                     "kernel_options": used_options,
                     "note": "torch.compile(flex_attention) fwd+bwd, block mask built once outside the timed region"}})


_REAL_STDOUT = None


def emit(obj) -> None:
    """The one JSON line goes to the process's original stdout; everything else (NCCL banners, warnings) was
    redirected to stderr in main()."""
    out = _REAL_STDOUT or sys.stdout
    out.write(json.dumps(obj) + "\n")
    out.flush()


def main():
    global _REAL_STDOUT
    _REAL_STDOUT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)  # libraries that print to fd 1 (e.g. the NCCL version banner) must not pollute the JSON line
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "flex_gpu"],
                    help="ours: this package's CUDA path.  reference: the reference's CPU path on a bounded sample.  "
                         "flex_gpu: PyTorch FlexAttention (the reference's GPU path) on the same inputs, single GPU.")
    ap.add_argument("--no-balance", action="store_true", help="training step: keep the seed order of packs instead of the density-aware schedule")
    ap.add_argument("--bucket-mb", type=int, default=256, help="training step: DDP bucket size in MB (the reference uses 256, main.py:414)")
    ap.add_argument("--fp32-buckets", action="store_true", help="training step: all-reduce fp32 gradient buckets (default: bf16-compressed)")
    ap.add_argument("--no-train", action="store_true", help="skip the short training-step measurement appended to the 32k line")
    ap.add_argument("--workload", default="32k", choices=["32k", "16k", "train4", "train5"],
                    help="32k: the headline mask sweep (default).  16k: B=1, T=16384, H=16, cross_doc_link p=0.15 "
                         "(the single-GPU 16k configuration; small enough for an ncu capture)")
    args = ap.parse_args()
    if args.workload == "16k":
        global B, T, MASKS, SEED, WORKLOAD
        B, T, MASKS, SEED, WORKLOAD = 1, 16384, ["link_p15"], 1002, "attn_fwd_bwd_16k_cross_doc_link"
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU implementation (use --impl reference for the CPU arm)")
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.distributed.init_process_group("nccl", device_id=device)
    try:
        if args.impl == "flex_gpu":
            if rank == 0:
                run_flex_gpu(args, rank, 1, device)
        elif args.workload in ("train4", "train5"):
            res = run_train(args, rank, world, device, args.workload, steps=args.steps, warmup=max(3, args.warmup))
            if rank == 0:
                res.update({"n_gpus": world, "warmup": max(3, args.warmup), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                            "dtype": "bf16", "data": "synthetic", "config": {"workload": args.workload}})
                emit(res)
        else:
            run_ours(args, rank, world, device)
    finally:
        if world > 1:
            torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
