"""Generate the golden fixtures in this directory by running the reference itself.

Run once, in a container where the reference checkout is importable:

    python tests/golden/make_golden.py /path/to/tagseq2tagseq

It imports the reference's own mask code (model/graph_traversal/cross_doc_mask.py
and block_mask_creator.py) with bare namespace stubs for the packages that are
not installed (``model/__init__`` needs tunalab; block_mask_creator imports
matplotlib and the data package at module level), feeds it span / link tables and
stores what it returns:

* ``grants.npz``    -- ``_build_grant_bitmasks`` and ``_build_cross_doc_mask``
  outputs for hand-written scenarios (the span/link tables of
  tests/model/graph_traversal/test_grant_bitmask_equivalence.py:115-240 and the
  capacity scenario of :80-99) plus seeded random scenarios that also cover
  clipped spans, unknown targets and links outside every span.
* ``blockmaps.npz`` -- the ``BlockMask`` index tensors that the reference's
  ``create_doc_causal_block_mask`` and ``CrossDocLinkMaskCreator.__call__``
  return on CPU, for several sequence lengths including ragged ones.
* ``flex_fwd.npz``  -- out / lse of PyTorch's eager FlexAttention forward run
  with those reference BlockMasks on seeded q, k, v (no CPU backward exists).

The tests never import the reference; they read these files.
"""
from __future__ import annotations

import importlib.util
import json
import os
import random
import sys
import types
from dataclasses import dataclass, field
from typing import Dict, List

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


@dataclass
class Span:
    doc_id: int
    raw_identifier: str
    start: int
    end: int
    truncated: bool = False
    outgoing_identifiers: List[str] = field(default_factory=list)
    normed_identifier: str = ""


def load_reference(ref_root: str):
    def stub(name, **attrs):
        m = types.ModuleType(name)
        m.__path__ = []  # behave like a package
        for k, v in attrs.items():
            setattr(m, k, v)
        sys.modules[name] = m
        return m

    def load(name, rel):
        spec = importlib.util.spec_from_file_location(name, os.path.join(ref_root, rel))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod
        spec.loader.exec_module(mod)
        return mod

    stub("model")
    stub("model.graph_traversal")
    load("model.graph_traversal.link_detector", "model/graph_traversal/link_detector.py")
    cdm = load("model.graph_traversal.cross_doc_mask", "model/graph_traversal/cross_doc_mask.py")
    # block_mask_creator pulls matplotlib and the data package at import time
    stub("matplotlib")
    stub("matplotlib.pyplot")
    anything = type("Anything", (), {})
    stub("data")
    stub("data.pack_sampler", PackBatchSampler=anything)
    stub("data.dataset", GraphIndex=anything, PretokShardedBackend=anything)
    stub("data.layout", NullLayoutPolicy=anything)
    stub("data.collate", build_packed_batch=anything)
    stub("data.traversal", BFSStrategy=anything, DFSStrategy=anything, RandomWalkStrategy=anything,
         RandomSelectionStrategy=anything, CompositeTraversalStrategy=anything)
    bmc = load("model.graph_traversal.block_mask_creator", "model/graph_traversal/block_mask_creator.py")
    return cdm, bmc


class TableDetector:
    """Returns preset links; spans are matched on raw_identifier like the default protocol."""

    def __init__(self, links):
        self.links = links

    def detect_links(self, input_ids):
        return list(self.links)

    def index_doc_span(self, span):
        return span.raw_identifier


# --- scenario tables ---------------------------------------------------------------------------

def hand_scenarios():
    """(name, seq_len, [(doc_id,start,end)], {link_pos:[targets]}, max_grants)."""
    S = []
    S.append(("empty_no_links", 20, [(0, 0, 10), (1, 10, 20)], {}, 64))
    S.append(("single_grant", 16, [(0, 0, 5), (1, 5, 16)], {8: [0]}, 64))
    S.append(("two_nonoverlapping", 30, [(0, 0, 5), (1, 5, 15), (2, 15, 30)], {10: [0], 20: [1]}, 64))
    S.append(("overlapping_q", 30, [(0, 0, 5), (1, 5, 10), (2, 10, 30)], {15: [0], 18: [1]}, 64))
    S.append(("overlapping_kv", 30, [(0, 0, 5), (1, 5, 15), (2, 15, 30)], {10: [0], 20: [0]}, 64))
    S.append(("link_at_span_end", 20, [(0, 0, 5), (1, 5, 12)], {12: [0]}, 64))
    S.append(("link_before_span_end", 20, [(0, 0, 5), (1, 5, 12)], {11: [0]}, 64))
    S.append(("three_doc_chain", 30, [(0, 0, 8), (1, 8, 18), (2, 18, 30)], {12: [0], 22: [0], 25: [1]}, 64))
    S.append(("link_outside_spans", 20, [(0, 0, 5), (1, 5, 10)], {15: [0]}, 64))
    # capacity: one 4-token target, n sources of 4 tokens, each linking at start+1
    for n, mg in [(64, 64), (65, 64), (128, 128), (129, 128), (256, 256), (257, 256), (65, 128), (129, 256)]:
        spans = [(0, 0, 4)] + [(i, 4 * i, 4 * i + 4) for i in range(1, n + 1)]
        links = {4 * i + 1: [0] for i in range(1, n + 1)}
        S.append((f"capacity_{n}_of_{mg}", 4 + 4 * n, spans, links, mg))
    # spans reaching past the sequence end and before 0, multi-target link, unknown target, capped below max
    S.append(("clipped_spans", 40, [(0, -3, 9), (1, 9, 25), (2, 25, 47)], {12: [0], 30: [0, 1], 44: [1]}, 64))
    S.append(("unknown_target", 24, [(0, 0, 6), (1, 6, 24)], {9: [7], 11: [0]}, 64))
    return S


def random_scenario(rng: random.Random):
    n_docs = rng.randint(2, 9)
    widths = [rng.randint(1, 40) for _ in range(n_docs)]
    gap = [rng.choice([0, 0, 0, 1, 3]) for _ in range(n_docs)]  # uncovered tokens keep id -1
    spans, pos = [], 0
    for d, (w, g) in enumerate(zip(widths, gap)):
        pos += g
        spans.append((d, pos, pos + w))
        pos += w
    seq_len = pos - rng.choice([0, 0, 1, 5]) if pos > 8 else pos
    links: Dict[int, List[int]] = {}
    for _ in range(rng.randint(0, 14)):
        src = rng.randint(1, n_docs - 1)
        lp = rng.randint(spans[src][1], spans[src][2] + 1)
        links.setdefault(lp, []).append(rng.randint(0, src - 1))
    return seq_len, spans, links


def pack(a: np.ndarray) -> np.ndarray:
    return np.packbits(a.astype(np.uint8).reshape(-1))


def main(ref_root: str):
    cdm, bmc = load_reference(ref_root)
    out: Dict[str, np.ndarray] = {}
    meta = []

    def run_grants(name, seq_len, spans_t, links, max_grants, cap=None):
        spans = [Span(d, f"doc_{d}", a, b) for d, a, b in spans_t]
        cr = cdm.CrossDocLinkMaskCreator(link_detector=object(), max_grants=max_grants)
        dev = torch.device("cpu")
        dense = cr._build_cross_doc_mask(seq_len, spans, links, dev)
        qb, kb = cr._build_grant_bitmasks(seq_len, spans, links, dev, max_grants_cap=cap)
        out[f"{name}/q_bits"] = torch.stack(qb).numpy()
        out[f"{name}/kv_bits"] = torch.stack(kb).numpy()
        out[f"{name}/cross_dense"] = pack(dense.numpy())
        meta.append({"name": name, "seq_len": seq_len, "spans": spans_t,
                     "links": {str(k): v for k, v in links.items()}, "max_grants": max_grants, "cap": cap})

    for name, seq_len, spans_t, links, mg in hand_scenarios():
        run_grants(name, seq_len, spans_t, links, mg)
    run_grants("three_doc_chain_cap2", 30, [(0, 0, 8), (1, 8, 18), (2, 18, 30)], {12: [0], 22: [0], 25: [1]}, 64, cap=2)
    for seed in range(40):
        seq_len, spans_t, links = random_scenario(random.Random(1000 + seed))
        run_grants(f"fuzz_{seed}", seq_len, spans_t, links, 64)
    np.savez_compressed(os.path.join(HERE, "grants.npz"), **out)
    with open(os.path.join(HERE, "grants.json"), "w") as f:
        json.dump(meta, f)

    # --- block maps straight from the reference creators (CPU BlockMask) -------------------------
    bm_out: Dict[str, np.ndarray] = {}
    bm_meta = []
    fx_out: Dict[str, np.ndarray] = {}

    def docs_for(seq_len, rng, lo, hi, overshoot=0):
        spans, pos, d = [], 0, 0
        while pos < seq_len + overshoot:
            w = rng.randint(lo, hi)
            spans.append((d, pos, pos + w))
            pos += w
            d += 1
        return spans

    def save_bm(name, bm):
        for fld in ["kv_num_blocks", "kv_indices", "full_kv_num_blocks", "full_kv_indices",
                    "q_num_blocks", "q_indices", "full_q_num_blocks", "full_q_indices"]:
            bm_out[f"{name}/{fld}"] = getattr(bm, fld)[0, 0].numpy()

    cases = [("t300", 300, 7, 20, 150), ("t640", 640, 8, 30, 400), ("t1000", 1000, 9, 5, 260),
             ("t2047", 2047, 10, 16, 512), ("t2048", 2048, 11, 16, 512), ("t129", 129, 12, 40, 90),
             ("t128", 128, 13, 128, 128), ("t1", 1, 14, 1, 1), ("t1536_long", 1536, 15, 300, 900)]
    for name, seq_len, seed, lo, hi in cases:
        rng = random.Random(seed)
        spans_t = docs_for(seq_len, rng, lo, hi, overshoot=rng.choice([0, 17]))
        spans = [Span(d, f"doc_{d}", a, b) for d, a, b in spans_t]
        tokens = torch.zeros((1, seq_len), dtype=torch.int64)
        # doc_causal through the reference's registry wrapper (block_mask_creator.py:288-334)
        bm = bmc.make_mask_creator_callable("doc_causal")(tokens=tokens, doc_spans=spans)
        save_bm(f"{name}/doc_causal", bm)
        # cross_doc_link through CrossDocLinkMaskCreator.__call__ with preset links
        links = []
        for d, a, b in spans_t[1:]:
            for _ in range(rng.randint(0, 3)):
                lp = rng.randint(a + 1, b)
                links.append(cdm.LinkInfo(link_end_pos=lp, target_str=f"doc_{rng.randint(0, d - 1)}"))
        creator = cdm.CrossDocLinkMaskCreator(link_detector=TableDetector(links), max_grants=256)
        bm2 = bmc.make_mask_creator_callable_from(creator)(tokens=tokens, doc_spans=spans)
        save_bm(f"{name}/cross_doc_link", bm2)
        ltt = creator._match_links_to_docs(links, spans)
        dense = creator.build_dense_mask_for_visualization(tokens, spans)
        bm_out[f"{name}/cross_doc_link/dense"] = pack(dense.numpy())
        bm_meta.append({"name": name, "seq_len": seq_len, "spans": spans_t,
                        "links": {str(k): v for k, v in ltt.items()}, "max_grants": 256})
        if name == "t300":
            from torch.nn.attention.flex_attention import flex_attention
            g = torch.Generator().manual_seed(seed)
            q, k, v = (torch.randn(1, 2, seq_len, 64, generator=g) for _ in range(3))
            for mname, m in (("doc_causal", bm), ("cross_doc_link", bm2)):
                o, lse = flex_attention(q, k, v, block_mask=m, return_lse=True)
                fx_out[f"{name}/{mname}/out"] = o.numpy()
                fx_out[f"{name}/{mname}/lse"] = lse.numpy()
            fx_out[f"{name}/q"], fx_out[f"{name}/k"], fx_out[f"{name}/v"] = q.numpy(), k.numpy(), v.numpy()
    np.savez_compressed(os.path.join(HERE, "blockmaps.npz"), **bm_out)
    with open(os.path.join(HERE, "blockmaps.json"), "w") as f:
        json.dump(bm_meta, f)
    np.savez_compressed(os.path.join(HERE, "flex_fwd.npz"), **fx_out)
    print("wrote", len(out), "grant arrays,", len(bm_out), "block-map arrays,", len(fx_out), "flex arrays")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path to a tagseq2tagseq checkout>")
    main(sys.argv[1])
