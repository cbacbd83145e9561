"""Generate ``links.json`` by running the reference's own MarkdownLinkDetector.

    python tests/golden/make_golden_links.py /path/to/tagseq2tagseq

The reference module (model/graph_traversal/markdown_link_detector.py) is imported with bare namespace stubs
for its parent packages, given the synthetic byte-level vocabulary of tests/_synthvocab.py as ``decode_fn``, and run
on seeded synthetic token streams plus a few hand-written edge cases.  Stored per case: the tokens, the window and
the links the reference returned.  The tests read the file; they never import the reference.
"""
from __future__ import annotations

import importlib.util
import json
import os
import random
import sys
import types

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import _synthvocab as sv  # noqa: E402


def load_reference(ref_root: str):
    for name in ("model", "model.graph_traversal"):
        m = types.ModuleType(name)
        m.__path__ = []
        sys.modules[name] = m

    def load(name, rel):
        spec = importlib.util.spec_from_file_location(name, os.path.join(ref_root, rel))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod
        spec.loader.exec_module(mod)
        return mod

    load("model.graph_traversal.link_detector", "model/graph_traversal/link_detector.py")
    return load("model.graph_traversal.markdown_link_detector", "model/graph_traversal/markdown_link_detector.py")


def hand_cases():
    V = sv.VOCAB.index
    a, sp = 97, 32
    C = []
    C.append(("plain", 50, [257, a, MIDT, V(b"Foo"), V(b")")]))
    C.append(("no_start", 50, [a, a, MIDT, V(b"Foo"), V(b")")]))
    C.append(("start_at_100", 50, [257] + [a] * 99 + [MIDT, V(b"Foo"), V(b")")]))
    C.append(("start_at_101", 50, [257] + [a] * 100 + [MIDT, V(b"Foo"), V(b")")]))
    C.append(("nearest_start_wins", 50, [258, a, 257, a, MIDT, V(b"Bar"), V(b").")]))
    C.append(("close_inside_token", 50, [257, a, MIDT, V(b"Page"), V(b"s)"), a]))
    C.append(("close_first_of_two", 50, [257, a, MIDT, V(b"Page"), V(b"a)b"), V(b")")]))
    C.append(("empty_target", 50, [257, a, MIDT, V(b")"), V(b"Foo"), V(b")")]))
    C.append(("blank_target", 50, [257, a, MIDT, sp, V(b"  "), V(b" )")]))
    C.append(("nbsp_split_target", 50, [257, a, MIDT, V(b"\xc2"), V(b"\xa0"), V(b")")]))
    C.append(("split_utf8_target", 50, [257, a, MIDT, V(b"\xc3"), V(b"\xa9"), V(b")")]))
    C.append(("window_hit", 4, [257, a, MIDT, a, a, a, V(b")")]))
    C.append(("window_miss", 3, [257, a, MIDT, a, a, a, V(b")")]))
    C.append(("cut_by_end", 50, [257, a, MIDT, V(b"Foo")]))
    C.append(("mid_at_zero", 50, [MIDT, V(b"Foo"), V(b")")]))
    C.append(("mid_last", 50, [257, a, MIDT]))
    C.append(("two_mids", 50, [257, a, MIDT, MIDT, V(b"Foo"), V(b")"), V(b")")]))
    C.append(("paren_pair_token", 50, [257, a, MIDT, V(b"Foo"), V(b"()"), a]))
    return C


MIDT = sv.MID


def main(ref_root: str):
    mod = load_reference(ref_root)
    cases = []

    def run(name, window, toks):
        det = mod.MarkdownLinkDetector(sv.decode, window_tokens=window, link_start_token_ids=sv.STARTS, link_mid_token_id=sv.MID)
        links = det.detect_links(torch.tensor(toks, dtype=torch.long))
        cases.append({"name": name, "window": window, "tokens": toks, "links": [[l.link_end_pos, l.target_str] for l in links]})

    for name, window, toks in hand_cases():
        run(name, window, toks)
    for seed in range(12):
        rng = random.Random(4000 + seed)
        window = rng.choice([5, 12, 50])
        T = rng.choice([64, 300, 1000, 2500])
        run(f"stream_{seed}", window, sv.random_stream(rng, T, window))
    with open(os.path.join(HERE, "links.json"), "w") as f:
        json.dump({"cases": cases}, f)
    n_links = sum(len(c["links"]) for c in cases)
    print(f"wrote {len(cases)} cases, {n_links} links")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden_links.py <path to a tagseq2tagseq checkout>")
    main(sys.argv[1])
