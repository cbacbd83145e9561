"""GPU: ts2ts_detect_links through the MarkdownLinkDetector mirror, against the reference fixtures and the oracle."""
import json
import os
import random

import pytest
import torch

import _synthvocab as sv
from oracle import link_detect as old

pytestmark = pytest.mark.gpu
CASES = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "links.json")))["cases"]


def detector(window):
    from tagseq2tagseq_b200.link_detect import MarkdownLinkDetector
    return MarkdownLinkDetector(sv.decode, window_tokens=window, link_start_token_ids=sv.STARTS, link_mid_token_id=sv.MID,
                                vocab_size=len(sv.VOCAB))


@pytest.mark.parametrize("dtype", [torch.int64, torch.int32])
def test_links_equal_the_reference_fixtures(dtype):
    dets = {}
    for case in CASES:
        det = dets.setdefault(case["window"], detector(case["window"]))
        ids = torch.tensor(case["tokens"], dtype=dtype, device="cuda")
        got = det.detect_links(ids)
        assert [[l.link_end_pos, l.target_str] for l in got] == case["links"], case["name"]


def test_candidate_triples_equal_the_oracle():
    for case in CASES:
        det = detector(case["window"])
        ids = torch.tensor(case["tokens"], dtype=torch.int64, device="cuda")
        want = old.candidates(case["tokens"], sv.decode, mid_id=sv.MID, start_ids=sv.STARTS, window=case["window"])
        assert det.candidates(ids) == want, case["name"]


def test_long_stream_and_output_growth():
    # 32768 tokens with more candidates than the first output buffer holds
    rng = random.Random(7)
    toks = []
    while len(toks) < 32768:
        toks += [sv.STARTS[rng.randrange(2)], 97 + rng.randrange(26), sv.MID, 97 + rng.randrange(26), sv.CLOSERS[rng.randrange(len(sv.CLOSERS))]]
        toks += [97 + rng.randrange(26) for _ in range(rng.randrange(12))]
    toks = toks[:32768]
    det = detector(50)
    want = old.candidates(toks, sv.decode, mid_id=sv.MID, start_ids=sv.STARTS, window=50)
    assert len(want) > 1024
    ids = torch.tensor(toks, dtype=torch.int64, device="cuda")
    assert det.candidates(ids) == want
    assert [(l.link_end_pos, l.target_str) for l in det.detect_links(ids)] == old.detect_links(toks, sv.decode, sv.MID, sv.STARTS, 50)


def test_feeds_the_cross_doc_mask_creator():
    from tagseq2tagseq_b200 import CrossDocLinkMaskCreator, DocSpan, from_reference
    V = sv.VOCAB.index
    # doc 0 "Foo" [0,6), doc 1 "Bar" [6,14), doc 2 [14,30) links to Foo and to an unknown page
    toks = [97] * 14 + [257, 98, sv.MID, V(b"Foo"), V(b")"), 99, 258, 98, sv.MID, V(b"wiki"), V(b")"), 100, 257, sv.MID, V(b"Bar"), V(b").")]
    spans = [DocSpan(0, "foo", 0, 6, False, [], "Foo"), DocSpan(1, "bar", 6, 14, False, [], "Bar"),
             DocSpan(2, "baz", 14, 30, False, ["Foo", "Bar"], "Baz")]
    ids = torch.tensor([toks], dtype=torch.int64, device="cuda")
    creator = CrossDocLinkMaskCreator(link_detector=detector(50), max_grants=64)
    spec = creator(ids, spans)
    links = old.detect_links(toks, sv.decode, sv.MID, sv.STARTS, 50)
    assert links == [(19, "Foo"), (25, "wiki"), (30, "Bar")]
    want = from_reference(spans, {19: [0], 30: [1]}, len(toks), max_grants_cap=64, device=ids.device)
    assert torch.equal(spec.doc_ids, want.doc_ids) and torch.equal(spec.link_bits, want.link_bits)
    assert torch.equal(spec.q_row_ids, want.q_row_ids) and torch.equal(spec.kv_col_ids, want.kv_col_ids)


def test_argument_errors():
    det = detector(50)
    with pytest.raises(RuntimeError):
        det.detect_links(torch.tensor([1, 2, 3]))
    with pytest.raises(ValueError):
        det.detect_links(torch.zeros((2, 3), dtype=torch.int64, device="cuda"))
    with pytest.raises(TypeError):
        det.detect_links(torch.zeros(3, dtype=torch.float32, device="cuda"))
    assert det.detect_links(torch.zeros(0, dtype=torch.int64, device="cuda")) == []
