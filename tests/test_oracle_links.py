"""CPU: the link-scan oracle against the fixtures produced by the reference's MarkdownLinkDetector."""
import json
import os

import pytest

import _synthvocab as sv
from oracle import link_detect as old

CASES = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "links.json")))["cases"]


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_oracle_matches_reference_links(case):
    got = old.detect_links(case["tokens"], sv.decode, mid_id=sv.MID, start_ids=sv.STARTS, window=case["window"])
    assert [[p, s] for p, s in got] == case["links"]


def test_fixture_covers_the_edge_cases():
    by_name = {c["name"]: c for c in CASES}
    assert by_name["start_at_100"]["links"] and not by_name["start_at_101"]["links"]
    assert by_name["window_hit"]["links"] and not by_name["window_miss"]["links"]
    assert not by_name["empty_target"]["links"] and not by_name["nbsp_split_target"]["links"]
    assert sum(len(c["links"]) for c in CASES) > 100


def test_candidates_are_a_superset_in_order():
    for case in CASES:
        cands = old.candidates(case["tokens"], sv.decode, mid_id=sv.MID, start_ids=sv.STARTS, window=case["window"])
        assert cands == sorted(cands)
        ends = [c[2] + 1 for c in cands]
        for end, _ in case["links"]:
            assert end in ends
        for mid, start, close in cands:
            assert case["tokens"][mid] == sv.MID and case["tokens"][start] in sv.STARTS and 0 < mid - start <= 100
            assert mid < close <= mid + case["window"]


def test_per_token_close_table_is_exact_for_a_byte_level_vocabulary():
    # the device scan replaces "the decoded window contains ')'" by a per-token flag
    for tok, raw in enumerate(sv.VOCAB):
        assert (")" in sv.decode([tok])) == (b")" in raw)
