"""Host-side mask adapters of the package against reference-generated fixtures (CPU only)."""
import math

import numpy as np
import pytest
import torch

from oracle import masks as om
from tagseq2tagseq_b200 import mask_spec as ms
from tagseq2tagseq_b200 import synth
from tests import _golden as G

GRANTS = G.grant_cases()


@pytest.mark.parametrize("entry", GRANTS, ids=[e["name"] for e in GRANTS])
def test_grant_classes_equal_reference_bitmask_mask(entry):
    """(row class, column class, link bits) must describe exactly the mask the reference's int64 bitmasks
    describe -- including the grants dropped by the cap (cross_doc_mask.py:239-257)."""
    arrs = G.grant_arrays()
    spans, links, t = G.spans_of(entry), G.links_of(entry), entry["seq_len"]
    cap = entry["cap"] if entry["cap"] is not None else entry["max_grants"]
    ids = ms.build_document_ids(t, spans)
    assert np.array_equal(ids, om.document_ids(t, spans))
    ref = om.cross_doc_link_dense(ids, arrs[f"{entry['name']}/q_bits"], arrs[f"{entry['name']}/kv_bits"])
    grants = ms.ordered_grants(t, spans, links, cap)
    if grants:
        row, col, link = ms.grant_classes(t, grants)
        mine = om.class_mask_dense(ids, row, col, link)
    else:
        mine = om.doc_causal_dense(ids)
    assert np.array_equal(mine, ref)


def test_warmup_schedule_matches_reference_formula():
    # cross_doc_mask.py:76-85: cosine ascent from start to max over warmup steps
    c = ms.CrossDocLinkMaskCreator(link_detector=None, max_grants=256, max_grants_start=16, max_grants_warmup_steps=100)
    for step in (0, 1, 37, 50, 99, 100, 500):
        c._step = step
        if step >= 100:
            exp = 256
        else:
            exp = round(16 + (256 - 16) * (1.0 - math.cos(math.pi * step / 100)) / 2.0)
        assert c._current_max_grants() == exp
    assert ms.CrossDocLinkMaskCreator(None, max_grants=200)._n_chunks == 4
    assert ms.CrossDocLinkMaskCreator(None)._current_max_grants() == 64


def test_match_links_enforces_dag():
    # tests/model/graph_traversal/test_cross_doc_mask.py:79-100
    class Det:
        def index_doc_span(self, span):
            return span.raw_identifier
    spans = [ms.DocSpan(0, "a", 0, 10, raw_identifier="A"), ms.DocSpan(1, "b", 10, 30, raw_identifier="B")]
    c = ms.CrossDocLinkMaskCreator(Det())
    links = [ms.LinkInfo(5, "B"), ms.LinkInfo(15, "A"), ms.LinkInfo(15, "missing"), ms.LinkInfo(20, "A")]
    assert c._match_links_to_docs(links, spans) == {15: [0], 20: [0]}


def test_registry_behaviour():
    # the same four names, in the same order, as the reference's registry (block_mask_creator.py:251-256)
    assert ms.list_mask_creators() == ["doc_causal", "causal", "full", "doc_bidirectional"]
    with pytest.raises(ValueError, match="Unknown mask creator"):
        ms.get_mask_creator("sliding")
    for name in ("full", "doc_bidirectional"):  # known names whose masks the causal kernels cannot compute
        with pytest.raises(NotImplementedError, match="non-causal"):
            ms.get_mask_creator(name)(torch.zeros((1, 8), dtype=torch.int64), [])
    fn = ms.make_mask_creator_callable("doc_causal")
    with pytest.raises(ValueError, match="tokens"):
        fn(doc_spans=[])


def test_synthetic_generator_is_seeded_and_counts_pairs():
    a, b = synth.config2_pack(), synth.config2_pack()
    assert np.array_equal(a.doc_ids, b.doc_ids) and np.array_equal(a.link_bits, b.link_bits)
    assert a.seq_len == 16384 and a.lengths.sum() == 16384 and a.lengths.min() >= 1
    p = synth.make_pack(5, 1500, 60, 4, 400, p_link=0.3)
    dense = om.class_mask_dense(p.doc_ids, None, None, p.link_bits)
    assert int(dense.sum()) == p.unmasked_pairs()
    p1 = synth.config1_pack()
    assert p1.seq_len == 2048 and p1.link_bits is None
    doc, link = synth.stack_packs([synth.make_pack(1, 512, 50, 4, 100, p_link=0.5), synth.make_pack(2, 512, 20, 4, 100, p_link=0.5)])
    assert doc.shape == (2, 512) and link.shape[0] == 2 and link.dtype == np.int64


@pytest.mark.parametrize("seed", range(60))
def test_fuzz_reference_format_adapter_against_oracle(seed):
    """Random spans (gaps, clipping, repeated doc ids), random links (several targets per position, unknown targets,
    positions outside every span) and random caps: the adapter's (row, col, link bits) must give the same mask as the
    oracle's restatement of the reference bitmask construction."""
    from types import SimpleNamespace
    rng = np.random.default_rng(7000 + seed)
    n_docs = int(rng.integers(1, 12))
    spans, pos = [], -int(rng.integers(0, 4))
    for d in range(n_docs):
        pos += int(rng.choice([0, 0, 1, 4]))
        w = int(rng.integers(1, 60))
        doc_id = d if rng.random() > 0.1 else int(rng.integers(0, max(1, d)))  # occasionally a repeated id
        spans.append(SimpleNamespace(doc_id=doc_id, start=pos, end=pos + w, raw_identifier=f"d{d}"))
        pos += w
    seq_len = max(1, pos - int(rng.choice([0, 0, 3, 17])))
    links = {}
    for _ in range(int(rng.integers(0, 40))):
        lp = int(rng.integers(0, pos + 3))
        links.setdefault(lp, []).append(int(rng.integers(0, n_docs + 1)))
    max_grants = int(rng.choice([64, 128, 256]))
    cap = int(rng.choice([max_grants, max_grants, 3, 1, 10]))
    ids = ms.build_document_ids(seq_len, spans)
    qb, kb = om.grant_bitmasks(seq_len, spans, links, max_grants=max_grants, cap=cap)
    ref = om.cross_doc_link_dense(om.document_ids(seq_len, spans), qb, kb)
    grants = ms.ordered_grants(seq_len, spans, links, cap)
    if grants:
        row, col, link = ms.grant_classes(seq_len, grants)
        mine = om.class_mask_dense(ids, row, col, link)
    else:
        mine = om.doc_causal_dense(ids)
    assert np.array_equal(mine, ref)


def _dense_from_classes(row, col, link, t):
    lu = np.ascontiguousarray(link).view(np.uint64)
    m = np.zeros((t, t), dtype=bool)
    for q in range(t):
        if row[q] < 0:
            continue
        words = lu[int(row[q])]
        for k in range(t):
            c = int(col[k])
            m[q, k] = c >= 0 and bool((int(words[c >> 6]) >> (c & 63)) & 1)
    return m


def _expand_segments(bounds, ids, t):
    out = np.full(t, -1, dtype=np.int32)
    for j in range(len(ids)):
        out[bounds[j]:bounds[j + 1]] = ids[j]
    return out


@pytest.mark.parametrize("seed", range(12))
def test_grant_segments_describe_the_same_mask_as_grant_classes(seed):
    """Classes worked out on the <= 2G+1 segment boundaries (what the device fill consumes) against the per-token
    construction, on random, overlapping and duplicate grants."""
    rng = np.random.default_rng(seed)
    t = int(rng.integers(20, 120))
    grants = []
    for _ in range(int(rng.integers(0, 80))):
        q0 = int(rng.integers(0, t - 1)); q1 = int(rng.integers(q0 + 1, t + 1))
        k0 = int(rng.integers(0, t - 1)); k1 = int(rng.integers(k0 + 1, t + 1))
        grants.append((q0, q1, k0, k1))
    if grants and seed % 3 == 0:
        grants.append(grants[0])
    row, col, link = ms.grant_classes(t, grants)
    (qb, qi), (kb, ki), link2 = ms.grant_segments(grants)
    assert len(qi) <= 2 * len(grants) + 1 and len(ki) <= 2 * len(grants) + 1
    a = _dense_from_classes(row, col, link, t)
    b = _dense_from_classes(_expand_segments(qb, qi, t), _expand_segments(kb, ki, t), link2, t)
    assert np.array_equal(a, b)


def test_decoder_layer_wrappers_refuse_cpu_tensors():
    import pytest
    import torch
    from tagseq2tagseq_b200 import lm_fused
    x = torch.zeros(4, 128)
    with pytest.raises(RuntimeError, match="CUDA"):
        lm_fused.add_rmsnorm(x, None, torch.ones(128), 1e-6)
    with pytest.raises(RuntimeError, match="CUDA"):
        lm_fused.swiglu(torch.zeros(4, 256, dtype=torch.bfloat16))
    with pytest.raises(RuntimeError, match="CUDA"):
        lm_fused.cross_entropy(torch.zeros(4, 512, dtype=torch.bfloat16), torch.zeros(4, dtype=torch.int64))
    cos, sin = lm_fused.rope_half_tables(5, 64, 10000.0, "cpu")
    assert cos.shape == (5, 32) and sin.shape == (5, 32) and float(cos[0, 0]) == 1.0 and float(sin[0, 0]) == 0.0
