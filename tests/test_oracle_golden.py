"""The CPU oracle against outputs of the reference itself (tests/golden/*.npz)."""
import numpy as np
import pytest
import torch

from oracle import attention as oattn
from oracle import block_map as obm
from oracle import masks as om
from tests import _golden as G

GRANTS = G.grant_cases()
BLOCKS = G.blockmap_cases()


@pytest.mark.parametrize("entry", GRANTS, ids=[e["name"] for e in GRANTS])
def test_grant_bitmasks_match_reference(entry):
    arrs = G.grant_arrays()
    spans, links, t = G.spans_of(entry), G.links_of(entry), entry["seq_len"]
    qb, kb = om.grant_bitmasks(t, spans, links, max_grants=entry["max_grants"], cap=entry["cap"])
    assert np.array_equal(qb, arrs[f"{entry['name']}/q_bits"])
    assert np.array_equal(kb, arrs[f"{entry['name']}/kv_bits"])
    dense = om.cross_doc_dense(t, spans, links)
    assert np.array_equal(dense, G.unpack(arrs[f"{entry['name']}/cross_dense"], (t, t)))
    # reference test property: bitmask form == dense form unless the cap truncated
    # (tests/model/graph_traversal/test_grant_bitmask_equivalence.py:360-408)
    n_valid = sum(1 for lp, ts in links.items() for tg in ts
                  if (g := om._find_grant(t, spans, lp, tg)) is not None and g[0] < g[1] and g[2] < g[3])
    cap = entry["cap"] if entry["cap"] is not None else entry["max_grants"]
    if n_valid <= cap:
        assert np.array_equal(om.bitmask_grant_dense(qb, kb), dense)
    elif entry["name"].startswith("capacity"):
        assert not np.array_equal(om.bitmask_grant_dense(qb, kb), dense)


def test_reference_spot_checks():
    # tests/model/graph_traversal/test_grant_bitmask_equivalence.py:128-147,203-218
    sp = [type("S", (), dict(doc_id=0, start=0, end=5)), type("S", (), dict(doc_id=1, start=5, end=16))]
    d = om.cross_doc_dense(16, sp, {8: [0]})
    assert d[8, 2] and not d[5, 2]
    sp = [type("S", (), dict(doc_id=0, start=0, end=5)), type("S", (), dict(doc_id=1, start=5, end=12))]
    assert not om.cross_doc_dense(20, sp, {12: [0]}).any()
    d = om.cross_doc_dense(20, sp, {11: [0]})
    assert d[11, 2] and not d[10, 2]


@pytest.mark.parametrize("entry", BLOCKS, ids=[e["name"] for e in BLOCKS])
@pytest.mark.parametrize("mask", ["doc_causal", "cross_doc_link"])
def test_block_map_matches_reference_blockmask(entry, mask):
    arrs = G.blockmap_arrays()
    spans, links, t = G.spans_of(entry), G.links_of(entry), entry["seq_len"]
    ids = om.document_ids(t, spans)
    if mask == "doc_causal":
        dense = om.doc_causal_dense(ids)
    else:
        qb, kb = om.grant_bitmasks(t, spans, links, max_grants=entry["max_grants"])
        dense = om.cross_doc_link_dense(ids, qb, kb)
        ref_dense = G.unpack(arrs[f"{entry['name']}/cross_doc_link/dense"], (t, t))
        assert np.array_equal(om.visualization_dense(t, spans, links), ref_dense)
        assert np.array_equal(dense, ref_dense)  # no fixture exceeds the cap
        assert not np.triu(dense, 1).any() and dense.diagonal().all()  # test_cross_doc_mask.py:103-125
    st = obm.block_states(dense)
    prefix = f"{entry['name']}/{mask}"
    n = st.shape[0]
    assert np.array_equal(st, G.blockmask_to_states(arrs, prefix, n))
    lists = obm.lists_from_states(st)
    for mine, cnt_name, idx_name in [("kv", "kv_num_blocks", "kv_indices"), ("full", "full_kv_num_blocks", "full_kv_indices"),
                                     ("q", "q_num_blocks", "q_indices"), ("full_q", "full_q_num_blocks", "full_q_indices")]:
        cnt = lists[f"{mine}_cnt"]
        assert np.array_equal(cnt, arrs[f"{prefix}/{cnt_name}"])
        for r in range(n):  # entries past the count are argsort filler in torch
            assert np.array_equal(lists[f"{mine}_idx"][r, : cnt[r]], arrs[f"{prefix}/{idx_name}"][r, : cnt[r]])


@pytest.mark.parametrize("mask", ["doc_causal", "cross_doc_link"])
def test_attention_forward_matches_flex_eager(mask):
    fx, arrs = G.flex_arrays(), G.blockmap_arrays()
    entry = [e for e in BLOCKS if e["name"] == "t300"][0]
    spans, links, t = G.spans_of(entry), G.links_of(entry), entry["seq_len"]
    ids = om.document_ids(t, spans)
    if mask == "doc_causal":
        dense = om.doc_causal_dense(ids)
    else:
        dense = G.unpack(arrs["t300/cross_doc_link/dense"], (t, t))
    q, k, v = (torch.from_numpy(fx[f"t300/{n}"]) for n in "qkv")
    out, lse = oattn.forward(q, k, v, torch.from_numpy(dense))
    assert torch.allclose(out, torch.from_numpy(fx[f"t300/{mask}/out"]), atol=2e-5, rtol=1e-5)
    assert torch.allclose(lse, torch.from_numpy(fx[f"t300/{mask}/lse"]), atol=2e-5, rtol=1e-5)


def test_attention_backward_matches_autograd_and_dead_rows():
    g = torch.Generator().manual_seed(5)
    q, k, v, do = (torch.randn(1, 2, 70, 32, generator=g) for _ in range(4))
    dense = torch.tril(torch.ones(70, 70, dtype=torch.bool))
    dense[:, :40] &= torch.rand(70, 40, generator=g) > 0.5
    dense |= torch.eye(70, dtype=torch.bool)
    qa, ka, va = (x.clone().requires_grad_(True) for x in (q, k, v))
    ref = torch.nn.functional.scaled_dot_product_attention(qa, ka, va, attn_mask=dense)
    ref.backward(do)
    out, lse, dq, dk, dv = oattn.forward_backward(q, k, v, dense, do)
    for a, b in [(out, ref), (dq, qa.grad), (dk, ka.grad), (dv, va.grad)]:
        assert torch.allclose(a, b.detach(), atol=1e-4, rtol=1e-4)
    dense[7] = False  # fully masked row: O = 0, LSE = -inf, zero gradient, no NaN elsewhere
    out, lse, dq, dk, dv = oattn.forward_backward(q, k, v, dense, do)
    assert torch.all(out[:, :, 7] == 0) and torch.all(torch.isinf(lse[:, :, 7])) and torch.all(dq[:, :, 7] == 0)
    assert all(torch.isfinite(x).all() for x in (out, dq, dk, dv))


def test_class_mask_reproduces_doc_level_links():
    rng = np.random.default_rng(0)
    lens = [5, 9, 3, 12, 7]
    ids = np.repeat(np.arange(5), lens).astype(np.int32)
    link = np.zeros((5, 1), dtype=np.int64)
    for a in range(5):
        for b in range(a):
            if rng.random() < 0.5:
                link[a, 0] |= 1 << b
    dense = om.class_mask_dense(ids, None, None, link)
    t = ids.size
    for qi in range(t):
        for ki in range(t):
            exp = qi >= ki and (ids[qi] == ids[ki] or bool((link[ids[qi], 0] >> ids[ki]) & 1))
            assert dense[qi, ki] == exp


def test_streamed_oracle_equals_dense_oracle():
    g = torch.Generator().manual_seed(9)
    t, d = 300, 32
    q, k, v, do = (torch.randn(t, d, generator=g) for _ in range(4))
    dense = torch.tril(torch.ones(t, t, dtype=torch.bool)) & (torch.rand(t, t, generator=g) > 0.3)
    dense |= torch.eye(t, dtype=torch.bool)
    ref = oattn.forward_backward(q[None, None], k[None, None], v[None, None], dense, do[None, None])
    got = oattn.forward_backward_streamed(q, k, v, do, lambda a, b: dense[a:b], slab=64)
    for a, b in zip(got, ref):
        assert torch.allclose(a, b[0, 0], atol=1e-5, rtol=1e-5)
