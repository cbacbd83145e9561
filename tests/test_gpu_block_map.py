"""Block-map pre-pass (CUDA, through the C ABI) against the oracle and the reference's own BlockMasks: bit-exact."""
import numpy as np
import pytest
import torch

from oracle import block_map as obm
from oracle import masks as om
from tests import _golden as G

pytestmark = pytest.mark.gpu

BLOCKS = G.blockmap_cases()


def _check_lists(bm, st, b=0):
    lists = obm.lists_from_states(st)
    for name in ("kv", "full", "q", "full_q"):
        cnt = getattr(bm, f"{name}_cnt")[b].cpu().numpy()
        idx = getattr(bm, f"{name}_idx")[b].cpu().numpy()
        assert np.array_equal(cnt, lists[f"{name}_cnt"]), name
        assert np.array_equal(idx, lists[f"{name}_idx"]), name


@pytest.mark.parametrize("entry", BLOCKS, ids=[e["name"] for e in BLOCKS])
@pytest.mark.parametrize("mask", ["doc_causal", "cross_doc_link"])
def test_reference_fixtures(entry, mask):
    """Spans / links -> from_reference -> ts2ts_block_map == BlockMask that the reference's creators returned."""
    from tagseq2tagseq_b200 import from_reference
    arrs = G.blockmap_arrays()
    spans, links, t = G.spans_of(entry), G.links_of(entry), entry["seq_len"]
    spec = from_reference(spans, links if mask == "cross_doc_link" else None, t, max_grants_cap=entry["max_grants"])
    bm = spec.block_map(with_lists=True)
    st = bm.state[0].cpu().numpy()
    prefix = f"{entry['name']}/{mask}"
    assert np.array_equal(st, G.blockmask_to_states(arrs, prefix, st.shape[0]))
    for mine, cnt_name, idx_name in [("kv", "kv_num_blocks", "kv_indices"), ("full", "full_kv_num_blocks", "full_kv_indices"),
                                     ("q", "q_num_blocks", "q_indices"), ("full_q", "full_q_num_blocks", "full_q_indices")]:
        cnt = getattr(bm, f"{mine}_cnt")[0].cpu().numpy()
        idx = getattr(bm, f"{mine}_idx")[0].cpu().numpy()
        assert np.array_equal(cnt, arrs[f"{prefix}/{cnt_name}"])
        for r in range(st.shape[0]):
            assert np.array_equal(idx[r, : cnt[r]], arrs[f"{prefix}/{idx_name}"][r, : cnt[r]])
            assert np.all(idx[r, cnt[r]:] == -1)
    _check_lists(bm, st)


@pytest.mark.parametrize("t,median,lo,hi,p", [(1, 5, 1, 5, 0.0), (127, 30, 2, 60, 0.4), (128, 30, 2, 60, 0.4), (129, 300, 100, 300, 0.0),
                                              (300, 20, 1, 50, 0.5), (2048, 128, 16, 512, 0.0), (4000, 200, 32, 2048, 0.15),
                                              (3000, 3, 1, 6, 0.3)])
def test_synthetic_packs_against_oracle(t, median, lo, hi, p):
    from tagseq2tagseq_b200 import build_block_map, synth
    packs = [synth.make_pack(100 + t + b, t, median, lo, hi, p_link=p) for b in range(2)]
    doc_np, link_np = synth.stack_packs(packs)
    dev = torch.device("cuda")
    bm = build_block_map(torch.from_numpy(doc_np).to(dev), None if link_np is None else torch.from_numpy(link_np).to(dev), with_lists=True)
    for b in range(2):
        dense = om.class_mask_dense(doc_np[b], None, None, None if link_np is None else link_np[b])
        st = obm.block_states(dense)
        assert np.array_equal(bm.state[b].cpu().numpy(), st)
        _check_lists(bm, st, b)


def test_explicit_row_and_column_classes_and_odd_ids():
    """Row / column classes that differ from the doc ids, negative classes, repeated and negative doc ids."""
    from tagseq2tagseq_b200 import build_block_map
    rng = np.random.default_rng(0)
    t = 700
    doc = np.repeat(np.array([7, -1, 7, 3, -5, 9], dtype=np.int32), [100, 50, 150, 200, 120, 80])
    row = np.repeat(np.array([0, -1, 1, 2, 3, 1], dtype=np.int32), [100, 50, 150, 200, 120, 80])
    row[330:400] = 4  # a second row class inside one document
    col = np.repeat(np.array([2, 0, -1, 1, 70, 3], dtype=np.int32), [100, 50, 150, 200, 120, 80])
    link = rng.integers(-2**62, 2**62, size=(5, 2), dtype=np.int64)
    dev = torch.device("cuda")
    bm = build_block_map(torch.from_numpy(doc)[None].to(dev), torch.from_numpy(link)[None].to(dev),
                         torch.from_numpy(row)[None].to(dev), torch.from_numpy(col)[None].to(dev), with_lists=True)
    st = obm.block_states(om.class_mask_dense(doc, row, col, link))
    assert np.array_equal(bm.state[0].cpu().numpy(), st)
    _check_lists(bm, st)


def test_full_size_32k_properties_and_streamed_oracle():
    """The benchmark's 32k packs: state map equals the slab-streamed oracle; lists are mutual transposes."""
    from tagseq2tagseq_b200 import build_block_map, synth
    pack = synth.config3_pack(1003, "link_p30")
    dev = torch.device("cuda")
    bm = build_block_map(torch.from_numpy(pack.doc_ids)[None].to(dev), torch.from_numpy(pack.link_bits)[None].to(dev), with_lists=True)
    st = bm.state[0].cpu().numpy()
    assert np.array_equal(st, obm.block_states_streamed(pack.doc_ids, None, None, pack.link_bits))
    assert not np.triu(st, 1).any() and np.all(np.diag(st) == 1)
    kv_cnt, q_cnt = bm.kv_cnt[0].cpu().numpy(), bm.q_cnt[0].cpu().numpy()
    assert kv_cnt.sum() == q_cnt.sum() == (st == 1).sum()
    assert bm.full_cnt[0].sum().item() == bm.full_q_cnt[0].sum().item() == (st == 2).sum()


def test_rejects_bad_arguments():
    from tagseq2tagseq_b200 import build_block_map
    dev = torch.device("cuda")
    with pytest.raises(ValueError):
        build_block_map(torch.zeros((1, 8), dtype=torch.int64, device=dev))
    with pytest.raises(RuntimeError, match="CUDA"):
        build_block_map(torch.zeros((1, 8), dtype=torch.int32))
    with pytest.raises(ValueError):
        build_block_map(torch.zeros((1, 8), dtype=torch.int32, device=dev), torch.zeros((2, 1, 1), dtype=torch.int64, device=dev))


@pytest.mark.parametrize("seed", range(8))
def test_fuzz_random_classes_and_ragged_lengths(seed):
    """Random doc runs with random row / column classes (including -1 and out-of-range values) and random link
    bits, at lengths around tile boundaries."""
    from tagseq2tagseq_b200 import build_block_map
    rng = np.random.default_rng(900 + seed)
    t = int(rng.choice([65, 128, 255, 257, 511, 640, 1000, 1283]))
    def runs(values, mean_len):
        out = []
        while len(out) < t:
            out += [int(rng.choice(values))] * int(rng.integers(1, mean_len))
        return np.asarray(out[:t], dtype=np.int32)
    doc = runs(list(range(-2, 9)), 90)
    row = runs([-1, 0, 1, 2, 3, 4, 5, 6, 9], 70)      # 9 is out of range for R = 7
    col = runs([-1, 0, 1, 2, 63, 64, 65, 127, 200], 50)  # 200 is out of range for W = 2
    link = rng.integers(-2**63, 2**63 - 1, size=(7, 2), dtype=np.int64)
    link[rng.random((7, 2)) < 0.4] = 0
    dev = torch.device("cuda")
    bm = build_block_map(torch.from_numpy(doc)[None].to(dev), torch.from_numpy(link)[None].to(dev),
                         torch.from_numpy(row)[None].to(dev), torch.from_numpy(col)[None].to(dev), with_lists=True)
    st = obm.block_states(om.class_mask_dense(doc, row, col, link))
    assert np.array_equal(bm.state[0].cpu().numpy(), st)
    _check_lists(bm, st)


def test_tile_cost_counts_the_non_skipped_tiles_and_orders_packs_like_the_exact_pair_count():
    """The cost the density-aware schedule uses: non-skipped 128 x 128 tiles from the pre-pass (one read-back per pack),
    equal to the oracle's count, and ranking heavy-tailed packs like the exact number of unmasked pairs does."""
    from oracle import block_map as obm
    from tagseq2tagseq_b200 import synth
    from tagseq2tagseq_b200.replicas import schedule_packs, step_time_model, tile_cost
    dev = torch.device("cuda")
    packs = [synth.make_pack(600 + i, 4096, 150, 16, 2048, p_link=0.15, heavy_frac=0.05, heavy_lo=1024, heavy_hi=2048) for i in range(8)]
    costs = []
    for pk in packs:
        doc = torch.from_numpy(pk.doc_ids)[None].to(dev)
        link = torch.from_numpy(pk.link_bits)[None].to(dev)
        c = tile_cost(doc, link)
        dense = om.class_mask_dense(pk.doc_ids, None, None, pk.link_bits)
        assert c == int((obm.block_states(dense) != obm.SKIP).sum())
        costs.append(float(c))
    exact = [float(pk.unmasked_pairs()) for pk in packs]
    sched = schedule_packs(costs, 2)
    naive = [[0, 1], [2, 3], [4, 5], [6, 7]]
    assert step_time_model(exact, sched) <= step_time_model(exact, naive)  # tile counts balance the true cost too
