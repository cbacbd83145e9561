"""Boundary behaviour on the GPU: a bounded wait that runs out, a plan that belongs to another call, the operator under
torch.compile and torch.library.opcheck, the `causal` creator, and a batch served by a one-sequence mask."""
import ctypes
import os

import numpy as np
import pytest
import torch

from oracle import attention as oattn
from oracle import masks as om

pytestmark = pytest.mark.gpu

O_TOL, LSE_TOL, GRAD_TOL = 2e-2, 1e-2, 1e-2


def test_bounded_wait_runs_out_and_reports_its_code():
    """The one way a device wait may fail here: nothing ever arrives on the barrier, the poll limit (4096 in the
    self-test library) is reached, the code lands in the status word and the kernel returns.  ts2ts_read_status hands
    the code back as its return value."""
    from tagseq2tagseq_b200 import _lib, build
    L = _lib.lib()
    st = ctypes.CDLL(build.SELFTEST_LIB)
    st.ts2ts_selftest_bounded_wait.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p]
    st.ts2ts_selftest_spin_limit.restype = ctypes.c_uint
    assert st.ts2ts_selftest_spin_limit() <= 1 << 16
    dev = torch.device("cuda")
    plan = torch.zeros(L.ts2ts_plan_bytes(1, 128), dtype=torch.uint8, device=dev)  # status word 0 = 0
    cycles = torch.zeros(1, dtype=torch.int64, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    assert st.ts2ts_selftest_bounded_wait(plan.data_ptr(), 77, cycles.data_ptr(), stream) == 0
    out = ctypes.c_int32(0)
    rc = L.ts2ts_read_status(plan.data_ptr(), stream, ctypes.byref(out))
    assert rc == 1077 and out.value == 1077            # > 0: the recorded code, as include/ts2ts_attn.h promises
    assert b"1077" in L.ts2ts_last_error_string()
    assert 0 < int(cycles.item()) < 50_000_000         # gave up after thousands of polls, not after seconds
    torch.cuda.synchronize()                           # the context is still usable
    assert float(torch.ones(4, device=dev).sum()) == 4.0


def test_plan_of_another_call_is_refused_with_a_status_code():
    """A plan built for (B=1, T=512) handed to calls with T=384: the buffer is large enough, so the host check passes,
    but the stamp the pre-pass left does not match and both kernels return without touching a list."""
    from tagseq2tagseq_b200 import build_block_map, read_status
    from tagseq2tagseq_b200.attention import _attn_bwd, _attn_fwd
    dev = torch.device("cuda")
    plan = build_block_map(torch.zeros((1, 512), dtype=torch.int32, device=dev)).plan
    doc = torch.zeros((1, 384), dtype=torch.int32, device=dev)
    q, k, v = (torch.randn(1, 2, 384, 128, device=dev).bfloat16() for _ in range(3))
    out, lse = _attn_fwd(q, k, v, doc, None, None, None, plan, 0.1)
    assert read_status(plan) == 1900
    good = build_block_map(doc).plan
    out, lse = _attn_fwd(q, k, v, doc, None, None, None, good, 0.1)
    assert read_status(good) == 0
    plan2 = build_block_map(torch.zeros((1, 512), dtype=torch.int32, device=dev)).plan
    _attn_bwd(q, k, v, out, torch.ones_like(q), lse, doc, None, None, None, plan2, 0.1)
    assert read_status(plan2) == 2901
    never_built = torch.zeros_like(good)
    _attn_fwd(q, k, v, doc, None, None, None, never_built, 0.1)
    assert read_status(never_built) == 1900


def _masked_case(t, seed, dev):
    from tagseq2tagseq_b200 import synth
    pack = synth.make_pack(seed, t, 50, 4, 200, p_link=0.25)
    doc = torch.from_numpy(pack.doc_ids)[None].to(dev)
    link = torch.from_numpy(pack.link_bits)[None].to(dev)
    dense = torch.from_numpy(om.class_mask_dense(pack.doc_ids, None, None, pack.link_bits))[None]
    g = torch.Generator().manual_seed(seed)
    q, k, v, do = (torch.randn(1, 2, t, 64, generator=g).bfloat16() for _ in range(4))
    return doc, link, dense, q, k, v, do


def test_operator_under_torch_compile_dynamic_and_opcheck():
    """The reference compiles its backbone with dynamic=True (main.py:387-397), so the operator must trace with fake
    tensors, stay one graph node and accept a sequence length it was not first compiled for."""
    from tagseq2tagseq_b200 import build_block_map
    from tagseq2tagseq_b200.attention import masked_attn
    dev = torch.device("cuda")

    def fn(q, k, v, doc, link, plan):
        out, lse = masked_attn(q * 1.0, k, v, doc, link, plan=plan)
        return out * 2.0, lse

    compiled = torch.compile(fn, dynamic=True, fullgraph=True, backend="aot_eager")
    for t, seed in ((256, 1), (384, 2)):
        doc, link, dense, q, k, v, do = _masked_case(t, seed, dev)
        plan = build_block_map(doc, link).plan
        qd, kd, vd = (x.to(dev).requires_grad_(True) for x in (q, k, v))
        out, lse = compiled(qd, kd, vd, doc, link, plan)
        out.backward(do.to(dev))
        ro, rl, rdq, rdk, rdv = oattn.forward_backward(q, k, v, dense, do * 2.0)
        assert (out.float().cpu() - 2.0 * ro).abs().max().item() <= 2 * O_TOL
        assert (lse.cpu() - rl).abs().max().item() <= LSE_TOL
        for a, b in ((qd.grad, rdq), (kd.grad, rdk), (vd.grad, rdv)):
            assert ((a.float().cpu() - b).norm() / b.norm()).item() <= GRAD_TOL
    doc, link, dense, q, k, v, do = _masked_case(256, 3, dev)
    plan = build_block_map(doc, link).plan
    args = (q.to(dev), k.to(dev), v.to(dev), doc, link, None, None, plan, 0.125)
    torch.library.opcheck(torch.ops.ts2ts.masked_attn_fwd.default, args,
                          test_utils=("test_schema", "test_faketensor", "test_autograd_registration"))


def test_causal_creator_matches_plain_causal_attention():
    """`causal` of the reference's registry (block_mask_creator.py:143-172): block map and attention against the oracle."""
    from oracle import block_map as obm
    from tagseq2tagseq_b200 import mask_spec as ms
    from tagseq2tagseq_b200.attention import flex_attention
    dev = torch.device("cuda")
    t = 700
    spec = ms.make_mask_creator_callable("causal")(tokens=torch.zeros((1, t), dtype=torch.int64, device=dev), doc_spans=[])
    dense = np.tril(np.ones((t, t), dtype=bool))
    assert np.array_equal(spec.block_map(with_lists=True).state[0].cpu().numpy(), obm.block_states(dense))
    g = torch.Generator().manual_seed(4)
    q, k, v, do = (torch.randn(1, 2, t, 128, generator=g).bfloat16() for _ in range(4))
    qd, kd, vd = (x.to(dev).requires_grad_(True) for x in (q, k, v))
    out, lse = flex_attention(qd, kd, vd, block_mask=spec, return_lse=True)
    out.backward(do.to(dev))
    ro, rl, rdq, rdk, rdv = oattn.forward_backward(q, k, v, torch.from_numpy(dense)[None], do)
    assert (out.float().cpu() - ro).abs().max().item() <= O_TOL and (lse.cpu() - rl).abs().max().item() <= LSE_TOL
    for a, b in ((qd.grad, rdq), (kd.grad, rdk), (vd.grad, rdv)):
        assert ((a.float().cpu() - b).norm() / b.norm()).item() <= GRAD_TOL


def test_one_sequence_mask_serves_a_batch_and_expanded_inputs():
    """The reference's BlockMask has B=None and broadcasts; here a one-sequence MaskSpec is expanded once per batch size
    (its plan is cached) and stride-0 q/k/v views are copied instead of being rejected."""
    from tagseq2tagseq_b200.attention import flex_attention
    from tagseq2tagseq_b200.mask_spec import MaskSpec
    dev = torch.device("cuda")
    doc, link, dense, q, k, v, do = _masked_case(300, 7, dev)
    spec = MaskSpec(doc_ids=doc, link_bits=link)
    qb = q.to(dev).expand(3, -1, -1, -1)  # stride 0 over the batch
    kb, vb = k.to(dev).expand(3, -1, -1, -1), v.to(dev).expand(3, -1, -1, -1)
    out = flex_attention(qb, kb, vb, block_mask=spec)
    plan_first = spec.expanded(3).plan
    out2 = flex_attention(qb, kb, vb, block_mask=spec)
    assert spec.expanded(3).plan.data_ptr() == plan_first.data_ptr()  # no second pre-pass
    ro = oattn.forward_backward(q, k, v, dense, do)[0]
    for b in range(3):
        assert (out[b].float().cpu() - ro[0]).abs().max().item() <= O_TOL
    assert torch.equal(out, out2)


def test_segment_ids_filled_on_the_device_and_reference_format_adapter():
    """ts2ts_segment_ids against a numpy expansion (empty table, gaps, a table that ends before T), and from_reference
    on the GPU -- classes from segments, ids filled by the kernel -- against the host construction on reference-style
    grants that start in the middle of their source documents."""
    from types import SimpleNamespace
    from tagseq2tagseq_b200 import mask_spec as ms
    dev = torch.device("cuda")
    t = 1000
    for bounds, ids in (([0], []), ([5, 17, 400, 401, 999], [3, -1, 0, 7]), ([0, 1000], [2]), ([10, 20, 30], [1, 1])):
        got = ms.segment_ids(np.asarray(bounds, dtype=np.int32), np.asarray(ids, dtype=np.int32), t, dev)[0].cpu().numpy()
        want = np.full(t, -1, dtype=np.int32)
        for j, v in enumerate(ids):
            want[bounds[j]:bounds[j + 1]] = v
        assert np.array_equal(got, want)
    rng = np.random.default_rng(3)
    lengths = rng.integers(20, 120, size=14)
    starts = np.concatenate([[0], np.cumsum(lengths)[:-1]])
    t = int(lengths.sum())
    spans = [SimpleNamespace(doc_id=i, start=int(starts[i]), end=int(starts[i] + lengths[i])) for i in range(len(lengths))]
    links = {}
    for a in range(1, len(lengths)):
        for b in range(a):
            if rng.random() < 0.3:
                links.setdefault(int(starts[a] + rng.integers(1, lengths[a])), []).append(b)
    spec = ms.from_reference(spans, links, t, max_grants_cap=64, device=dev)
    grants = ms.ordered_grants(t, spans, links, 64)
    row, col, link = ms.grant_classes(t, grants)
    want = om.class_mask_dense(ms.build_document_ids(t, spans), row, col, link)
    got = om.class_mask_dense(spec.doc_ids[0].cpu().numpy(), spec.q_row_ids[0].cpu().numpy(), spec.kv_col_ids[0].cpu().numpy(),
                              spec.link_bits[0].cpu().numpy())
    assert np.array_equal(got, want)


@pytest.mark.parametrize("d,t,p", [(128, 1000, 0.25), (64, 777, 0.0), (128, 129, 0.4)])
def test_decode_step_with_cached_keys_equals_the_row_of_the_full_forward(d, t, p):
    """One new token against cached K / V: must equal the corresponding row of the whole-sequence attention, which is
    what the reference recomputes for every generated token (model/generation_loop.py:90-92).  Checked against the
    fp32 oracle and against this package's own full forward, at the last position and at an inner one (q_pos)."""
    from tagseq2tagseq_b200 import build_block_map, synth
    from tagseq2tagseq_b200.attention import masked_attn, masked_attn_decode
    dev = torch.device("cuda")
    pack = synth.make_pack(31, t, 60, 4, 300, p_link=p)
    doc = torch.from_numpy(pack.doc_ids)[None].to(dev).expand(2, -1).contiguous()
    link = None if pack.link_bits is None else torch.from_numpy(pack.link_bits)[None].to(dev).expand(2, -1, -1).contiguous()
    dense = torch.from_numpy(om.class_mask_dense(pack.doc_ids, None, None, pack.link_bits))[None]
    g = torch.Generator().manual_seed(5)
    q, k, v, do = (torch.randn(2, 3, t, d, generator=g).bfloat16() for _ in range(4))
    full, full_lse = masked_attn(q.to(dev), k.to(dev), v.to(dev), doc, link, plan=build_block_map(doc, link).plan)
    for pos in (t - 1, t // 2):
        q_pos = None if pos == t - 1 else torch.full((2,), pos, dtype=torch.int32, device=dev)
        out, lse = masked_attn_decode(q[:, :, pos:pos + 1].to(dev), k.to(dev), v.to(dev), doc, link, q_pos=q_pos)
        assert out.shape == (2, 3, 1, d) and lse.shape == (2, 3)
        for b in range(2):
            ro, rl = oattn.forward_backward(q[b:b + 1], k[b:b + 1], v[b:b + 1], dense, do[b:b + 1])[:2]
            assert (out[b, :, 0].float().cpu() - ro[0, :, pos]).abs().max().item() <= O_TOL
            assert (lse[b].cpu() - rl[0, :, pos]).abs().max().item() <= LSE_TOL
        assert (out[:, :, 0].float() - full[:, :, pos].float()).abs().max().item() <= O_TOL
        assert (lse - full_lse[:, :, pos]).abs().max().item() <= LSE_TOL
    # a strided cache (heads interleaved as in a fused projection) is read in place
    kc = k.permute(0, 2, 1, 3).contiguous().to(dev).permute(0, 2, 1, 3)
    vc = v.permute(0, 2, 1, 3).contiguous().to(dev).permute(0, 2, 1, 3)
    out2, _ = masked_attn_decode(q[:, :, t - 1:t].to(dev), kc, vc, doc, link)
    out1, _ = masked_attn_decode(q[:, :, t - 1:t].to(dev), k.to(dev), v.to(dev), doc, link)
    assert torch.equal(out1, out2)
