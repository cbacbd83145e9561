"""The memory-bound kernels of the decoder layer (include/ts2ts_lm.h) against plain PyTorch fp32 formulas of the same
ops, forward and backward, and the whole decoder against an unfused PyTorch model with the same parameters."""
import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


@pytest.mark.parametrize("n,c,with_a", [(37, 128, True), (300, 768, True), (65, 2048, False), (9, 8192, True)])
def test_add_rmsnorm_matches_torch(n, c, with_a):
    from tagseq2tagseq_b200.lm_fused import add_rmsnorm
    torch.manual_seed(n + c)
    eps = 1e-6
    x = torch.randn(n, c, device=DEV, requires_grad=True)
    a = (torch.randn(n, c, device=DEV) * 0.5).bfloat16().requires_grad_(True) if with_a else None
    w = (1 + 0.1 * torch.randn(c, device=DEV)).requires_grad_(True)
    r1, r2 = torch.randn(n, c, device=DEV), torch.randn(n, c, device=DEV)
    x_out, h = add_rmsnorm(x, a, w, eps)
    assert x_out.dtype == torch.float32 and h.dtype == torch.bfloat16
    ((x_out * r1).sum() + (h.float() * r2).sum()).backward()
    got = [x.grad.clone(), None if a is None else a.grad.clone(), w.grad.clone()]
    xr = x.detach().clone().requires_grad_(True)
    ar = None if a is None else a.detach().float().requires_grad_(True)
    wr = w.detach().clone().requires_grad_(True)
    xo = xr if ar is None else xr + ar
    hr = F.rms_norm(xo, (c,), wr, eps)
    ((xo * r1).sum() + (hr * r2).sum()).backward()
    assert torch.equal(x_out, xo.detach())
    assert _rel(h, hr) <= 4e-3                    # one bf16 rounding
    # the reference differentiates the unrounded h; the kernel receives the same upstream gradient r2 rounded to bf16
    assert _rel(got[0], xr.grad) <= 6e-3
    if a is not None:
        assert _rel(got[1], ar.grad) <= 8e-3
    assert _rel(got[2], wr.grad) <= 6e-3


def test_rope_in_place_and_its_inverse():
    from tagseq2tagseq_b200 import _lib
    from tagseq2tagseq_b200.lm_fused import rope_half_tables
    from tagseq2tagseq_b200.train_step import apply_rope, rope_tables
    torch.manual_seed(1)
    B, T, H, D = 2, 77, 3, 64
    qkv = torch.randn(B, T, 3, H, D, device=DEV).bfloat16()
    orig = qkv.clone()
    cos_h, sin_h = rope_half_tables(T, D, 10000.0, DEV)
    L = _lib.lib()
    st = torch.cuda.current_stream().cuda_stream
    assert L.ts2ts_rope_qk_inplace(qkv.data_ptr(), cos_h.data_ptr(), sin_h.data_ptr(), B, T, H, D, 1.0, st) == 0
    cos, sin = (c[None, :, None, None, :] for c in rope_tables(T, D, 10000.0, DEV))
    want = apply_rope(orig[:, :, :2].float(), cos, sin)
    assert _rel(qkv[:, :, :2], want) <= 4e-3
    assert torch.equal(qkv[:, :, 2], orig[:, :, 2])               # v untouched
    assert L.ts2ts_rope_qk_inplace(qkv.data_ptr(), cos_h.data_ptr(), sin_h.data_ptr(), B, T, H, D, -1.0, st) == 0
    assert _rel(qkv, orig) <= 8e-3                                # rotated back, two bf16 roundings


@pytest.mark.parametrize("n,f", [(50, 256), (129, 3072), (7, 5504)])
def test_swiglu_matches_torch(n, f):
    from tagseq2tagseq_b200.lm_fused import swiglu
    torch.manual_seed(f)
    gu = (torch.randn(n, 2 * f, device=DEV) * 2).bfloat16().requires_grad_(True)
    r = torch.randn(n, f, device=DEV).bfloat16()
    act = swiglu(gu)
    (act.float() * r.float()).sum().backward()
    gr = gu.detach().float().requires_grad_(True)
    g, u = gr.chunk(2, dim=-1)
    ref = F.silu(g) * u
    (ref * r.float()).sum().backward()
    assert _rel(act, ref) <= 4e-3
    assert _rel(gu.grad, gr.grad) <= 4e-3


@pytest.mark.parametrize("n,v", [(33, 512), (5, 50304), (200, 1000)])
def test_cross_entropy_matches_torch(n, v):
    from tagseq2tagseq_b200.lm_fused import cross_entropy
    torch.manual_seed(v)
    base = (torch.randn(n, v, device=DEV) * 3).bfloat16()
    base[:, :24] = float("-inf")                                  # a masked stretch of the vocabulary
    tgt = torch.randint(24, v, (n,), device=DEV)
    ref_in = base.float().requires_grad_(True)
    ref = F.cross_entropy(ref_in, tgt)
    (ref * 1.7).backward()
    logits = base.clone().requires_grad_(True)
    work = logits * 1.0                                           # a non-leaf buffer the op may overwrite
    loss = cross_entropy(work, tgt)
    (loss * 1.7).backward()
    assert abs(loss.item() - ref.item()) <= 1e-4 * max(1.0, abs(ref.item()))
    assert _rel(logits.grad, ref_in.grad) <= 5e-3


def _pack_and_spec(t, seed=21):
    from tagseq2tagseq_b200 import synth
    from tagseq2tagseq_b200.mask_spec import MaskSpec
    pack = synth.make_pack(seed, t, 60, 8, 300, p_link=0.3)
    return MaskSpec(doc_ids=torch.from_numpy(pack.doc_ids)[None].to(DEV), link_bits=torch.from_numpy(pack.link_bits)[None].to(DEV))


def test_qkv_attention_equals_rope_plus_operator():
    from tagseq2tagseq_b200.attention import masked_attn
    from tagseq2tagseq_b200.lm_fused import qkv_attention, rope_half_tables
    from tagseq2tagseq_b200.train_step import apply_rope, rope_tables
    torch.manual_seed(3)
    B, T, H, D = 1, 700, 2, 64
    spec = _pack_and_spec(T)
    base = torch.randn(B, T, 3 * H * D, device=DEV).bfloat16()
    do = torch.randn(B, T, H * D, device=DEV).bfloat16()
    leaf = base.clone().requires_grad_(True)
    out = qkv_attention(leaf * 1.0, *rope_half_tables(T, D, 10000.0, DEV), spec, H, D)
    out.backward(do)
    # the same through separate steps: rotation in fp32 by the PyTorch formula, operator on [B,H,T,D] tensors
    ref_leaf = base.clone().requires_grad_(True)
    packed = ref_leaf.view(B, T, 3, H, D)
    cos, sin = (c[None, :, None, None, :] for c in rope_tables(T, D, 10000.0, DEV))
    qk = apply_rope(packed[:, :, :2].float(), cos, sin).bfloat16()
    q, k, v = qk[:, :, 0].permute(0, 2, 1, 3), qk[:, :, 1].permute(0, 2, 1, 3), packed[:, :, 2].permute(0, 2, 1, 3)
    ref, _ = masked_attn(q, k, v, spec.doc_ids, spec.link_bits, plan=spec.plan)
    ref = ref.permute(0, 2, 1, 3).reshape(B, T, H * D)
    ref.backward(do)
    assert _rel(out, ref) <= 1e-2
    assert _rel(leaf.grad, ref_leaf.grad) <= 2e-2


def test_decoder_matches_an_unfused_pytorch_model():
    from tagseq2tagseq_b200.attention import masked_attn
    from tagseq2tagseq_b200.train_step import DecoderLM, LMConfig, RMS_EPS, apply_rope, rope_tables
    torch.manual_seed(11)
    cfg = LMConfig(n_layers=2, d_model=128, n_heads=2, head_dim=64, mlp_hidden=256, vocab=512)
    T = 640
    spec = _pack_and_spec(T, seed=5)
    model = DecoderLM(cfg).to(DEV)
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() == 1:
                p.add_(0.1 * torch.randn_like(p))                 # norm weights away from 1 so their gradients matter
    tok = torch.randint(0, cfg.vocab, (1, T + 1), device=DEV)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        loss = model(tok, spec)
    loss.backward()
    got = {n: p.grad.detach().clone() for n, p in model.named_parameters()}
    model.zero_grad(set_to_none=True)

    def reference(tokens):
        inp, tgt = tokens[:, :-1], tokens[:, 1:]
        x = model.embed(inp)
        cos, sin = (c[None, :, None, None, :] for c in rope_tables(T, cfg.head_dim, cfg.rope_base, DEV))
        for blk in model.blocks:
            h = F.rms_norm(x, (cfg.d_model,), blk.ln1.weight, RMS_EPS)
            qkv = blk.qkv(h.bfloat16()).view(1, T, 3, cfg.n_heads, cfg.head_dim)
            qk = apply_rope(qkv[:, :, :2].float(), cos, sin).bfloat16()
            q, k, v = qk[:, :, 0].permute(0, 2, 1, 3), qk[:, :, 1].permute(0, 2, 1, 3), qkv[:, :, 2].permute(0, 2, 1, 3)
            o, _ = masked_attn(q, k, v, spec.doc_ids, spec.link_bits, plan=spec.plan)
            x = x + blk.proj(o.transpose(1, 2).reshape(1, T, -1)).float()
            h = F.rms_norm(x, (cfg.d_model,), blk.ln2.weight, RMS_EPS)
            g, u = blk.gate_up(h.bfloat16()).float().chunk(2, dim=-1)
            x = x + blk.down((F.silu(g) * u).bfloat16()).float()
        h = F.rms_norm(x, (cfg.d_model,), model.norm.weight, RMS_EPS)
        logits = model.head(h.bfloat16())
        return F.cross_entropy(logits.float().view(-1, cfg.vocab), tgt.reshape(-1))

    with torch.autocast("cuda", dtype=torch.bfloat16):
        ref = reference(tok)
    ref.backward()
    assert abs(loss.item() - ref.item()) <= 2e-3 * abs(ref.item())
    assert math.isfinite(loss.item())
    for n, p in model.named_parameters():
        assert _rel(got[n], p.grad) <= 3e-2, n
