"""Decoder-only LM training step around the masked-attention operator, with DDP over NCCL.

This is the scaling half of the benchmark: the call order of the reference's training module
(model/modules/training_module.py:195-211: shift tokens, build the mask once, embed -> backbone -> norm -> logits ->
cross-entropy) and its DDP settings (main.py:404-415: static graph, no unused parameters, 256 MB buckets), with a
plain pre-norm decoder (RMSNorm, fused QKV, RoPE, SwiGLU) standing in for the reference's tunalab modules, which are
not available.  Every layer calls the masked-attention kernels on the packed QKV projection (lm_fused.qkv_attention);
the block plan is built once per micro-batch and shared by all layers, as the reference shares its BlockMask
(block_mask_creator.py:132-139).  The GEMMs are cuBLAS through torch and the optimizer is torch's fused AdamW; the
memory-bound pieces between them (residual add + RMSNorm, rotary embedding, SwiGLU, cross-entropy) are single-pass
kernels of this library, as the reference's are fused modules.
"""
from __future__ import annotations

import math
from contextlib import nullcontext as _nullcontext
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .lm_fused import add_rmsnorm, cross_entropy, qkv_attention, rope_half_tables, swiglu
from .mask_spec import MaskSpec

RMS_EPS = float(torch.finfo(torch.float32).eps)  # what nn.RMSNorm uses for fp32 input when eps is None


@dataclass
class LMConfig:
    n_layers: int = 12
    d_model: int = 768
    n_heads: int = 12
    head_dim: int = 64
    mlp_hidden: int = 3072
    vocab: int = 50304
    rope_base: float = 10000.0

    @property
    def matmul_params(self) -> int:
        """Parameters that take part in a GEMM per token (all linear layers and the output head)."""
        d, hd = self.d_model, self.n_heads * self.head_dim
        per_layer = d * 3 * hd + hd * d + 3 * d * self.mlp_hidden
        return self.n_layers * per_layer + d * self.vocab


def config4() -> LMConfig:
    return LMConfig(12, 768, 12, 64, 3072, 50304)


def config5() -> LMConfig:
    # SwiGLU hidden int(8/3 * 2048) = 5461 (model/modules/layer.py:26) rounded up to a multiple of 128 for GEMM alignment
    return LMConfig(24, 2048, 16, 128, 5504, 50304)


def rope_tables(T: int, head_dim: int, base: float, device, dtype=torch.float32):
    """cos and sin of the rotation angles, both halves filled: [T, head_dim] each, computed in fp32."""
    inv = 1.0 / (base ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    ang = torch.arange(T, device=device, dtype=torch.float32)[:, None] * inv[None, :]
    return torch.cat([ang.cos(), ang.cos()], dim=-1).to(dtype), torch.cat([ang.sin(), ang.sin()], dim=-1).to(dtype)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [..., T, *, *, D] with cos / sin broadcastable to it; rotates pairs (first half, second half) in x's dtype:
    x * cos + rotate_half(x) * sin with rotate_half(x) = (-x2, x1)."""
    h = x.shape[-1] // 2
    rot = torch.cat([-x[..., h:], x[..., :h]], dim=-1)
    return x * cos + rot * sin


class Block(nn.Module):
    """Pre-norm decoder layer.  It receives the residual stream ``x`` (fp32) and the branch output ``a`` (bf16) that
    has not been added to it yet, so that the add fuses with the RMSNorm that follows; it returns the pair in the
    same form: x <- x + a; x <- x + attn(norm(x)) is returned as (x, mlp branch output)."""

    def __init__(self, cfg: LMConfig):
        super().__init__()
        hd = cfg.n_heads * cfg.head_dim
        self.cfg = cfg
        self.ln1 = nn.RMSNorm(cfg.d_model)
        self.qkv = nn.Linear(cfg.d_model, 3 * hd, bias=False)
        self.proj = nn.Linear(hd, cfg.d_model, bias=False)
        self.ln2 = nn.RMSNorm(cfg.d_model)
        self.gate_up = nn.Linear(cfg.d_model, 2 * cfg.mlp_hidden, bias=False)
        self.down = nn.Linear(cfg.mlp_hidden, cfg.d_model, bias=False)

    def forward(self, x, a, mask: MaskSpec, cos, sin):
        c = self.cfg
        x, h = add_rmsnorm(x, a, self.ln1.weight, RMS_EPS)
        attn = qkv_attention(self.qkv(h), cos, sin, mask, c.n_heads, c.head_dim)   # rotary + masked attention, layer.py:32-35
        x, h = add_rmsnorm(x, self.proj(attn), self.ln2.weight, RMS_EPS)
        return x, self.down(swiglu(self.gate_up(h)))


class DecoderLM(nn.Module):
    def __init__(self, cfg: LMConfig):
        super().__init__()
        self.cfg = cfg
        self.embed = nn.Embedding(cfg.vocab, cfg.d_model)
        self.blocks = nn.ModuleList(Block(cfg) for _ in range(cfg.n_layers))
        self.norm = nn.RMSNorm(cfg.d_model)
        self.head = nn.Linear(cfg.d_model, cfg.vocab, bias=False)
        for p in self.parameters():
            if p.dim() >= 2:
                nn.init.normal_(p, std=0.02)

    def forward(self, tokens: torch.Tensor, mask: MaskSpec) -> torch.Tensor:
        """tokens int64 [B, T+1]; returns the mean next-token cross-entropy (training_module.py:195-211).  Runs under
        bf16 autocast: the linear layers compute in bf16, the residual stream, norms, rotary angles and the loss in fp32."""
        inp, tgt = tokens[:, :-1], tokens[:, 1:]
        T = inp.shape[1]
        x = self.embed(inp).float()
        cos, sin = rope_half_tables(T, self.cfg.head_dim, self.cfg.rope_base, inp.device)
        a = None
        for blk in self.blocks:
            x, a = blk(x, a, mask, cos, sin)
        _, h = add_rmsnorm(x, a, self.norm.weight, RMS_EPS)
        logits = self.head(h)
        if logits.dtype != torch.bfloat16:
            logits = logits.to(torch.bfloat16)
        return cross_entropy(logits.view(-1, logits.shape[-1]), tgt.reshape(-1))


class TrainStep:
    """One optimizer step on one packed sequence per rank: forward under bf16 autocast, backward (DDP all-reduces
    the gradients, overlapped with the backward), fused AdamW on fp32 parameters.

    DDP settings follow main.py:404-415 (static graph, no unused parameters, 256 MB buckets; the first bucket keeps
    torch's small default so that the last gradients to be produced start their all-reduce early).  With
    ``bf16_grads`` the buckets are cast to bf16 for the all-reduce and back (torch's ``bf16_compress_hook``), which
    halves the bytes on NVLink; the parameters and the optimizer state stay fp32."""

    def __init__(self, cfg: LMConfig, device: torch.device, world: int = 1, lr: float = 3e-4, seed: int = 0,
                 bf16_grads: bool = True, bucket_cap_mb: int = 256):
        torch.manual_seed(seed)  # identical initial weights on every rank
        self.cfg, self.device, self.world = cfg, device, world
        model = DecoderLM(cfg).to(device)
        self.model = model
        self.bf16_grads = bool(bf16_grads and world > 1)
        if world > 1:
            self.model = torch.nn.parallel.DistributedDataParallel(
                model, device_ids=[device.index], static_graph=True, find_unused_parameters=False, bucket_cap_mb=bucket_cap_mb,
                gradient_as_bucket_view=True)
            if self.bf16_grads:
                from torch.distributed.algorithms.ddp_comm_hooks import default_hooks
                self.model.register_comm_hook(None, default_hooks.bf16_compress_hook)
        self.opt = torch.optim.AdamW(model.parameters(), lr=lr, betas=(0.9, 0.95), weight_decay=0.1, fused=True)

    @property
    def grad_bytes_per_step(self) -> int:
        """Bytes each rank contributes to the gradient all-reduce of one step."""
        n = sum(p.numel() for p in self.model.parameters())
        return n * (2 if self.bf16_grads else 4)

    def forward_backward(self, tokens: torch.Tensor, mask: MaskSpec, sync: bool = True) -> torch.Tensor:
        """Loss and gradients without the optimizer step.  ``sync=False`` skips the gradient all-reduce (DDP's
        ``no_sync``): the difference between the two is what the collective costs this rank."""
        self.opt.zero_grad(set_to_none=True)
        ctx = self.model.no_sync() if (not sync and self.world > 1) else _nullcontext()
        with ctx:
            with torch.autocast("cuda", dtype=torch.bfloat16):
                loss = self.model(tokens, mask)
            loss.backward()
        return loss.detach()

    def step(self, tokens: torch.Tensor, mask: MaskSpec) -> torch.Tensor:
        loss = self.forward_backward(tokens, mask)
        self.opt.step()
        return loss


def train_flops_per_step(cfg: LMConfig, T: int, unmasked_pairs: int) -> float:
    """6 * P_matmul * T for the linear layers (forward + backward) plus 14 * D * H * N per layer for attention."""
    return 6.0 * cfg.matmul_params * T + cfg.n_layers * 14.0 * cfg.head_dim * cfg.n_heads * unmasked_pairs
