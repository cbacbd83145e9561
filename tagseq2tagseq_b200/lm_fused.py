"""Autograd wrappers over the decoder-layer kernels of include/ts2ts_lm.h, plus the attention call on the packed QKV
projection.  They stand where the reference's layer uses fused modules (model/modules/layer.py:20-35,
model/modules/training_module.py:205); every op is one pass over HBM, fp32 arithmetic, bf16 activations.
CUDA only: there is no CPU path.
"""
from __future__ import annotations

import contextlib
import math
from typing import Optional, Tuple

import torch

from . import _lib
from .mask_spec import MaskSpec

__all__ = ["add_rmsnorm", "qkv_attention", "swiglu", "cross_entropy", "rope_half_tables"]


_NO_GUARD = contextlib.nullcontext()


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _on_device(t: torch.Tensor):
    """Device guard for the launches; free when the tensor already lives on the current device (the usual case: the
    training step issues a few hundred of these calls per step from Python)."""
    return _NO_GUARD if t.device.index == torch.cuda.current_device() else torch.cuda.device(t.device)


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("the decoder-layer kernels run on CUDA tensors only (no CPU path exists)")


class _AddRMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_in: torch.Tensor, a: Optional[torch.Tensor], w: torch.Tensor, eps: float):
        _need_cuda(x_in, a, w)
        if x_in.dtype != torch.float32 or w.dtype != torch.float32 or (a is not None and a.dtype != torch.bfloat16):
            raise TypeError("add_rmsnorm: x and w are fp32, a is bf16")
        x_in = x_in.contiguous()
        a = None if a is None else a.contiguous()
        C = x_in.shape[-1]
        N = x_in.numel() // C
        x_out = torch.empty_like(x_in)
        h = torch.empty(x_in.shape, dtype=torch.bfloat16, device=x_in.device)
        rstd = torch.empty(N, dtype=torch.float32, device=x_in.device)
        with _on_device(x_in):
            code = _lib.lib().ts2ts_add_rmsnorm_fwd(x_in.data_ptr(), None if a is None else a.data_ptr(), w.data_ptr(), x_out.data_ptr(),
                                                    h.data_ptr(), rstd.data_ptr(), N, C, eps, _stream(x_in))
        _lib.check(code, "ts2ts_add_rmsnorm_fwd")
        ctx.save_for_backward(x_out, w, rstd)
        ctx.has_a = a is not None
        return x_out, h

    @staticmethod
    def backward(ctx, dx_up: Optional[torch.Tensor], dh: Optional[torch.Tensor]):
        x, w, rstd = ctx.saved_tensors
        C = x.shape[-1]
        N = x.numel() // C
        if dh is None:  # h had no user: only the residual path carries a gradient
            dh = torch.zeros(x.shape, dtype=torch.bfloat16, device=x.device)
        dh = dh.contiguous()
        dx_up = None if dx_up is None else dx_up.contiguous()
        dx = torch.empty_like(x)
        da = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device) if ctx.has_a else None
        dw = torch.zeros_like(w)
        L = _lib.lib()
        ws = torch.empty(L.ts2ts_add_rmsnorm_bwd_workspace_bytes(N, C), dtype=torch.uint8, device=x.device)
        with _on_device(x):
            code = L.ts2ts_add_rmsnorm_bwd(dh.data_ptr(), None if dx_up is None else dx_up.data_ptr(), x.data_ptr(), w.data_ptr(),
                                           rstd.data_ptr(), dx.data_ptr(), None if da is None else da.data_ptr(), dw.data_ptr(),
                                           ws.data_ptr(), ws.numel(), N, C, _stream(x))
        _lib.check(code, "ts2ts_add_rmsnorm_bwd")
        return dx, da, dw, None


def add_rmsnorm(x: torch.Tensor, a: Optional[torch.Tensor], weight: torch.Tensor, eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """(x + a, rmsnorm(x + a) * weight): the fp32 residual stream and the bf16 input of the next linear layer."""
    return _AddRMSNorm.apply(x, a, weight, eps)


def rope_half_tables(T: int, head_dim: int, base: float, device) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos and sin of the rotation angles, fp32 [T, head_dim / 2] (pair i rotates with frequency base^(-2i/head_dim))."""
    inv = 1.0 / (base ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    ang = torch.arange(T, device=device, dtype=torch.float32)[:, None] * inv[None, :]
    return ang.cos().contiguous(), ang.sin().contiguous()


def _strides_bhtd(t: torch.Tensor):
    return _lib.strides3(t)


class _QKVAttention(torch.autograd.Function):
    """qkv [B,T,3*H*D] (the fused projection's output) -> attention output [B,T,H*D].  q and k are rotated in place;
    the attention kernels read q, k, v and write the output, and later dq, dk, dv, through strides of the packed
    buffers, so no tensor is transposed, split or concatenated in memory."""

    @staticmethod
    def forward(ctx, qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, mask: MaskSpec, n_heads: int, head_dim: int):
        _need_cuda(qkv, cos, sin)
        if qkv.dtype != torch.bfloat16 or not qkv.is_contiguous():
            raise TypeError("qkv_attention: qkv must be a contiguous bf16 tensor")
        B, T, _ = qkv.shape
        H, D = n_heads, head_dim
        if qkv.shape[-1] != 3 * H * D:
            raise ValueError("qkv_attention: last dimension must be 3 * n_heads * head_dim")
        L = _lib.lib()
        st = _stream(qkv)
        with _on_device(qkv):
            _lib.check(L.ts2ts_rope_qk_inplace(qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), B, T, H, D, 1.0, st), "ts2ts_rope_qk_inplace")
        ctx.mark_dirty(qkv)
        packed = qkv.view(B, T, 3, H, D)
        q, k, v = (packed[:, :, i].permute(0, 2, 1, 3) for i in range(3))          # [B,H,T,D] views
        out = torch.empty((B, T, H, D), dtype=torch.bfloat16, device=qkv.device)
        out_v = out.permute(0, 2, 1, 3)
        lse = torch.empty((B, H, T), dtype=torch.float32, device=qkv.device)
        doc, link, rows, cols, plan = mask.doc_ids, mask.link_bits, mask.q_row_ids, mask.kv_col_ids, mask.plan
        R, W = (0, 0) if link is None else (link.shape[1], link.shape[2])
        scale = 1.0 / math.sqrt(D)
        with _on_device(qkv):
            code = L.ts2ts_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), _strides_bhtd(q), _strides_bhtd(k), _strides_bhtd(v), B, H, T, D,
                                    scale, doc.data_ptr(), None if rows is None else rows.data_ptr(), None if cols is None else cols.data_ptr(),
                                    None if link is None else link.data_ptr(), R, W, plan.data_ptr(), plan.numel(), out_v.data_ptr(),
                                    _strides_bhtd(out_v), lse.data_ptr(), st)
        _lib.check(code, "ts2ts_attn_fwd")
        ctx.save_for_backward(qkv, out, lse, cos, sin)
        ctx.mask, ctx.dims, ctx.scale = mask, (B, T, H, D), scale
        return out.view(B, T, H * D), qkv

    @staticmethod
    def backward(ctx, dout: torch.Tensor, _dqkv_unused):
        qkv, out, lse, cos, sin = ctx.saved_tensors
        B, T, H, D = ctx.dims
        mask = ctx.mask
        L = _lib.lib()
        st = _stream(qkv)
        packed = qkv.view(B, T, 3, H, D)
        q, k, v = (packed[:, :, i].permute(0, 2, 1, 3) for i in range(3))
        out_v = out.permute(0, 2, 1, 3)
        dout_v = dout.contiguous().view(B, T, H, D).permute(0, 2, 1, 3)
        dqkv = torch.empty_like(qkv)
        dpacked = dqkv.view(B, T, 3, H, D)
        dq, dk, dv = (dpacked[:, :, i].permute(0, 2, 1, 3) for i in range(3))
        ws = torch.empty(L.ts2ts_attn_bwd_workspace_bytes(B, H, T, D), dtype=torch.uint8, device=qkv.device)
        doc, link, rows, cols, plan = mask.doc_ids, mask.link_bits, mask.q_row_ids, mask.kv_col_ids, mask.plan
        R, W = (0, 0) if link is None else (link.shape[1], link.shape[2])
        with _on_device(qkv):
            code = L.ts2ts_attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out_v.data_ptr(), dout_v.data_ptr(), lse.data_ptr(),
                                    _strides_bhtd(q), _strides_bhtd(k), _strides_bhtd(v), _strides_bhtd(out_v), _strides_bhtd(dout_v), B, H, T, D,
                                    ctx.scale, doc.data_ptr(), None if rows is None else rows.data_ptr(),
                                    None if cols is None else cols.data_ptr(), None if link is None else link.data_ptr(), R, W,
                                    plan.data_ptr(), plan.numel(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), _strides_bhtd(dq),
                                    _strides_bhtd(dk), _strides_bhtd(dv), ws.data_ptr(), ws.numel(), st)
            _lib.check(code, "ts2ts_attn_bwd")
            # gradient of the rotated q, k -> gradient of the projection's output: the inverse rotation, in place
            _lib.check(L.ts2ts_rope_qk_inplace(dqkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), B, T, H, D, -1.0, st), "ts2ts_rope_qk_inplace")
        return dqkv, None, None, None, None, None


def qkv_attention(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, mask: MaskSpec, n_heads: int, head_dim: int) -> torch.Tensor:
    """Rotary embedding + masked attention on the packed projection qkv [B,T,3*H*D] (bf16, overwritten: q and k are
    rotated in place).  cos / sin: fp32 [T, head_dim/2] from ``rope_half_tables``.  Returns [B,T,H*D]."""
    out, _ = _QKVAttention.apply(qkv, cos, sin, mask, n_heads, head_dim)
    return out


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu: torch.Tensor):
        _need_cuda(gu)
        if gu.dtype != torch.bfloat16:
            raise TypeError("swiglu: bf16 input")
        gu = gu.contiguous()
        F = gu.shape[-1] // 2
        N = gu.numel() // (2 * F)
        act = torch.empty(gu.shape[:-1] + (F,), dtype=torch.bfloat16, device=gu.device)
        with _on_device(gu):
            _lib.check(_lib.lib().ts2ts_swiglu_fwd(gu.data_ptr(), act.data_ptr(), N, F, _stream(gu)), "ts2ts_swiglu_fwd")
        ctx.save_for_backward(gu)
        return act

    @staticmethod
    def backward(ctx, dact: torch.Tensor):
        (gu,) = ctx.saved_tensors
        F = gu.shape[-1] // 2
        N = gu.numel() // (2 * F)
        dact = dact.contiguous()
        dgu = torch.empty_like(gu)
        with _on_device(gu):
            _lib.check(_lib.lib().ts2ts_swiglu_bwd(gu.data_ptr(), dact.data_ptr(), dgu.data_ptr(), N, F, _stream(gu)), "ts2ts_swiglu_bwd")
        return dgu


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up with gate, up = gate_up.chunk(2, dim=-1)."""
    return _SwiGLU.apply(gate_up)


class _CrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits: torch.Tensor, target: torch.Tensor):
        _need_cuda(logits, target)
        if logits.dtype != torch.bfloat16 or logits.dim() != 2 or not logits.is_contiguous():
            raise TypeError("cross_entropy: logits must be a contiguous bf16 [N,V] tensor")
        target = target.contiguous().to(torch.int64)
        N, V = logits.shape
        lse = torch.empty(N, dtype=torch.float32, device=logits.device)
        loss = torch.empty(N, dtype=torch.float32, device=logits.device)
        with _on_device(logits):
            _lib.check(_lib.lib().ts2ts_ce_fwd(logits.data_ptr(), target.data_ptr(), lse.data_ptr(), loss.data_ptr(), N, V, _stream(logits)),
                       "ts2ts_ce_fwd")
        ctx.save_for_backward(logits, target, lse)
        return loss.sum() / N

    @staticmethod
    def backward(ctx, g: torch.Tensor):
        logits, target, lse = ctx.saved_tensors
        N, V = logits.shape
        g = g.reshape(1).to(torch.float32).contiguous()
        # the logits are not needed again: their buffer becomes the gradient
        with _on_device(logits):
            _lib.check(_lib.lib().ts2ts_ce_bwd(logits.data_ptr(), target.data_ptr(), lse.data_ptr(), g.data_ptr(), 1.0 / N, N, V, _stream(logits)),
                       "ts2ts_ce_bwd")
        return logits, None


def cross_entropy(logits: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
    """Mean cross-entropy of bf16 logits [N,V] against int64 targets [N]; the backward overwrites ``logits`` with
    their gradient, so the caller must not use them afterwards."""
    return _CrossEntropy.apply(logits, target)
