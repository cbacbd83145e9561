"""Torch operator over the C ABI: ``ts2ts::masked_attn`` (forward + autograd) and a ``flex_attention``-shaped shim.

The reference calls ``flex_attention(q, k, v, block_mask=block_mask)`` from its attention module
(model/modules/layer.py:33; the symbol is swapped at run time in generate.py:167-178).  ``flex_attention``
below has that signature and accepts a ``MaskSpec`` where the reference passes a ``BlockMask``.
There is no CPU or PyTorch fallback: non-CUDA tensors raise.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from . import _lib
from .mask_spec import MaskSpec, build_block_map

__all__ = ["masked_attn", "masked_attn_decode", "flex_attention"]


def _opt_ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _check_qkv(q, k, v):
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise RuntimeError("ts2ts::masked_attn runs on CUDA tensors only (no CPU path exists)")
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
        raise TypeError("q, k, v must be bfloat16")
    if q.dim() != 4 or q.shape != k.shape or q.shape != v.shape:
        raise ValueError("q, k, v must share the shape [B,H,T,D]")
    if q.shape[-1] not in (64, 128):
        raise ValueError("head dimension must be 64 or 128")


def _rowmajor(t: torch.Tensor) -> torch.Tensor:
    """The kernels need a unit stride in D and 16-byte aligned rows; anything else is copied once."""
    if t.stride(-1) != 1 or any(s <= 0 or (s * 2) % 16 for s in t.stride()[:-1]) or t.data_ptr() % 16:
        return t.contiguous()  # also expanded (stride 0) views: the TMA descriptors need positive strides
    return t


@torch.library.custom_op("ts2ts::masked_attn_fwd", mutates_args=())
def _attn_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, doc_ids: torch.Tensor, link_bits: Optional[torch.Tensor],
              q_row_ids: Optional[torch.Tensor], kv_col_ids: Optional[torch.Tensor], plan: torch.Tensor,
              scale: float) -> Tuple[torch.Tensor, torch.Tensor]:
    _check_qkv(q, k, v)
    q, k, v = _rowmajor(q), _rowmajor(k), _rowmajor(v)
    B, H, T, D = q.shape
    out = torch.empty((B, H, T, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, H, T), dtype=torch.float32, device=q.device)
    R, W = (0, 0) if link_bits is None else (link_bits.shape[1], link_bits.shape[2])
    with torch.cuda.device(q.device):
        code = _lib.lib().ts2ts_attn_fwd(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), _lib.strides3(q), _lib.strides3(k), _lib.strides3(v), B, H, T, D, scale,
            doc_ids.data_ptr(), _opt_ptr(q_row_ids), _opt_ptr(kv_col_ids), _opt_ptr(link_bits), R, W, plan.data_ptr(),
            plan.numel(), out.data_ptr(), _lib.strides3(out), lse.data_ptr(), torch.cuda.current_stream(q.device).cuda_stream)
    _lib.check(code, "ts2ts_attn_fwd")
    return out, lse


@_attn_fwd.register_fake
def _(q, k, v, doc_ids, link_bits, q_row_ids, kv_col_ids, plan, scale):
    B, H, T, D = q.shape
    return q.new_empty((B, H, T, D)), q.new_empty((B, H, T), dtype=torch.float32)


@torch.library.custom_op("ts2ts::masked_attn_bwd", mutates_args=())
def _attn_bwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor, dout: torch.Tensor, lse: torch.Tensor,
              doc_ids: torch.Tensor, link_bits: Optional[torch.Tensor], q_row_ids: Optional[torch.Tensor],
              kv_col_ids: Optional[torch.Tensor], plan: torch.Tensor, scale: float) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    q, k, v, out, dout = (_rowmajor(t) for t in (q, k, v, out, dout))
    B, H, T, D = q.shape
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    dq, dk, dv = _rowmajor(dq), _rowmajor(dk), _rowmajor(dv)
    L = _lib.lib()
    ws = torch.empty(L.ts2ts_attn_bwd_workspace_bytes(B, H, T, D), dtype=torch.uint8, device=q.device)
    R, W = (0, 0) if link_bits is None else (link_bits.shape[1], link_bits.shape[2])
    with torch.cuda.device(q.device):
        code = L.ts2ts_attn_bwd(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), dout.data_ptr(), lse.data_ptr(), _lib.strides3(q),
            _lib.strides3(k), _lib.strides3(v), _lib.strides3(out), _lib.strides3(dout), B, H, T, D, scale, doc_ids.data_ptr(),
            _opt_ptr(q_row_ids), _opt_ptr(kv_col_ids), _opt_ptr(link_bits), R, W, plan.data_ptr(), plan.numel(), dq.data_ptr(),
            dk.data_ptr(), dv.data_ptr(), _lib.strides3(dq), _lib.strides3(dk), _lib.strides3(dv), ws.data_ptr(), ws.numel(),
            torch.cuda.current_stream(q.device).cuda_stream)
    _lib.check(code, "ts2ts_attn_bwd")
    return dq, dk, dv


@_attn_bwd.register_fake
def _(q, k, v, out, dout, lse, doc_ids, link_bits, q_row_ids, kv_col_ids, plan, scale):
    return torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)


def _setup_context(ctx, inputs, output):
    q, k, v, doc_ids, link_bits, q_row_ids, kv_col_ids, plan, scale = inputs
    out, lse = output
    ctx.save_for_backward(q, k, v, out, lse, doc_ids, link_bits, q_row_ids, kv_col_ids, plan)
    ctx.scale = scale
    ctx.mark_non_differentiable(lse)


def _backward(ctx, dout, dlse):
    q, k, v, out, lse, doc_ids, link_bits, q_row_ids, kv_col_ids, plan = ctx.saved_tensors
    dq, dk, dv = _attn_bwd(q, k, v, out, dout, lse, doc_ids, link_bits, q_row_ids, kv_col_ids, plan, ctx.scale)
    return dq, dk, dv, None, None, None, None, None, None


_attn_fwd.register_autograd(_backward, setup_context=_setup_context)


def masked_attn(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, doc_ids: torch.Tensor,
                link_bits: Optional[torch.Tensor] = None, *, q_row_ids: Optional[torch.Tensor] = None,
                kv_col_ids: Optional[torch.Tensor] = None, scale: Optional[float] = None,
                plan: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Masked attention with autograd.

    q, k, v   bf16 [B,H,T,D] on CUDA, D in {64,128}
    doc_ids   int32 [B,T]
    link_bits int64 [B,R,W] or None (None = doc_causal): bit c of row r lets row class r read column class c
    q_row_ids / kv_col_ids  int32 [B,T] classes per token, default doc_ids
    plan      block plan from ``build_block_map`` / ``MaskSpec.plan``; built here when omitted

    allowed(q,kv) = q >= kv and (doc_ids[q] == doc_ids[kv] or bit(link_bits[row(q)], col(kv))).
    Returns (out like q, lse fp32 [B,H,T] in natural log); rows with no allowed key give out = 0, lse = -inf.
    """
    _check_qkv(q, k, v)
    if doc_ids.dtype != torch.int32 or doc_ids.shape != (q.shape[0], q.shape[2]):
        raise ValueError("doc_ids must be int32 [B,T] matching q")
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else float(scale)
    if not scale > 0:
        raise ValueError("scale must be positive")
    doc_ids = doc_ids.contiguous()
    link_bits = None if link_bits is None else link_bits.contiguous()
    q_row_ids = None if q_row_ids is None else q_row_ids.contiguous()
    kv_col_ids = None if kv_col_ids is None else kv_col_ids.contiguous()
    if plan is None:
        plan = build_block_map(doc_ids, link_bits, q_row_ids, kv_col_ids).plan
    return _attn_fwd(q, k, v, doc_ids, link_bits, q_row_ids, kv_col_ids, plan, scale)


@torch.library.custom_op("ts2ts::masked_attn_decode", mutates_args=())
def _attn_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, doc_ids: torch.Tensor,
                 link_bits: Optional[torch.Tensor], q_row_ids: Optional[torch.Tensor], kv_col_ids: Optional[torch.Tensor],
                 q_pos: Optional[torch.Tensor], scale: float) -> Tuple[torch.Tensor, torch.Tensor]:
    B, H, Tk, D = k_cache.shape
    q, k_cache, v_cache = _rowmajor(q), _rowmajor(k_cache), _rowmajor(v_cache)
    out = torch.empty((B, H, 1, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, H), dtype=torch.float32, device=q.device)
    L = _lib.lib()
    ws = torch.empty(L.ts2ts_attn_decode_workspace_bytes(B, H, Tk, D), dtype=torch.uint8, device=q.device)
    R, W = (0, 0) if link_bits is None else (link_bits.shape[1], link_bits.shape[2])
    with torch.cuda.device(q.device):
        code = L.ts2ts_attn_decode(
            q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), _lib.strides3(q), _lib.strides3(k_cache), _lib.strides3(v_cache),
            B, H, Tk, D, scale, doc_ids.data_ptr(), _opt_ptr(q_row_ids), _opt_ptr(kv_col_ids), _opt_ptr(link_bits), R, W,
            _opt_ptr(q_pos), out.data_ptr(), _lib.strides3(out), lse.data_ptr(), ws.data_ptr(), ws.numel(),
            torch.cuda.current_stream(q.device).cuda_stream)
    _lib.check(code, "ts2ts_attn_decode")
    return out, lse


@_attn_decode.register_fake
def _(q, k_cache, v_cache, doc_ids, link_bits, q_row_ids, kv_col_ids, q_pos, scale):
    B, H, Tk, D = k_cache.shape
    return q.new_empty((B, H, 1, D)), q.new_empty((B, H), dtype=torch.float32)


def masked_attn_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, doc_ids: torch.Tensor,
                       link_bits: Optional[torch.Tensor] = None, *, q_row_ids: Optional[torch.Tensor] = None,
                       kv_col_ids: Optional[torch.Tensor] = None, q_pos: Optional[torch.Tensor] = None,
                       scale: Optional[float] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """One decoding step with KV reuse: the attention row of the newest token of every sequence.

    q        bf16 [B,H,1,D]: the new token's query
    k_cache, v_cache   bf16 [B,H,Tk,D]: keys / values of tokens 0..Tk-1, the new token's included
    doc_ids (and q_row_ids / kv_col_ids / link_bits as in ``masked_attn``) describe all Tk cached tokens
    q_pos    int32 [B] position of the query token (default Tk - 1); later keys are never read

    Returns (out bf16 [B,H,1,D], lse fp32 [B,H]); equal to row q_pos of ``masked_attn`` over the same Tk tokens, which
    is what the reference obtains by recomputing the whole sequence for every generated token
    (model/generation_loop.py:90-92).  Forward only."""
    if not (q.is_cuda and k_cache.is_cuda and v_cache.is_cuda):
        raise RuntimeError("ts2ts::masked_attn_decode runs on CUDA tensors only (no CPU path exists)")
    if q.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16 or v_cache.dtype != torch.bfloat16:
        raise TypeError("q, k_cache, v_cache must be bfloat16")
    if k_cache.dim() != 4 or k_cache.shape != v_cache.shape or q.shape != (k_cache.shape[0], k_cache.shape[1], 1, k_cache.shape[3]):
        raise ValueError("expected q [B,H,1,D] and k_cache, v_cache [B,H,Tk,D]")
    if k_cache.shape[-1] not in (64, 128):
        raise ValueError("head dimension must be 64 or 128")
    if doc_ids.dtype != torch.int32 or doc_ids.shape != (k_cache.shape[0], k_cache.shape[2]):
        raise ValueError("doc_ids must be int32 [B,Tk] matching the cache")
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else float(scale)
    if not scale > 0:
        raise ValueError("scale must be positive")
    cont = lambda t: None if t is None else t.contiguous()
    if q_pos is not None and (q_pos.dtype != torch.int32 or q_pos.shape != (k_cache.shape[0],)):
        raise ValueError("q_pos must be int32 [B]")
    return _attn_decode(q, k_cache, v_cache, doc_ids.contiguous(), cont(link_bits), cont(q_row_ids), cont(kv_col_ids), cont(q_pos), scale)


def flex_attention(query, key, value, score_mod=None, block_mask=None, scale=None, enable_gqa=False, return_lse=False,
                   kernel_options=None, *, return_aux=None):
    """Drop-in for ``torch.nn.attention.flex_attention.flex_attention`` on the reference's call path, where
    ``block_mask`` is the ``MaskSpec`` produced by this package's mask creators."""
    if score_mod is not None or enable_gqa or return_aux is not None:
        raise NotImplementedError("only block_mask / scale / return_lse are used on the reference's path")
    if not isinstance(block_mask, MaskSpec):
        raise TypeError("block_mask must be a MaskSpec from tagseq2tagseq_b200.mask_spec")
    m = block_mask.expanded(query.shape[0])  # a one-sequence spec serves every sequence of the batch; its plan is cached
    out, lse = masked_attn(query, key, value, m.doc_ids, m.link_bits, q_row_ids=m.q_row_ids, kv_col_ids=m.kv_col_ids,
                           scale=scale, plan=m.plan)
    return (out, lse) if return_lse else out
