"""Dense-masked attention in fp32, forward and backward.  Test infrastructure only.

Conventions of the reference's attention operator (PyTorch FlexAttention,
reached from model/modules/layer.py:33): ``O = softmax(scale * Q K^T + mask) V``,
``LSE`` in natural log, a fully masked row gives O = 0, LSE = -inf and no
gradient (torch/_higher_order_ops/flex_attention.py:218-287, 947-1075).  The
backward is written out explicitly (P = exp(S - LSE), dV = P^T dO,
dP = dO V^T, dS = P * (dP - rowsum(O * dO)), dQ = scale dS K, dK = scale dS^T Q)
so it does not depend on autograd's handling of -inf rows.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch


def forward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, dense: torch.Tensor,
            scale: Optional[float] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """q,k,v [B,H,T,D] (any float dtype, upcast to fp32); dense bool [B,T,T] or [T,T].
    Returns out fp32 [B,H,T,D], lse fp32 [B,H,T]."""
    q, k, v = q.float(), k.float(), v.float()
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else scale
    m = dense if dense.dim() == 3 else dense[None]
    s = torch.matmul(q, k.transpose(-1, -2)) * scale
    s = s.masked_fill(~m[:, None], float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)[..., None])
    p = torch.where(torch.isinf(lse)[..., None], torch.zeros_like(p), p)
    return torch.matmul(p, v), lse


def forward_backward(q, k, v, dense, dout, scale: Optional[float] = None):
    """Returns (out, lse, dq, dk, dv), all fp32."""
    q, k, v, dout = q.float(), k.float(), v.float(), dout.float()
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else scale
    m = dense if dense.dim() == 3 else dense[None]
    s = torch.matmul(q, k.transpose(-1, -2)) * scale
    s = s.masked_fill(~m[:, None], float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    dead = torch.isinf(lse)
    p = torch.exp(s - torch.where(dead, torch.zeros_like(lse), lse)[..., None])
    p = torch.where(dead[..., None], torch.zeros_like(p), p)
    out = torch.matmul(p, v)
    delta = (out * dout).sum(-1, keepdim=True)
    dv = torch.matmul(p.transpose(-1, -2), dout)
    dp = torch.matmul(dout, v.transpose(-1, -2))
    ds = p * (dp - delta)
    dq = torch.matmul(ds, k) * scale
    dk = torch.matmul(ds.transpose(-1, -2), q) * scale
    return out, lse, dq, dk, dv


def forward_backward_streamed(q, k, v, dout, slab_mask, scale: Optional[float] = None, slab: int = 2048):
    """Same math as ``forward_backward`` for ONE (batch, head) slice q,k,v,dout [T,D], evaluated in slabs of query rows so
    that a 32k-token sequence needs [slab, T] scores at a time.  ``slab_mask(q0, q1)`` returns the bool mask [q1-q0, T]
    of those rows.  Runs on whatever device the inputs live on (fp32; keep TF32 matmuls off).
    Returns (out [T,D], lse [T], dq, dk, dv)."""
    q, k, v, dout = q.float(), k.float(), v.float(), dout.float()
    t, d = q.shape
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    out = torch.empty_like(q)
    lse = torch.empty(t, dtype=torch.float32, device=q.device)
    dq = torch.empty_like(q)
    dk = torch.zeros_like(k)
    dv = torch.zeros_like(v)
    for q0 in range(0, t, slab):
        q1 = min(t, q0 + slab)
        m = slab_mask(q0, q1)
        s = (q[q0:q1] @ k.T) * scale
        s = s.masked_fill(~m, float("-inf"))
        l = torch.logsumexp(s, dim=-1)
        dead = torch.isinf(l)
        p = torch.exp(s - torch.where(dead, torch.zeros_like(l), l)[:, None])
        p = torch.where(dead[:, None], torch.zeros_like(p), p)
        o = p @ v
        out[q0:q1], lse[q0:q1] = o, l
        do = dout[q0:q1]
        delta = (o * do).sum(-1, keepdim=True)
        dv += p.T @ do
        ds = p * (do @ v.T - delta)
        dq[q0:q1] = (ds @ k) * scale
        dk += (ds.T @ q[q0:q1]) * scale
    return out, lse, dq, dk, dv
