"""128x128 block map of a dense mask, restated on the CPU.  Test infrastructure only.

Follows what ``torch.nn.attention.flex_attention.create_block_mask`` does for
the reference (called at block_mask_creator.py:132-139 and
cross_doc_mask.py:359-366): pad the dense mask with False to a multiple of the
block size, sum each block, call a block *full* when the sum equals
block*block and *partial* when it is strictly between
(torch/nn/attention/flex_attention.py:1034-1084); the index lists are the
positions of the ones in ascending order (stable descending argsort of a 0/1
row, torch/nn/attention/flex_attention.py:402-409) and the backward lists are
the same construction on the transposed maps (1130-1153).
"""
from __future__ import annotations

import numpy as np

SKIP, PARTIAL, FULL = 0, 1, 2


def block_states(dense: np.ndarray, block: int = 128) -> np.ndarray:
    """uint8[QB,KB] in {0 skip, 1 partial, 2 full}."""
    t_q, t_k = dense.shape
    qb, kb = -(-t_q // block), -(-t_k // block)
    pad = np.zeros((qb * block, kb * block), dtype=np.int64)
    pad[:t_q, :t_k] = dense
    sums = pad.reshape(qb, block, kb, block).sum(axis=(1, 3))
    st = np.zeros((qb, kb), dtype=np.uint8)
    st[sums > 0] = PARTIAL
    st[sums == block * block] = FULL
    return st


def block_states_streamed(doc_ids, q_row_ids, kv_col_ids, link_bits, block: int = 128) -> np.ndarray:
    """Same map as ``block_states(class_mask_dense(...))`` computed one 128-row slab at a time, so that
    32k-token sequences need 4 MB of mask at once instead of 1 GB."""
    from .masks import class_mask_dense
    t = doc_ids.shape[0]
    nb = -(-t // block)
    st = np.zeros((nb, nb), dtype=np.uint8)
    for qb in range(nb):
        q0, q1 = qb * block, min(t, (qb + 1) * block)
        slab = class_mask_dense(doc_ids, q_row_ids, kv_col_ids, link_bits, q_range=(q0, q1))
        pad = np.zeros((q1 - q0, nb * block), dtype=np.int32)
        pad[:, :t] = slab
        sums = pad.reshape(q1 - q0, nb, block).sum(axis=(0, 2))
        st[qb, sums > 0] = PARTIAL
        st[qb, sums == block * block] = FULL
    return st


def lists_from_states(state: np.ndarray):
    """Ordered lists in the BlockMask convention.  Returns a dict with
    ``kv_cnt[QB]``, ``kv_idx[QB,KB]`` (partial), ``full_cnt``, ``full_idx``,
    and the transposed ``q_cnt[KB]``, ``q_idx[KB,QB]``, ``full_q_cnt``,
    ``full_q_idx``.  Entries past the count are -1."""
    def one(mat):
        n_r, n_c = mat.shape
        cnt = mat.sum(axis=1).astype(np.int32)
        idx = np.full((n_r, n_c), -1, dtype=np.int32)
        for r in range(n_r):
            nz = np.nonzero(mat[r])[0]
            idx[r, : nz.size] = nz
        return cnt, idx
    part = state == PARTIAL
    full = state == FULL
    out = {}
    out["kv_cnt"], out["kv_idx"] = one(part)
    out["full_cnt"], out["full_idx"] = one(full)
    out["q_cnt"], out["q_idx"] = one(part.T)
    out["full_q_cnt"], out["full_q_idx"] = one(full.T)
    return out
