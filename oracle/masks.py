"""Mask construction restated on the CPU (numpy).  Test infrastructure only.

Every function cites the reference lines it follows.  Spans are any objects
with ``doc_id``, ``start`` and ``end`` attributes (data/collate.py:16-33).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

INT64_MIN = -(1 << 63)


def document_ids(seq_len: int, spans: Sequence) -> np.ndarray:
    """int32[T] doc id per token, -1 where no span covers it; spans are clipped
    to [0, T) and later spans overwrite earlier ones
    (block_mask_creator.py:107-117, cross_doc_mask.py:325-330)."""
    ids = np.full((seq_len,), -1, dtype=np.int32)
    for s in spans:
        a, b = max(0, s.start), min(seq_len, s.end)
        if a < b:
            ids[a:b] = s.doc_id
    return ids


def doc_causal_dense(doc_ids: np.ndarray) -> np.ndarray:
    """bool[T,T]: q >= kv and same document (block_mask_creator.py:121-129)."""
    t = doc_ids.shape[0]
    q = np.arange(t)[:, None]
    kv = np.arange(t)[None, :]
    return (q >= kv) & (doc_ids[:, None] == doc_ids[None, :])


def _find_grant(seq_len, spans, link_pos, target_doc_id):
    """Source / target span lookup and clipping shared by the dense and the
    bitmask construction (cross_doc_mask.py:175-202 and 258-281).  Returns
    ``None`` when the grant is dropped, else (q0, q1, kv0, kv1); the ranges may
    be empty, which the callers test exactly like the reference does."""
    src = None
    for s in spans:
        if s.start < link_pos <= s.end:  # link_end_pos is exclusive
            src = s
            break
    if src is None:
        return None
    tgt = None
    for s in spans:
        if s.doc_id == target_doc_id:
            tgt = s
            break
    if tgt is None:
        return None
    return (link_pos, min(seq_len, src.end), max(0, tgt.start), min(seq_len, tgt.end))


def cross_doc_dense(seq_len: int, spans: Sequence, link_to_target: Dict[int, List[int]]) -> np.ndarray:
    """bool[T,T] link grants only, no cap (cross_doc_mask.py:151-208)."""
    m = np.zeros((seq_len, seq_len), dtype=bool)
    for link_pos, targets in sorted(link_to_target.items()):
        for tgt in targets:
            g = _find_grant(seq_len, spans, link_pos, tgt)
            if g is None:
                continue
            q0, q1, k0, k1 = g
            if q0 < q1 and k0 < k1:
                m[q0:q1, k0:k1] = True
    return m


def grant_bitmasks(seq_len: int, spans: Sequence, link_to_target: Dict[int, List[int]],
                   max_grants: int = 64, cap: Optional[int] = None) -> Tuple[np.ndarray, np.ndarray]:
    """int64[n_chunks,T] query and key bitmasks (cross_doc_mask.py:210-300).

    Grants are taken in ``sorted(link_to_target.items())`` order; grant k sets
    bit k%64 of chunk k//64 (bit 63 is INT64_MIN); only grants with non-empty
    ranges consume an index; the first grant that would exceed ``cap`` ends the
    whole construction."""
    n_chunks = max(1, (max_grants + 63) // 64)
    cap = max_grants if cap is None else cap
    qb = np.zeros((n_chunks, seq_len), dtype=np.int64)
    kb = np.zeros((n_chunks, seq_len), dtype=np.int64)
    idx = 0
    truncated = False
    for link_pos, targets in sorted(link_to_target.items()):
        if truncated:
            break
        for tgt in targets:
            if idx >= cap:
                truncated = True
                break
            g = _find_grant(seq_len, spans, link_pos, tgt)
            if g is None:
                continue
            q0, q1, k0, k1 = g
            if q0 < q1 and k0 < k1:
                chunk, bit_pos = idx // 64, idx % 64
                bit = np.int64((1 << bit_pos) if bit_pos < 63 else INT64_MIN)
                qb[chunk, q0:q1] |= bit
                kb[chunk, k0:k1] |= bit
                idx += 1
    return qb, kb


def bitmask_grant_dense(q_bits: np.ndarray, kv_bits: np.ndarray) -> np.ndarray:
    """bool[T,T]: some chunk has a common bit (cross_doc_mask.py:352-355)."""
    out = np.zeros((q_bits.shape[1], kv_bits.shape[1]), dtype=bool)
    for c in range(q_bits.shape[0]):
        out |= (q_bits[c][:, None] & kv_bits[c][None, :]) != 0
    return out


def cross_doc_link_dense(doc_ids: np.ndarray, q_bits: np.ndarray, kv_bits: np.ndarray) -> np.ndarray:
    """bool[T,T]: causal and (same doc or in a grant) (cross_doc_mask.py:348-357)."""
    t = doc_ids.shape[0]
    causal = np.arange(t)[:, None] >= np.arange(t)[None, :]
    same = doc_ids[:, None] == doc_ids[None, :]
    return causal & (same | bitmask_grant_dense(q_bits, kv_bits))


def visualization_dense(seq_len: int, spans: Sequence, link_to_target: Dict[int, List[int]]) -> np.ndarray:
    """bool[T,T] uncapped dense twin (cross_doc_mask.py:371-409)."""
    ids = document_ids(seq_len, spans)
    t = seq_len
    causal = np.arange(t)[:, None] >= np.arange(t)[None, :]
    same = ids[:, None] == ids[None, :]
    return causal & (same | cross_doc_dense(seq_len, spans, link_to_target))


def class_mask_dense(doc_ids: np.ndarray, q_row_ids: Optional[np.ndarray], kv_col_ids: Optional[np.ndarray],
                     link_bits: Optional[np.ndarray], q_range: Optional[Tuple[int, int]] = None) -> np.ndarray:
    """bool[T,T] (or the row slab [q0:q1, T] when ``q_range`` is given) for the operator's own mask
    encoding (one batch element):

        q >= kv and (doc[q] == doc[kv] or bit(link_bits[row[q]], col[kv]))

    ``link_bits`` is int64[R,W]; a negative row or column class grants nothing.
    This is the same predicate as cross_doc_mask.py:348-357 with the grant
    test factored through (row class, column class)."""
    t = doc_ids.shape[0]
    q0, q1 = (0, t) if q_range is None else q_range
    causal = np.arange(q0, q1)[:, None] >= np.arange(t)[None, :]
    m = doc_ids[q0:q1, None] == doc_ids[None, :]
    if link_bits is not None and link_bits.size:
        row = (doc_ids if q_row_ids is None else q_row_ids)[q0:q1]
        col = doc_ids if kv_col_ids is None else kv_col_ids
        r_n, w_n = link_bits.shape
        table = np.zeros((r_n + 1, 64 * w_n + 1), dtype=bool)  # last row / col = "no class"
        u = link_bits.astype(np.int64).view(np.uint64)
        for w in range(w_n):
            for b in range(64):
                table[:r_n, 64 * w + b] = ((u[:, w] >> np.uint64(b)) & np.uint64(1)).astype(bool)
        ri = np.where((row >= 0) & (row < r_n), row, r_n)
        ci = np.where((col >= 0) & (col < 64 * w_n), col, 64 * w_n)
        m = m | table[ri][:, ci]
    return causal & m
