"""Mask layer: what the reference's block_mask_creator callables return, re-expressed for the CUDA path.

The reference builds a torch ``BlockMask`` by materialising the dense T x T mask
(model/graph_traversal/block_mask_creator.py:87-141, cross_doc_mask.py:302-369).  Here a mask is a
``MaskSpec``: per-token document ids plus, for ``cross_doc_link``, per-token row / column classes and
a small row-class x column-class bit matrix.  The 128x128 block map is derived from it on the GPU by
``ts2ts_block_map`` and cached on the spec, so one spec serves every layer and head of a micro-batch.

The callables mirror the reference's names and signatures:
``create_doc_causal_block_mask``, ``CrossDocLinkMaskCreator``, ``MASK_CREATORS``, ``get_mask_creator``,
``list_mask_creators``, ``make_mask_creator_callable_from``, ``make_mask_creator_callable``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Dict, List, NamedTuple, Optional, Sequence, Tuple

import numpy as np
import torch

from . import _lib

TILE = 128


@dataclass
class DocSpan:
    """Where one document sits in a packed sequence (fields of data/collate.py:16-33)."""
    doc_id: int
    normed_identifier: str
    start: int  # inclusive
    end: int    # exclusive
    truncated: bool = False
    outgoing_identifiers: List[str] = field(default_factory=list)
    raw_identifier: str = ""


class LinkInfo(NamedTuple):
    """A detected link (model/graph_traversal/link_detector.py:15-19)."""
    link_end_pos: int
    target_str: str


class BlockMap(NamedTuple):
    """Output of the pre-pass.  ``plan`` is the opaque device buffer the attention kernels read; the other
    fields are the BlockMask-shaped views (``None`` when not requested)."""
    plan: torch.Tensor
    state: Optional[torch.Tensor] = None
    kv_cnt: Optional[torch.Tensor] = None
    kv_idx: Optional[torch.Tensor] = None
    full_cnt: Optional[torch.Tensor] = None
    full_idx: Optional[torch.Tensor] = None
    q_cnt: Optional[torch.Tensor] = None
    q_idx: Optional[torch.Tensor] = None
    full_q_cnt: Optional[torch.Tensor] = None
    full_q_idx: Optional[torch.Tensor] = None


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _check_mask_tensors(doc_ids, link_bits, q_row_ids, kv_col_ids):
    if doc_ids.dim() != 2 or doc_ids.dtype != torch.int32:
        raise ValueError("doc_ids must be int32 [B,T]")
    if not doc_ids.is_cuda:
        raise RuntimeError("the masked-attention path runs on CUDA only; doc_ids is not a CUDA tensor")
    for name, t in (("q_row_ids", q_row_ids), ("kv_col_ids", kv_col_ids)):
        if t is not None and (t.shape != doc_ids.shape or t.dtype != torch.int32 or t.device != doc_ids.device):
            raise ValueError(f"{name} must be int32 on the same device with the shape of doc_ids")
    if link_bits is not None:
        if link_bits.dim() != 3 or link_bits.dtype != torch.int64 or link_bits.shape[0] != doc_ids.shape[0]:
            raise ValueError("link_bits must be int64 [B,R,W]")
        if link_bits.device != doc_ids.device:
            raise ValueError("link_bits must be on the device of doc_ids")


def build_block_map(doc_ids: torch.Tensor, link_bits: Optional[torch.Tensor] = None,
                    q_row_ids: Optional[torch.Tensor] = None, kv_col_ids: Optional[torch.Tensor] = None,
                    with_lists: bool = False) -> BlockMap:
    """Run the integer pre-pass (``ts2ts_block_map``) on the current stream."""
    _check_mask_tensors(doc_ids, link_bits, q_row_ids, kv_col_ids)
    L = _lib.lib()
    doc_ids = doc_ids.contiguous()
    link_bits = None if link_bits is None else link_bits.contiguous()
    q_row_ids = None if q_row_ids is None else q_row_ids.contiguous()
    kv_col_ids = None if kv_col_ids is None else kv_col_ids.contiguous()
    B, T = doc_ids.shape
    if T == 0 or B == 0:
        raise ValueError("empty sequence")
    nb = (T + TILE - 1) // TILE
    dev = doc_ids.device
    with torch.cuda.device(dev):
        plan = torch.empty(L.ts2ts_plan_bytes(B, T), dtype=torch.uint8, device=dev)
        outs = [None] * 9
        if with_lists:
            outs[0] = torch.empty((B, nb, nb), dtype=torch.uint8, device=dev)
            for i in (1, 3, 5, 7):
                outs[i] = torch.empty((B, nb), dtype=torch.int32, device=dev)
                outs[i + 1] = torch.empty((B, nb, nb), dtype=torch.int32, device=dev)
        R, W = (0, 0) if link_bits is None else (link_bits.shape[1], link_bits.shape[2])
        code = L.ts2ts_block_map(_ptr(doc_ids), _ptr(q_row_ids), _ptr(kv_col_ids), _ptr(link_bits), B, T, R, W,
                                 plan.data_ptr(), plan.numel(), *[_ptr(o) for o in outs],
                                 torch.cuda.current_stream(dev).cuda_stream)
    _lib.check(code, "ts2ts_block_map")
    return BlockMap(plan, *outs)


def read_status(plan: torch.Tensor) -> int:
    """Synchronise and return the device status word of a plan (0 = all kernels completed normally)."""
    import ctypes
    out = ctypes.c_int32(0)
    with torch.cuda.device(plan.device):
        code = _lib.lib().ts2ts_read_status(plan.data_ptr(), torch.cuda.current_stream(plan.device).cuda_stream, ctypes.byref(out))
    if code < 0:
        _lib.check(code, "ts2ts_read_status")
    return int(out.value)  # a positive return value is the recorded code itself


@dataclass
class MaskSpec:
    """The object passed where the reference passes a ``BlockMask``
    (training_module.py:199-200 -> backbone.py:70 -> layer.py:32-33)."""
    doc_ids: torch.Tensor                      # int32 [B,T]
    link_bits: Optional[torch.Tensor] = None   # int64 [B,R,W]
    q_row_ids: Optional[torch.Tensor] = None   # int32 [B,T]
    kv_col_ids: Optional[torch.Tensor] = None  # int32 [B,T]
    _block_map: Optional[BlockMap] = None
    _expanded: Optional[Dict[int, "MaskSpec"]] = None

    def expanded(self, batch: int) -> "MaskSpec":
        """This spec repeated over ``batch`` sequences (the reference's B=None BlockMask broadcasts over the batch),
        with its own block plan; built once per batch size and kept."""
        if self.doc_ids.shape[0] == batch:
            return self
        if self.doc_ids.shape[0] != 1:
            raise ValueError("only a spec of one sequence can be broadcast over a batch")
        if self._expanded is None:
            self._expanded = {}
        if batch not in self._expanded:
            rep = lambda t: None if t is None else t.expand(batch, *t.shape[1:]).contiguous()
            self._expanded[batch] = MaskSpec(rep(self.doc_ids), rep(self.link_bits), rep(self.q_row_ids), rep(self.kv_col_ids))
        return self._expanded[batch]

    @property
    def seq_len(self) -> int:
        return int(self.doc_ids.shape[1])

    @property
    def seq_lengths(self) -> Tuple[int, int]:  # BlockMask.seq_lengths
        return (self.seq_len, self.seq_len)

    BLOCK_SIZE = (TILE, TILE)

    def block_map(self, with_lists: bool = False) -> BlockMap:
        if self._block_map is None or (with_lists and self._block_map.state is None):
            self._block_map = build_block_map(self.doc_ids, self.link_bits, self.q_row_ids, self.kv_col_ids, with_lists)
        return self._block_map

    @property
    def plan(self) -> torch.Tensor:
        return self.block_map().plan


# --------------------------------------------------------------------------------------------- host adapters

def build_document_ids(seq_len: int, doc_spans: Sequence[Any]) -> np.ndarray:
    """int32[T]: doc id per token, -1 where uncovered, spans clipped to [0,T)
    (block_mask_creator.py:107-117)."""
    ids = np.full(seq_len, -1, dtype=np.int32)
    for s in doc_spans:
        a, b = max(0, s.start), min(seq_len, s.end)
        if a < b:
            ids[a:b] = s.doc_id
    return ids


def ordered_grants(seq_len: int, doc_spans: Sequence[Any], link_to_target: Dict[int, List[int]], cap: int):
    """The (q0, q1, kv0, kv1) ranges that receive a grant bit, in bit order, under the reference's
    rules (cross_doc_mask.py:239-294): links by ascending position, targets in list order, source span
    = first span with start < pos <= end, target span = first span with that doc_id, both clipped to
    [0,T); empty ranges are dropped without using a bit; the first grant beyond ``cap`` ends everything."""
    by_id: Dict[int, Any] = {}
    for s in doc_spans:
        by_id.setdefault(s.doc_id, s)
    grants = []
    for pos in sorted(link_to_target):
        src = next((s for s in doc_spans if s.start < pos <= s.end), None)
        stop = False
        for tgt_id in link_to_target[pos]:
            if len(grants) >= cap:
                stop = True
                break
            tgt = by_id.get(tgt_id)
            if src is None or tgt is None:
                continue
            q0, q1 = pos, min(seq_len, src.end)
            k0, k1 = max(0, tgt.start), min(seq_len, tgt.end)
            if q0 < q1 and k0 < k1:
                grants.append((q0, q1, k0, k1))
        if stop:
            break
    return grants


def grant_classes(seq_len: int, grants: Sequence[Tuple[int, int, int, int]]):
    """Fold a grant list into (q_row_ids int32[T], kv_col_ids int32[T], link_bits int64[R,W]).

    Tokens covered by the same set of grants form one class; bit c of row r says some grant covers
    both -- exactly ``any_c (q_bits[c][q] & kv_bits[c][kv]) != 0`` of cross_doc_mask.py:348-357."""
    n = len(grants)
    words = max(1, (n + 63) // 64)
    qb = np.zeros((seq_len, words), dtype=np.uint64)
    kb = np.zeros((seq_len, words), dtype=np.uint64)
    for g, (q0, q1, k0, k1) in enumerate(grants):
        bit = np.uint64(1) << np.uint64(g & 63)
        qb[q0:q1, g >> 6] |= bit
        kb[k0:k1, g >> 6] |= bit

    def classes(m):
        ids = np.full(seq_len, -1, dtype=np.int32)
        nz = np.nonzero(m.any(axis=1))[0]
        if nz.size == 0:
            return ids, np.zeros((0, words), dtype=np.uint64)
        pats, inv = np.unique(m[nz], axis=0, return_inverse=True)
        ids[nz] = inv.reshape(-1).astype(np.int32)
        return ids, pats

    row_ids, row_pat = classes(qb)
    col_ids, col_pat = classes(kb)
    R, C = max(1, row_pat.shape[0]), col_pat.shape[0]
    W = max(1, (C + 63) // 64)
    link = np.zeros((R, W), dtype=np.uint64)
    for c in range(C):
        hit = (row_pat & col_pat[c][None, :]).any(axis=1)
        link[: row_pat.shape[0], c >> 6] |= hit.astype(np.uint64) << np.uint64(c & 63)
    return row_ids, col_ids, link.view(np.int64)


def grant_segments(grants: Sequence[Tuple[int, int, int, int]]):
    """The same classes as ``grant_classes`` worked out on segment boundaries instead of tokens.

    The set of grants that covers a token only changes where a grant starts or ends, so there are at most 2 G + 1
    segments per side however long the sequence is.  Returns, for the query side and the key side, (bounds int32[S+1],
    ids int32[S]) with id -1 for segments no grant covers, and link_bits int64[R, W]: bit c of row r is set when some
    grant covers both row class r and column class c.  Classes are numbered in order of first appearance."""
    def side(ranges):
        pts = sorted({p for a, b in ranges for p in (a, b)})
        if not pts:
            return np.zeros(1, dtype=np.int32), np.zeros(0, dtype=np.int32), []
        bounds = np.asarray(pts, dtype=np.int32)
        starts = np.asarray([a for a, _ in ranges], dtype=np.int64)
        ends = np.asarray([b for _, b in ranges], dtype=np.int64)
        cover = (starts[None, :] <= bounds[:-1, None]) & (bounds[:-1, None] < ends[None, :])  # [S, G]
        ids, patterns, seen = np.full(len(pts) - 1, -1, dtype=np.int32), [], {}
        for j in range(len(pts) - 1):
            if not cover[j].any():
                continue
            key = cover[j].tobytes()
            if key not in seen:
                seen[key] = len(patterns)
                patterns.append(cover[j])
            ids[j] = seen[key]
        return bounds, ids, patterns

    qb, qi, rows = side([(g[0], g[1]) for g in grants])
    kb, ki, cols = side([(g[2], g[3]) for g in grants])
    R, C = max(1, len(rows)), len(cols)
    W = max(1, (C + 63) // 64)
    link = np.zeros((R, W), dtype=np.uint64)
    if rows and cols:
        hit = (np.stack(rows)[:, None, :] & np.stack(cols)[None, :, :]).any(axis=2)  # [R, C]
        for c in range(C):
            link[: len(rows), c >> 6] |= hit[:, c].astype(np.uint64) << np.uint64(c & 63)
    return (qb, qi), (kb, ki), link.view(np.int64)


def segment_ids(bounds: np.ndarray, ids: np.ndarray, seq_len: int, device: torch.device) -> torch.Tensor:
    """int32[1, T] on the device from a segment table (``ts2ts_segment_ids``): one small host-to-device copy of the
    table, then one kernel; nothing of length T crosses PCIe."""
    table = torch.from_numpy(np.concatenate([bounds.astype(np.int32), ids.astype(np.int32)])).to(device, non_blocking=True)
    out = torch.empty((1, seq_len), dtype=torch.int32, device=device)
    n_seg = int(ids.shape[0])
    with torch.cuda.device(device):
        code = _lib.lib().ts2ts_segment_ids(table.data_ptr(), table.data_ptr() + 4 * (n_seg + 1), n_seg, seq_len, out.data_ptr(),
                                            torch.cuda.current_stream(device).cuda_stream)
    _lib.check(code, "ts2ts_segment_ids")
    return out


def from_reference(doc_spans: Sequence[Any], link_to_target: Optional[Dict[int, List[int]]], seq_len: int,
                   max_grants_cap: int = 64, device: Optional[torch.device] = None) -> MaskSpec:
    """MaskSpec equal to the reference's mask for these spans and matched links
    (``doc_causal`` when ``link_to_target`` is None or empty)."""
    device = torch.device("cuda") if device is None else device
    ids = torch.from_numpy(build_document_ids(seq_len, doc_spans))[None].to(device)
    if not link_to_target:
        return MaskSpec(doc_ids=ids)
    grants = ordered_grants(seq_len, doc_spans, link_to_target, max_grants_cap)
    if not grants:
        return MaskSpec(doc_ids=ids)
    if torch.device(device).type == "cuda":  # classes on segment boundaries (host, O(G^2)); per-token ids filled on the device
        (qb, qi), (kb, ki), link = grant_segments(grants)
        return MaskSpec(doc_ids=ids, link_bits=torch.from_numpy(link)[None].to(device),
                        q_row_ids=segment_ids(qb, qi, seq_len, device), kv_col_ids=segment_ids(kb, ki, seq_len, device))
    row, col, link = grant_classes(seq_len, grants)
    return MaskSpec(doc_ids=ids, link_bits=torch.from_numpy(link)[None].to(device),
                    q_row_ids=torch.from_numpy(row)[None].to(device), kv_col_ids=torch.from_numpy(col)[None].to(device))


# --------------------------------------------------------------------------------------------- creators

def create_doc_causal_block_mask(tokens: torch.Tensor, doc_spans: List[Any], **kwargs) -> MaskSpec:
    """Causal attention inside each document only (block_mask_creator.py:87-141)."""
    return from_reference(doc_spans, None, tokens.shape[-1], device=tokens.device)


class CrossDocLinkMaskCreator:
    """doc_causal plus link grants: tokens from a link's end to the end of the linking document may read
    the whole target document (cross_doc_mask.py:26-85, 302-369).  Same constructor arguments and
    ``max_grants`` cosine warm-up as the reference; returns a ``MaskSpec``."""

    def __init__(self, link_detector, max_grants: int = 64, max_grants_start: Optional[int] = None,
                 max_grants_warmup_steps: int = 0):
        self.link_detector = link_detector
        self.max_grants = max_grants
        self._max_grants_start = max_grants_start if max_grants_start is not None else max_grants
        self._max_grants_warmup_steps = max_grants_warmup_steps
        self._step = 0
        self._n_chunks = max(1, (max_grants + 63) // 64)

    def _current_max_grants(self) -> int:
        if self._max_grants_warmup_steps <= 0 or self._step >= self._max_grants_warmup_steps:
            return self.max_grants
        frac = self._step / self._max_grants_warmup_steps
        return round(self._max_grants_start
                     + (self.max_grants - self._max_grants_start) * (1.0 - math.cos(math.pi * frac)) / 2.0)

    def _match_links_to_docs(self, links, doc_spans) -> Dict[int, List[int]]:
        """link_end_pos -> [target doc ids]; a target must start before the link (cross_doc_mask.py:87-149)."""
        index = {}
        for span in doc_spans:
            index[self.link_detector.index_doc_span(span)] = (span.doc_id, span.start)
        out: Dict[int, List[int]] = {}
        for link in links:
            hit = index.get(link.target_str)
            if hit is None or hit[1] >= link.link_end_pos:
                continue
            out.setdefault(link.link_end_pos, []).append(hit[0])
        return out

    def __call__(self, tokens: torch.Tensor, doc_spans: List[Any], **kwargs) -> MaskSpec:
        seq_len = tokens.shape[-1]
        links = self.link_detector.detect_links(tokens[0])
        link_to_target = self._match_links_to_docs(links, doc_spans)
        cap = self._current_max_grants()
        self._step += 1
        return from_reference(doc_spans, link_to_target, seq_len, max_grants_cap=cap, device=tokens.device)


def create_causal_block_mask(tokens: torch.Tensor, doc_spans: List[Any], **kwargs) -> MaskSpec:
    """Plain causal attention over the whole sequence (block_mask_creator.py:143-172): one document id everywhere,
    so the doc_causal kernels compute it unchanged."""
    seq_len = tokens.shape[-1]
    return MaskSpec(doc_ids=torch.zeros((1, seq_len), dtype=torch.int32, device=tokens.device))


def _needs_non_causal_kernel(name: str):
    def creator(tokens: torch.Tensor, doc_spans: List[Any], **kwargs) -> MaskSpec:
        raise NotImplementedError(
            f"mask creator '{name}' lets queries read later keys; the CUDA kernels of this package are causal "
            "(every mask is intersected with q >= kv), so a non-causal forward / backward kernel would be needed")
    return creator


MASK_CREATORS = {
    "doc_causal": create_doc_causal_block_mask,
    "causal": create_causal_block_mask,
    # present in the reference's registry (block_mask_creator.py:251-256) but not computable by causal kernels:
    "full": _needs_non_causal_kernel("full"),
    "doc_bidirectional": _needs_non_causal_kernel("doc_bidirectional"),
    # 'cross_doc_link' needs a LinkDetector: build CrossDocLinkMaskCreator yourself and wrap it with
    # make_mask_creator_callable_from (same rule as block_mask_creator.py:254-263).
}


def get_mask_creator(name: str):
    if name not in MASK_CREATORS:
        raise ValueError(f"Unknown mask creator '{name}'. Available options: {', '.join(MASK_CREATORS)}")
    return MASK_CREATORS[name]


def list_mask_creators() -> List[str]:
    return list(MASK_CREATORS)


def make_mask_creator_callable_from(creator):
    """(**batch) -> MaskSpec adapter, as block_mask_creator.py:288-317."""

    @torch._dynamo.disable
    def callable_wrapper(**batch):
        tokens = batch.get("tokens")
        if tokens is None:
            raise ValueError("Batch must contain 'tokens' key")
        extra = {k: v for k, v in batch.items() if k not in ("tokens", "doc_spans")}
        return creator(tokens, batch.get("doc_spans", []), **extra)

    return callable_wrapper


def make_mask_creator_callable(mask_type: str):
    return make_mask_creator_callable_from(get_mask_creator(mask_type))
