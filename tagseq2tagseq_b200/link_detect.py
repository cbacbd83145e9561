"""Markdown link detector whose token scan runs on the GPU.

Mirror of the reference's ``MarkdownLinkDetector`` (model/graph_traversal/markdown_link_detector.py:19-108): same
constructor arguments, same ``detect_links(input_ids) -> List[LinkInfo]`` and ``index_doc_span`` (the LinkDetector
protocol, model/graph_traversal/link_detector.py:22-84), so it can be handed to ``CrossDocLinkMaskCreator``
unchanged.  The reference walks the sequence with one ``.item()`` per token it looks at; here the positions of every
"[ ... ](" ... ")" candidate come from ``ts2ts_detect_links`` in one pass over the device tensor, and only the few
target tokens of each candidate are copied back and decoded (with the reference's own growing-window rule, so the
strings and the non-empty test are the reference's).

The per-token table "this token's bytes contain ')'" is built once from ``decode_fn`` over ``vocab_size`` ids.  It is
exact for byte-level BPE vocabularies (GPT-2's): ')' is a single ASCII byte, which no neighbouring token can change.
"""
from __future__ import annotations

import ctypes
from typing import Any, Callable, List, Optional, Tuple

import torch

from . import _lib
from .mask_spec import LinkInfo


class MarkdownLinkDetector:
    def __init__(self, decode_fn: Callable[[List[int]], str], window_tokens: int = 50,
                 link_start_token_ids: Optional[List[int]] = None, link_mid_token_id: int = 16151,
                 vocab_size: int = 50257):
        if link_start_token_ids is None:
            link_start_token_ids = [58, 685]  # '[' and ' [' in GPT-2
        if not 1 <= len(set(link_start_token_ids)) <= 8:
            raise ValueError("between 1 and 8 link start token ids are supported")
        self.decode_fn = decode_fn
        self.window_tokens = int(window_tokens)
        self.link_start_token_ids = set(link_start_token_ids)
        self.link_mid_token_id = int(link_mid_token_id)
        self.vocab_size = int(vocab_size)
        self._close_host: Optional[torch.Tensor] = None
        self._close_dev = {}

    def index_doc_span(self, span: Any) -> str:
        """Exact match against ``raw_identifier`` (markdown_link_detector.py:53-55)."""
        return span.raw_identifier

    # ------------------------------------------------------------------ device side
    def _close_flags(self, device: torch.device) -> torch.Tensor:
        if self._close_host is None:
            flags = torch.zeros(self.vocab_size, dtype=torch.uint8)
            for tok in range(self.vocab_size):
                try:
                    if ")" in self.decode_fn([tok]):
                        flags[tok] = 1
                except Exception:  # ids the tokenizer does not know never close a link
                    pass
            self._close_host = flags
        key = (device.type, device.index)
        if key not in self._close_dev:
            self._close_dev[key] = self._close_host.to(device)
        return self._close_dev[key]

    def candidates(self, input_ids: torch.Tensor) -> List[Tuple[int, int, int]]:
        """(position of '](', position of '[', position of the closing token) for every candidate, ascending."""
        if input_ids.dim() != 1:
            raise ValueError("input_ids must be 1-D")
        if not input_ids.is_cuda:
            raise RuntimeError("the link scan runs on the GPU: input_ids must be a CUDA tensor (there is no CPU path)")
        if input_ids.dtype not in (torch.int32, torch.int64):
            raise TypeError("input_ids must be int32 or int64")
        T = input_ids.shape[0]
        if T == 0:
            return []
        tokens = input_ids.contiguous()
        L = _lib.lib()
        dev = tokens.device
        flags = self._close_flags(dev)
        starts = sorted(self.link_start_token_ids)
        start_arr = (ctypes.c_int64 * len(starts))(*starts)
        with torch.cuda.device(dev):
            scratch = torch.empty(L.ts2ts_detect_links_scratch_bytes(T), dtype=torch.uint8, device=dev)
            stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
            max_links = 1024
            while True:
                out = torch.empty((max_links, 3), dtype=torch.int32, device=dev)
                count = torch.zeros(1, dtype=torch.int32, device=dev)
                _lib.check(L.ts2ts_detect_links(tokens.data_ptr(), tokens.element_size(), T, self.link_mid_token_id, start_arr,
                                                len(starts), flags.data_ptr(), self.vocab_size, 100, self.window_tokens,
                                                scratch.data_ptr(), scratch.numel(), out.data_ptr(), max_links,
                                                count.data_ptr(), stream), "ts2ts_detect_links")
                n = int(count.item())
                if n <= max_links:
                    break
                max_links = n
        return [tuple(r) for r in out[:n].cpu().tolist()]

    # ------------------------------------------------------------------ protocol
    def detect_links(self, input_ids: torch.Tensor) -> List[LinkInfo]:
        cands = self.candidates(input_ids)
        if not cands:
            return []
        # one gather of the target windows instead of one .item() per token
        lo = min(c[0] for c in cands) + 1
        hi = min(input_ids.shape[0], max(c[0] for c in cands) + 1 + self.window_tokens)
        host = input_ids[lo:hi].cpu().tolist()
        links: List[LinkInfo] = []
        for mid, _start, close in cands:
            chunk = host[mid + 1 - lo:close + 1 - lo]
            decoded = self.decode_fn(chunk)
            idx = decoded.find(")")
            if idx < 0:
                # the per-token table promised a ')' that the joint decoding does not show (not a byte-level
                # vocabulary): fall back to the reference's growing window for this candidate
                idx, found = self._grow(host, mid + 1 - lo, min(mid + 1 + self.window_tokens, input_ids.shape[0]) - lo)
                if idx < 0:
                    continue
                decoded, close = found[0], found[1] + lo
            target = decoded[:idx].strip()
            if target:
                links.append(LinkInfo(link_end_pos=close + 1, target_str=target))
        return links

    def _grow(self, host: List[int], begin: int, end: int):
        chunk: List[int] = []
        for j in range(begin, min(end, len(host))):
            chunk.append(host[j])
            decoded = self.decode_fn(chunk)
            if ")" in decoded:
                return decoded.index(")"), (decoded, j)
        return -1, None
