"""CPU restatement of the markdown link scan (test infrastructure only; never imported by the product).

Follows ``MarkdownLinkDetector.detect_links`` (model/graph_traversal/markdown_link_detector.py:57-108) step by
step with plain Python loops over a list of token ids:

* candidates are the positions of ``link_mid_token_id`` in ascending order (``:69-71``);
* the opening bracket is the first of ``link_start_token_ids`` met walking back from ``mid - 1`` to
  ``max(0, mid - 100)`` inclusive (``:74-79``); without one the candidate is dropped (``:81-82``);
* the window ``tokens[mid+1 : min(mid+1+window, T)]`` is decoded token by token, growing, until the decoded text
  contains ')' (``:88-99``); the target is the stripped text before the first ')' and must be non-empty;
  an empty target ends the candidate without a link;
* a link is ``(link_end_pos = closing position + 1, target_str)`` (``:101-102``).

``candidates`` returns the integer part alone -- ``(mid, start, close)`` triples, what the CUDA scan produces --
and ``detect_links`` the full result.  Pinned against the reference run on seeded synthetic token streams
(tests/golden/links.json).
"""
from __future__ import annotations

from typing import Callable, Iterable, List, Sequence, Tuple


def candidates(tokens: Sequence[int], decode_fn: Callable[[List[int]], str], mid_id: int = 16151,
               start_ids: Iterable[int] = (58, 685), window: int = 50, back_limit: int = 100) -> List[Tuple[int, int, int]]:
    start_ids = set(start_ids)
    T = len(tokens)
    out = []
    for mid in range(T):
        if tokens[mid] != mid_id:
            continue
        start = None
        for i in range(mid - 1, max(-1, mid - back_limit - 1), -1):
            if tokens[i] in start_ids:
                start = i
                break
        if start is None:
            continue
        chunk: List[int] = []
        for j in range(mid + 1, min(mid + 1 + window, T)):
            chunk.append(tokens[j])
            if ")" in decode_fn(chunk):
                out.append((mid, start, j))
                break
    return out


def detect_links(tokens: Sequence[int], decode_fn: Callable[[List[int]], str], mid_id: int = 16151,
                 start_ids: Iterable[int] = (58, 685), window: int = 50) -> List[Tuple[int, str]]:
    links = []
    for mid, _start, close in candidates(tokens, decode_fn, mid_id, start_ids, window):
        decoded = decode_fn(list(tokens[mid + 1:close + 1]))
        target = decoded[:decoded.index(")")].strip()
        if target:
            links.append((close + 1, target))
    return links
