"""Seeded synthetic packs: document lengths and a link DAG with the shapes of the reference's packed batches.

The reference trains on packs of tens to hundreds of documents drawn from its graph datasets
(data/pack_sampler.py, configs/stack_100m_32k.yaml:38), which are not available offline; this generator
stands in for them.  Lengths are floor(exp(N(ln median, sigma))) clipped to [lo, hi], with an optional
heavy tail (a fraction of documents drawn uniformly from [heavy_lo, heavy_hi]); documents are appended
until T tokens are filled and the last one is truncated.  Each document links to each earlier document
independently with probability p (whole-document grants).  numpy's PCG64 `default_rng(seed)` drives everything.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import numpy as np


@dataclass
class Pack:
    lengths: np.ndarray        # int64[n_docs]
    doc_ids: np.ndarray        # int32[T], local document index
    link_bits: Optional[np.ndarray]  # int64[n_docs, W] bit b of row a: doc a reads doc b; None for doc_causal
    links: List[tuple]         # (a, b) pairs

    @property
    def seq_len(self) -> int:
        return int(self.doc_ids.shape[0])

    def unmasked_pairs(self) -> int:
        """Exact number of allowed (q, kv) pairs: sum L(L+1)/2 + sum over links L_a * L_b."""
        L = self.lengths.astype(np.int64)
        n = int((L * (L + 1) // 2).sum())
        for a, b in self.links:
            n += int(L[a] * L[b])
        return n


def make_pack(seed: int, T: int, median: float, lo: int, hi: int, sigma: float = 1.0, p_link: float = 0.0,
              heavy_frac: float = 0.0, heavy_lo: int = 0, heavy_hi: int = 0) -> Pack:
    rng = np.random.default_rng(seed)
    lengths, total = [], 0
    while total < T:
        if heavy_frac > 0.0 and rng.random() < heavy_frac:
            n = int(rng.integers(heavy_lo, heavy_hi + 1))
        else:
            n = int(np.floor(np.exp(rng.normal(np.log(median), sigma))))
            n = max(lo, min(hi, n))
        n = min(n, T - total)
        lengths.append(n)
        total += n
    lengths = np.asarray(lengths, dtype=np.int64)
    n_docs = lengths.size
    doc_ids = np.repeat(np.arange(n_docs, dtype=np.int32), lengths)
    links, link_bits = [], None
    if p_link > 0.0:
        W = (n_docs + 63) // 64
        bits = np.zeros((n_docs, W), dtype=np.uint64)
        draw = rng.random((n_docs, n_docs)) < p_link
        for a in range(n_docs):
            for b in range(a):
                if draw[a, b]:
                    bits[a, b >> 6] |= np.uint64(1) << np.uint64(b & 63)
                    links.append((a, b))
        link_bits = bits.view(np.int64)
    return Pack(lengths=lengths, doc_ids=doc_ids, link_bits=link_bits, links=links)


# The workloads named by the benchmark configurations (sigma fixed at 1.0).
def config1_pack(seed: int = 1001) -> Pack:
    return make_pack(seed, 2048, 128, 16, 512)


def config2_pack(seed: int = 1002) -> Pack:
    return make_pack(seed, 16384, 200, 32, 2048, p_link=0.15)


def config3_pack(seed: int, mask: str) -> Pack:
    p = {"doc_causal": 0.0, "link_p05": 0.05, "link_p30": 0.3}[mask]
    return make_pack(seed, 32768, 150, 16, 4096, p_link=p, heavy_frac=0.05, heavy_lo=4096, heavy_hi=8192)


def config5_pack(seed: int = 1005) -> Pack:
    return make_pack(seed, 32768, 200, 32, 2048, p_link=0.3)


def stack_packs(packs: List[Pack]):
    """Batch packs of equal T: doc_ids int32[B,T], link_bits int64[B,R,W] (zero padded) or None."""
    doc_ids = np.stack([p.doc_ids for p in packs])
    if all(p.link_bits is None for p in packs):
        return doc_ids, None
    R = max(p.lengths.size for p in packs)
    W = (R + 63) // 64
    bits = np.zeros((len(packs), R, W), dtype=np.int64)
    for i, p in enumerate(packs):
        if p.link_bits is not None:
            bits[i, : p.link_bits.shape[0], : p.link_bits.shape[1]] = p.link_bits
    return doc_ids, bits
