"""Synthetic byte-level vocabulary for the link-scan tests (the GPT-2 BPE tables need a download).

Ids 0..255 are the single bytes; the ids after that are multi-byte tokens, among them the link delimiters,
tokens that hide a ')' behind other characters, UTF-8 sequences split across tokens and whitespace of every kind.
``decode`` joins the bytes and decodes them the way tiktoken does (invalid sequences become U+FFFD).
"""
from __future__ import annotations

import random
from typing import List

EXTRA = [b"](", b"[", b" [", b")", b").", b"s)", b" )", b" (", b"(", b" the", b"Foo", b"Bar", b" baz", b"_", b"Page", b" Title",
         b"\xc3\xa9", b"\xc3", b"\xa9", b"\xc2\xa0", b"\xc2", b"\xa0", b"\xe3\x80\x80", b"\xe3\x80", b"\x80", b"  ", b"\n", b"\t ",
         b"]", b"](x", b"x](", b" [[", b"wiki", b"/", b"#", b"%20", b"1", b"22", b" and", b",", b".", b"()", b")(", b"a)b"]
VOCAB: List[bytes] = [bytes([i]) for i in range(256)] + EXTRA
MID = 256            # b"]("
STARTS = [257, 258]  # b"[", b" ["
CLOSERS = [i for i, t in enumerate(VOCAB) if b")" in t]
PLAIN = [i for i, t in enumerate(VOCAB) if i >= 256 and b")" not in t and i not in (MID, 257, 258)]


def decode(ids: List[int]) -> str:
    return b"".join(VOCAB[i] for i in ids).decode("utf-8", errors="replace")


def random_stream(rng: random.Random, T: int, window: int) -> List[int]:
    """Token stream with planted links of every kind: well-formed, without an opening bracket in reach, with the
    closing token just inside / just outside the window, with empty or whitespace-only targets, cut by the end."""
    toks: List[int] = []
    filler = PLAIN + list(range(97, 123)) + [32, 10]
    while len(toks) < T:
        kind = rng.random()
        if kind < 0.55:
            toks.extend(rng.choice(filler) for _ in range(rng.randint(1, 30)))
        else:
            far = rng.random() < 0.15
            if rng.random() < 0.85:
                toks.append(rng.choice(STARTS))
            n_text = rng.choice([0, 1, 3, 8, 99, 100, 101, 140]) if far else rng.randint(0, 12)
            toks.extend(rng.choice(filler) for _ in range(n_text))
            toks.append(MID)
            shape = rng.random()
            if shape < 0.1:
                n_target = 0
            elif shape < 0.25:
                n_target = rng.choice([window - 2, window - 1, window, window + 1])
            else:
                n_target = rng.randint(1, 9)
            blank = rng.random() < 0.12
            pool = [32, 10, 9, VOCAB.index(b"  "), VOCAB.index(b"\xc2"), VOCAB.index(b"\xa0"), VOCAB.index(b"\xc2\xa0")] if blank else filler
            toks.extend(rng.choice(pool) for _ in range(max(0, n_target)))
            if rng.random() < 0.9:
                toks.append(rng.choice(CLOSERS))
    return toks[:T]
