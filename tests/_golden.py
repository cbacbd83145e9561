"""Loading helpers for the fixtures under tests/golden/ (made by tests/golden/make_golden.py)."""
import json
import os
from types import SimpleNamespace

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def spans_of(entry):
    return [SimpleNamespace(doc_id=d, start=a, end=b, raw_identifier=f"doc_{d}") for d, a, b in entry["spans"]]


def links_of(entry):
    return {int(k): list(v) for k, v in entry["links"].items()}


def unpack(bits, shape):
    n = int(np.prod(shape))
    return np.unpackbits(bits)[:n].reshape(shape).astype(bool)


def grant_cases():
    with open(os.path.join(GOLDEN, "grants.json")) as f:
        return json.load(f)


def grant_arrays():
    return np.load(os.path.join(GOLDEN, "grants.npz"))


def blockmap_cases():
    with open(os.path.join(GOLDEN, "blockmaps.json")) as f:
        return json.load(f)


def blockmap_arrays():
    return np.load(os.path.join(GOLDEN, "blockmaps.npz"))


def flex_arrays():
    return np.load(os.path.join(GOLDEN, "flex_fwd.npz"))


def blockmask_to_states(arrs, prefix, qb_n):
    """Rebuild the 0/1/2 state map from BlockMask kv lists (only the first num entries count)."""
    st = np.zeros((qb_n, qb_n), dtype=np.uint8)
    for r in range(qb_n):
        for c in arrs[f"{prefix}/kv_indices"][r][: arrs[f"{prefix}/kv_num_blocks"][r]]:
            st[r, c] = 1
        for c in arrs[f"{prefix}/full_kv_indices"][r][: arrs[f"{prefix}/full_kv_num_blocks"][r]]:
            st[r, c] = 2
    return st
