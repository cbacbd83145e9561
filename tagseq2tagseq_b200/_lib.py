"""ctypes binding of libts2ts_attn.so (declarations: include/ts2ts_attn.h and include/ts2ts_lm.h).

There is no fallback: if the library is missing and cannot be built, importing the
attention entry points raises.  Nothing here computes on the CPU.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_void_p, POINTER

from . import build as _build

_LIB = None

# name -> (restype, argtypes); must list every symbol include/ts2ts_attn.h and include/ts2ts_lm.h declare
SYMBOLS = {
    "ts2ts_version": (c_int, []),
    "ts2ts_last_error_string": (c_char_p, []),
    "ts2ts_plan_bytes": (c_size_t, [c_int, c_int]),
    "ts2ts_block_map": (c_int, [c_void_p] * 4 + [c_int] * 4 + [c_void_p, c_size_t] + [c_void_p] * 9 + [c_void_p]),
    "ts2ts_segment_ids": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "ts2ts_attn_fwd": (c_int, [c_void_p] * 3 + [POINTER(c_int64)] * 3 + [c_int] * 4 + [c_float] + [c_void_p] * 4 + [c_int] * 2
                       + [c_void_p, c_size_t, c_void_p, POINTER(c_int64), c_void_p, c_void_p]),
    "ts2ts_attn_decode_workspace_bytes": (c_size_t, [c_int] * 4),
    "ts2ts_attn_decode": (c_int, [c_void_p] * 3 + [POINTER(c_int64)] * 3 + [c_int] * 4 + [c_float] + [c_void_p] * 4 + [c_int] * 2
                          + [c_void_p, c_void_p, POINTER(c_int64), c_void_p, c_void_p, c_size_t, c_void_p]),
    "ts2ts_attn_bwd_workspace_bytes": (c_size_t, [c_int] * 4),
    "ts2ts_attn_bwd": (c_int, [c_void_p] * 6 + [POINTER(c_int64)] * 5 + [c_int] * 4 + [c_float] + [c_void_p] * 4 + [c_int] * 2
                       + [c_void_p, c_size_t] + [c_void_p] * 3 + [POINTER(c_int64)] * 3 + [c_void_p, c_size_t, c_void_p]),
    "ts2ts_attn_bwd_noalloc_max_bytes": (c_size_t, []),
    "ts2ts_attn_bwd_noalloc": (c_int, [c_void_p] * 6 + [POINTER(c_int64)] * 5 + [c_int] * 4 + [c_float] + [c_void_p] * 4 + [c_int] * 2
                               + [c_void_p, c_size_t] + [c_void_p] * 3 + [POINTER(c_int64)] * 3 + [c_void_p]),
    "ts2ts_detect_links_scratch_bytes": (c_size_t, [c_int]),
    "ts2ts_detect_links": (c_int, [c_void_p, c_int, c_int, c_int64, POINTER(c_int64), c_int, c_void_p, c_int, c_int, c_int,
                                   c_void_p, c_size_t, c_void_p, c_int, c_void_p, c_void_p]),
    "ts2ts_read_status": (c_int, [c_void_p, c_void_p, POINTER(c_int32)]),
    "ts2ts_profile_enable": (c_int, [c_int]),
    "ts2ts_profile_last_ms": (c_int, [c_int, POINTER(c_float)]),
    # include/ts2ts_lm.h
    "ts2ts_add_rmsnorm_fwd": (c_int, [c_void_p] * 6 + [c_int64, c_int, c_float, c_void_p]),
    "ts2ts_add_rmsnorm_bwd_workspace_bytes": (c_size_t, [c_int64, c_int]),
    "ts2ts_add_rmsnorm_bwd": (c_int, [c_void_p] * 9 + [c_size_t, c_int64, c_int, c_void_p]),
    "ts2ts_rope_qk_inplace": (c_int, [c_void_p] * 3 + [c_int] * 4 + [c_float, c_void_p]),
    "ts2ts_swiglu_fwd": (c_int, [c_void_p] * 2 + [c_int64, c_int, c_void_p]),
    "ts2ts_swiglu_bwd": (c_int, [c_void_p] * 3 + [c_int64, c_int, c_void_p]),
    "ts2ts_ce_fwd": (c_int, [c_void_p] * 4 + [c_int64, c_int, c_void_p]),
    "ts2ts_ce_bwd": (c_int, [c_void_p] * 4 + [c_float, c_int64, c_int, c_void_p]),
}


class Ts2tsError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        path = _build.LIB
        if not os.path.exists(path):
            path = _build.build_library()  # raises when nvcc is absent: no CPU path exists
        handle = ctypes.CDLL(path)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _LIB = handle
    return _LIB


def check(code: int, what: str) -> None:
    if code != 0:
        msg = lib().ts2ts_last_error_string().decode()
        if code == -5 or code == -4:
            raise ValueError(f"{what}: {msg}")
        raise Ts2tsError(f"{what} failed with status {code}: {msg}")


def strides3(t) -> "ctypes.Array":
    """Element strides (batch, head, token) of a [B,H,T,D] tensor as int64[3]."""
    return (c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))
