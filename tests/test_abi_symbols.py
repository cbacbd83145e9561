"""The C-ABI library loads without a GPU and exports every symbol the header declares (CPU only, no compute)."""
import ctypes
import os
import re

from tagseq2tagseq_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    for header in ("ts2ts_attn.h", "ts2ts_lm.h"):
        text = open(os.path.join(ROOT, "include", header)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b(ts2ts_\w+)\s*\(", text))
    return sorted(names)


def test_every_declared_symbol_is_exported_and_bound():
    names = declared_symbols()
    assert len(names) >= 9
    handle = ctypes.CDLL(build.build_library())
    for n in names:
        assert hasattr(handle, n), f"{n} declared in include/ but not exported"
    assert sorted(_lib.SYMBOLS) == names


def test_size_queries_and_argument_rejection_need_no_gpu():
    L = _lib.lib()
    assert L.ts2ts_version() >= 1000
    assert L.ts2ts_plan_bytes(0, 128) == 0 and L.ts2ts_plan_bytes(1, 0) == 0
    nb = 256
    assert L.ts2ts_plan_bytes(2, 32768) >= 2 * nb * nb * (1 + 4 + 4) + 2 * nb * 128 * 16
    assert L.ts2ts_attn_bwd_workspace_bytes(1, 1, 128, 96) == 0
    assert L.ts2ts_attn_bwd_workspace_bytes(2, 16, 32768, 128) >= 2 * 16 * 32768 * (128 * 4 + 8)
    # rejected before any CUDA call: bad sizes, null doc ids, short plan
    assert L.ts2ts_block_map(None, None, None, None, 0, 128, 0, 0, None, 0, *([None] * 9), None) < 0
    assert b"positive" in L.ts2ts_last_error_string()
    assert L.ts2ts_block_map(None, None, None, None, 1, 128, 0, 0, None, 0, *([None] * 9), None) < 0
    assert b"doc_ids" in L.ts2ts_last_error_string()
    s3 = (ctypes.c_int64 * 3)(128, 128, 128)
    assert L.ts2ts_attn_fwd(16, 16, 16, s3, s3, s3, 1, 1, 128, 96, 0.1, 16, None, None, None, 0, 0, 256, 1 << 20, 16, s3, 16, None) == -2
    bad = (ctypes.c_int64 * 3)(128, 128, 3)
    assert L.ts2ts_attn_fwd(16, 16, 16, bad, s3, s3, 1, 1, 128, 128, 0.1, 16, None, None, None, 0, 0, 256, 1 << 20, 16, s3, 16, None) == -5


def test_link_scan_argument_rejection_needs_no_gpu():
    L = _lib.lib()
    assert L.ts2ts_detect_links_scratch_bytes(0) == 0
    assert L.ts2ts_detect_links_scratch_bytes(1000) >= 8000
    starts = (ctypes.c_int64 * 2)(58, 685)
    ok_args = dict(tokens=16, tb=8, T=128, mid=16151, starts=starts, ns=2, flags=16, vocab=50257, back=100, win=50, scratch=16,
                   sbytes=1 << 20, links=16, maxl=8, count=16)

    def call(**kw):
        a = {**ok_args, **kw}
        return L.ts2ts_detect_links(a["tokens"], a["tb"], a["T"], a["mid"], a["starts"], a["ns"], a["flags"], a["vocab"], a["back"],
                                    a["win"], a["scratch"], a["sbytes"], a["links"], a["maxl"], a["count"], None)

    assert call(T=0) == -1
    assert call(tb=2) == -2
    assert call(tokens=None) == -3
    assert call(ns=0) == -6 and call(ns=9) == -6
    assert call(flags=None) == -6 and call(win=-1) == -6
    assert call(sbytes=16) == -9
    assert call(links=None) == -3


def test_decoder_layer_entry_points_reject_bad_arguments_without_a_gpu():
    L = _lib.lib()
    assert L.ts2ts_add_rmsnorm_bwd_workspace_bytes(0, 768) == 0 and L.ts2ts_add_rmsnorm_bwd_workspace_bytes(16, 6) == 0
    ws = L.ts2ts_add_rmsnorm_bwd_workspace_bytes(16384, 768)
    assert ws % (768 * 4) == 0 and 0 < ws <= 16384 * 768 * 4
    assert L.ts2ts_add_rmsnorm_bwd_workspace_bytes(3, 768) == 3 * 768 * 4          # never more partial rows than rows
    assert L.ts2ts_add_rmsnorm_fwd(16, None, 16, 16, 16, 16, 0, 768, 1e-6, None) == -1
    assert L.ts2ts_add_rmsnorm_fwd(16, None, 16, 16, 16, 16, 8, 770, 1e-6, None) == -2
    assert L.ts2ts_add_rmsnorm_fwd(None, None, 16, 16, 16, 16, 8, 768, 1e-6, None) == -3
    assert L.ts2ts_add_rmsnorm_fwd(20, None, 16, 16, 16, 16, 8, 768, 1e-6, None) == -5
    assert L.ts2ts_add_rmsnorm_bwd(16, None, 16, 16, 16, 16, None, 16, 16, 8, 16384, 768, None) == -4
    assert b"workspace" in L.ts2ts_last_error_string()
    assert L.ts2ts_rope_qk_inplace(16, 16, 16, 1, 128, 2, 40, 1.0, None) == -2
    assert L.ts2ts_rope_qk_inplace(16, 16, 16, 1, 128, 2, 64, 0.5, None) == -8
    assert L.ts2ts_swiglu_fwd(16, 16, 8, 12, None) == -2
    assert L.ts2ts_swiglu_bwd(16, None, 16, 8, 16, None) == -3
    assert L.ts2ts_ce_fwd(16, 16, 16, 16, 8, 50300, None) == -2
    assert L.ts2ts_ce_bwd(18, 16, 16, 16, 0.5, 8, 512, None) == -5
