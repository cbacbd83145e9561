"""The C-ABI library loads without a GPU and exports every symbol the header declares (CPU only, no compute)."""
import ctypes
import os
import re

from tagseq2tagseq_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "ts2ts_attn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ts2ts_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    names = declared_symbols()
    assert len(names) >= 9
    handle = ctypes.CDLL(build.build_library())
    for n in names:
        assert hasattr(handle, n), f"{n} declared in include/ts2ts_attn.h but not exported"
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
