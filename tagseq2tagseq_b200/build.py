"""Builds libts2ts_attn.so (hand-written sm_100a CUDA behind a C ABI) in-tree with nvcc.

    python -m tagseq2tagseq_b200.build [--force]

nvcc cross-compiles without a GPU.  The library links only the static CUDA runtime, so it
also loads on a machine without a driver (the symbol-export test does exactly that).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libts2ts_attn.so")
SELFTEST_LIB = os.path.join(HERE, "libts2ts_selftest.so")  # test-only: the bounded-wait self-test kernel
SOURCES = ["api.cu", "block_map.cu", "link_scan.cu", "attn_fwd.cu", "attn_bwd.cu", "attn_decode.cu", "lm_fused.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "--use_fast_math", "-Xptxas", "-v"]


def _nvcc() -> str:
    path = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(path):
        raise RuntimeError("nvcc not found; the CUDA extension cannot be built")
    return path


def _stale() -> bool:
    if not os.path.exists(LIB) or not os.path.exists(SELFTEST_LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(HERE, "..", "include", h) for h in ("ts2ts_attn.h", "ts2ts_lm.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build_library(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return LIB
    nvcc = _nvcc()
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)

    def compile_one(src):
        obj = os.path.join(objdir, src.replace(".cu", ".o"))
        cmd = [nvcc, *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{res.stdout}\n{res.stderr}")
        return obj, res.stderr

    with ThreadPoolExecutor(max_workers=6) as ex:
        results = list(ex.map(compile_one, SOURCES))
    if verbose:
        for _, log in results:
            print(log)
    cmd = [nvcc, "-shared", "-o", LIB, *[o for o, _ in results], "-cudart", "static"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    cmd = [nvcc, *[f for f in NVCC_FLAGS if f not in ("-Xptxas", "-v")], "-DTS2TS_SPIN_LIMIT=4096u", "-shared",
           os.path.join(CSRC, "selftest_wait.cu"), "-o", SELFTEST_LIB, "-cudart", "static"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"self-test library failed to build:\n{res.stdout}\n{res.stderr}")
    return LIB


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose=True))
