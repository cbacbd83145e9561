"""ts2ts_attn_bwd_noalloc: the backward entry point for callers that cannot allocate device memory.

Some hosts of this library have no way to get scratch memory when they need a backward pass: all of the GPU's
memory already belongs to another allocator, or the calling layer is forbidden to call cudaMalloc because it
synchronises the device.  For them the library carries its own fixed scratch array.  This test drives that entry
point through the C ABI, twice in a row (the array keeps the previous call's contents, so the second call proves
that stale values are cleared), and compares with the ordinary entry point fed a caller-owned workspace:
dk and dv bit for bit, dq within the suite's gradient tolerance (its fp32 reductions arrive in any order).

The file name sorts last on purpose: a run that stops at the first failure has then already run everything else.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

GRAD_TOL = 1e-2  # relative L2, same bound as tests/test_gpu_attention.py


def _bwd_args(q, k, v, out, do, lse, doc, link, plan, dq, dk, dv, scale):
    from tagseq2tagseq_b200 import _lib
    B, H, T, D = q.shape
    s3 = _lib.strides3
    R, W = (0, 0) if link is None else (link.shape[1], link.shape[2])
    return [q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), do.data_ptr(), lse.data_ptr(), s3(q), s3(k), s3(v), s3(out),
            s3(do), B, H, T, D, scale, doc.data_ptr(), None, None, None if link is None else link.data_ptr(), R, W, plan.data_ptr(),
            plan.numel(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), s3(dq), s3(dk), s3(dv)]


@pytest.mark.parametrize("t,h,d,p", [(1500, 4, 128, 0.3), (900, 3, 64, 0.0)])
def test_noalloc_backward_matches_workspace_backward_twice(t, h, d, p):
    from tagseq2tagseq_b200 import _lib, build_block_map, read_status, synth
    from tagseq2tagseq_b200.attention import _attn_fwd
    L = _lib.lib()
    dev = torch.device("cuda")
    stream = torch.cuda.current_stream(dev).cuda_stream
    assert L.ts2ts_attn_bwd_noalloc_max_bytes() == 64 << 20
    scale = d ** -0.5
    for call in range(2):  # two calls in a row, different data and masks, same built-in scratch
        pack = synth.make_pack(70 + call, t, 80, 8, 400, p_link=p)
        doc = torch.from_numpy(pack.doc_ids)[None].to(dev)
        link = None if pack.link_bits is None else torch.from_numpy(pack.link_bits)[None].to(dev)
        plan = build_block_map(doc, link).plan
        g = torch.Generator(device=dev).manual_seed(call)
        q, k, v, do = (torch.randn(1, h, t, d, device=dev, generator=g).bfloat16() for _ in range(4))
        out, lse = _attn_fwd(q, k, v, doc, link, None, None, plan, scale)
        ref = [torch.empty_like(q) for _ in range(3)]
        ws = torch.empty(L.ts2ts_attn_bwd_workspace_bytes(1, h, t, d), dtype=torch.uint8, device=dev)
        code = L.ts2ts_attn_bwd(*_bwd_args(q, k, v, out, do, lse, doc, link, plan, *ref, scale), ws.data_ptr(), ws.numel(), stream)
        assert code == 0, L.ts2ts_last_error_string()
        got = [torch.full_like(q, float("nan")) for _ in range(3)]
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info(dev)[0]
        code = L.ts2ts_attn_bwd_noalloc(*_bwd_args(q, k, v, out, do, lse, doc, link, plan, *got, scale), stream)
        assert code == 0, L.ts2ts_last_error_string()
        torch.cuda.synchronize()
        if call > 0:  # set-up happened in the first call; from then on the entry point must not take device memory
            assert torch.cuda.mem_get_info(dev)[0] == free_before
        assert read_status(plan) == 0
        assert torch.equal(got[1], ref[1]) and torch.equal(got[2], ref[2])
        rel = ((got[0].float() - ref[0].float()).norm() / ref[0].float().norm()).item()
        assert rel <= GRAD_TOL and torch.isfinite(got[0].float()).all()


def test_noalloc_rejects_problems_beyond_the_builtin_scratch():
    from tagseq2tagseq_b200 import _lib
    L = _lib.lib()
    # B=2, H=16, T=32768, D=128 needs ~520 MiB of scratch: refused before anything is launched
    s3 = (ctypes.c_int64 * 3)(16 * 32768 * 128, 32768 * 128, 128)
    code = L.ts2ts_attn_bwd_noalloc(256, 256, 256, 256, 256, 256, s3, s3, s3, s3, s3, 2, 16, 32768, 128, 0.1, 256, None, None, None,
                                    0, 0, 256, 1 << 30, 256, 256, 256, s3, s3, s3, None)
    assert code == -10
    assert b"built-in" in L.ts2ts_last_error_string()
