/* libts2ts_attn -- C ABI of the memory-bound pieces of the decoder layer that surround the attention call in
 * the training step (same library, same conventions as ts2ts_attn.h: device pointers, `stream` a cudaStream_t
 * passed as void*, 0 = OK, < 0 = rejected arguments or launch failure, no device memory allocated here).
 *
 * They stand where the reference's training step uses fused modules of its own:
 *   - RMSNorm before attention and MLP, residual adds around them (model/modules/layer.py:20-35),
 *   - rotary position embedding inside the attention module (model/modules/layer.py:33, rope_base in
 *     model/modules/backbone.py),
 *   - the SwiGLU MLP (model/modules/layer.py:26),
 *   - the fused output head + cross-entropy loss (model/modules/training_module.py:205).
 * All arithmetic is fp32; activations are bf16 in memory, the residual stream and the norm weights fp32.
 * Row-major, contiguous tensors; every row starts on a 16-byte boundary (C % 4 == 0, F % 8 == 0, V % 8 == 0,
 * D % 16 == 0).
 */
#ifndef TS2TS_LM_H_
#define TS2TS_LM_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* x_out[N,C] (fp32) = x_in[N,C] (fp32) + a[N,C] (bf16, may be NULL);  h[N,C] (bf16) = x_out * rstd * w[C] (fp32),
 * rstd[N] (fp32) = 1 / sqrt(mean(x_out^2) + eps).  x_out may alias x_in.  4 <= C <= 16384. */
int ts2ts_add_rmsnorm_fwd(const float* x_in, const void* a, const float* w, float* x_out, void* h, float* rstd, int64_t N, int C,
                          float eps, void* stream);

/* Gradient of ts2ts_add_rmsnorm_fwd.  dh[N,C] bf16 = gradient of h, dx_up[N,C] fp32 = gradient that reaches x_out
 * from its other users (may be NULL), x / w / rstd as saved by the forward.  Writes dx[N,C] fp32, the gradient of
 * x_in (and of a), its bf16 copy da[N,C] when da != NULL, and ADDS the weight gradient into dw[C] (fp32, zeroed by
 * the caller).  `workspace` (16-byte aligned, ts2ts_add_rmsnorm_bwd_workspace_bytes(N, C) bytes) holds the blocks'
 * partial weight gradients. */
size_t ts2ts_add_rmsnorm_bwd_workspace_bytes(int64_t N, int C);
int ts2ts_add_rmsnorm_bwd(const void* dh, const float* dx_up, const float* x, const float* w, const float* rstd, float* dx, void* da,
                          float* dw, void* workspace, size_t workspace_bytes, int64_t N, int C, void* stream);

/* Rotary embedding in place on the q and k slices of qkv[B,T,3,H,D] (bf16): pairs (i, i + D/2) are rotated by the
 * angle whose cosine / sine are cos[t,i], sin[t,i] (fp32 [T, D/2]).  sign = +1 rotates, sign = -1 rotates back, which
 * is also what turns the gradient of the rotated tensor into the gradient of the input. */
int ts2ts_rope_qk_inplace(void* qkv, const float* cos, const float* sin, int B, int T, int H, int D, float sign, void* stream);

/* act[N,F] = silu(gu[N, 0:F]) * gu[N, F:2F]  (bf16). */
int ts2ts_swiglu_fwd(const void* gu, void* act, int64_t N, int F, void* stream);
/* dgu[N,2F] from gu and dact[N,F]  (bf16). */
int ts2ts_swiglu_bwd(const void* gu, const void* dact, void* dgu, int64_t N, int F, void* stream);

/* Cross-entropy of logits[N,V] (bf16) against target[N] (int64): lse[N] = log-sum-exp of the row, loss[N] =
 * lse - logits[target] (both fp32; a target outside 0..V-1 gives loss 0 and, below, a zero gradient). */
int ts2ts_ce_fwd(const void* logits, const int64_t* target, float* lse, float* loss, int64_t N, int V, void* stream);
/* Overwrites logits with the gradient of  gscale[0] * inv_n * sum(loss):  (softmax - onehot) * gscale[0] * inv_n.
 * gscale is a device scalar (the incoming gradient of the mean loss), so no host synchronisation is needed. */
int ts2ts_ce_bwd(void* logits, const int64_t* target, const float* lse, const float* gscale, float inv_n, int64_t N, int V,
                 void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TS2TS_LM_H_ */
