// Masked attention for ONE new query token per sequence against cached K / V (decoding with KV reuse).
//
// The reference has no such path: its generation loop runs the whole forward over all T tokens for every generated
// token and keeps the last row of the logits (model/generation_loop.py:90-92, model/model.py:214-237;
// GENERATION_FEATURE_SPEC.md:163 lists KV caching as not implemented).  With the keys and values of the earlier
// tokens kept, the attention of the new token is one masked row: out = softmax(scale q K^T + mask row) V with
//     allowed(kv) = kv <= q_pos  and  ( doc_ids[q_pos] == doc_ids[kv]  or  bit(link_bits[row(q_pos)], col(kv)) ),
// the same predicate as the training kernels (cross_doc_mask.py:348-357), evaluated per key; no block plan is needed.
//
// HBM-bound work (every allowed key's K and V row is read once, 4 D bytes per key and head), split over the keys:
//   decode_partial_kernel   grid (key tiles of 128, H, B), 128 threads.  A tile none of whose keys is allowed costs
//                           one predicate per key and no K / V traffic.  Otherwise a half-warp reads one 2 D-byte K
//                           row per step (16 bytes per lane), the scores of the tile are softmax-ed locally in base
//                           2, and each thread accumulates its 8 (D = 128) or 4 (D = 64) output columns over the
//                           tile's V rows.  Result per tile: running maximum, sum and unnormalised output row.
//   decode_combine_kernel   grid (H, B), D threads: merges the tiles' partial results and writes out (bf16) and the
//                           natural-log LSE.  A token that may read no key gets out = 0, LSE = -inf.
#include "plan.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>

namespace ts2ts {

struct DecodeParams {
  const __nv_bfloat16 *q, *k, *v;
  int64_t q_sb, q_sh;              // q [B,H,1,D]: batch and head strides (elements)
  int64_t k_sb, k_sh, k_st, v_sb, v_sh, v_st;
  MaskArgs mask;                   // per-token arrays are [B,Tk]
  const int32_t* q_pos;            // [B] position of the query token in the cache, or nullptr = Tk - 1
  float* part;                     // [B,H,NB,2 + D]: m (base-2 exponent), l, o[D]
  __nv_bfloat16* out;              // [B,H,1,D]
  int64_t o_sb, o_sh;
  float* lse;                      // [B,H]
  int B, H, Tk, NB;
  float scale_log2;
};

template <int D>
__global__ void __launch_bounds__(128) decode_partial_kernel(const DecodeParams p) {
  constexpr int kVec = D / 16;  // bf16 elements per lane when 16 lanes share a row: 8 (16 bytes) or 4 (8 bytes)
  const int tile = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qpos = p.q_pos ? min(max(p.q_pos[b], 0), p.Tk - 1) : p.Tk - 1;
  float* part = p.part + (((size_t)b * p.H + h) * p.NB + tile) * (2 + D);
  __shared__ float s_score[kTile];
  __shared__ float s_o[4][D];
  __shared__ float s_red[8];

  // mask row of this tile: thread = key
  const int kv = tile * kTile + tid;
  bool ok = kv <= qpos;
  if (ok) {
    const size_t base = (size_t)b * p.Tk;
    const int qdoc = p.mask.doc[base + qpos];
    ok = p.mask.doc[base + kv] == qdoc;
    if (!ok && p.mask.link != nullptr) {
      const int row = p.mask.row[base + qpos], col = p.mask.col[base + kv];
      if (row >= 0 && row < p.mask.R && col >= 0 && col < 64 * p.mask.W)
        ok = (static_cast<unsigned long long>(p.mask.link[((size_t)b * p.mask.R + row) * p.mask.W + (col >> 6)]) >> (col & 63)) & 1ull;
    }
  }
  if (!__syncthreads_or(ok)) {  // nothing to read in this tile
    if (tid == 0) { part[0] = -CUDART_INF_F; part[1] = 0.f; }
    return;
  }

  // scores: a half-warp per key row, 16 rows per warp and step
  const int sub = lane >> 4, l16 = lane & 15;
  const __nv_bfloat16* qrow = p.q + (size_t)b * p.q_sb + (size_t)h * p.q_sh + l16 * kVec;
  float qf[kVec];
#pragma unroll
  for (int i = 0; i < kVec; ++i) qf[i] = __bfloat162float(qrow[i]);
  const __nv_bfloat16* kbase = p.k + (size_t)b * p.k_sb + (size_t)h * p.k_sh;
#pragma unroll 4
  for (int it = 0; it < 16; ++it) {
    const int r = warp * 32 + it * 2 + sub;  // key row inside the tile
    const int key = tile * kTile + r;
    float acc = 0.f;
    if (key <= qpos) {
      const __nv_bfloat16* krow = kbase + (size_t)key * p.k_st + l16 * kVec;
      if (kVec == 8) {
        const uint4 raw = *reinterpret_cast<const uint4*>(krow);
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(h2[i]);
          acc = fmaf(f.x, qf[2 * i], acc);
          acc = fmaf(f.y, qf[2 * i + 1], acc);
        }
      } else {
        const uint2 raw = *reinterpret_cast<const uint2*>(krow);
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const float2 f = __bfloat1622float2(h2[i]);
          acc = fmaf(f.x, qf[2 * i], acc);
          acc = fmaf(f.y, qf[2 * i + 1], acc);
        }
      }
    }
#pragma unroll
    for (int s = 8; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
    if (l16 == 0) s_score[r] = acc * p.scale_log2;
  }
  __syncthreads();

  // softmax over the tile: thread = key again
  const float sc = ok ? s_score[tid] : -CUDART_INF_F;
  float m = sc;
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, s));
  if (lane == 0) s_red[warp] = m;
  __syncthreads();
  m = fmaxf(fmaxf(s_red[0], s_red[1]), fmaxf(s_red[2], s_red[3]));  // finite: at least one key is allowed
  const float pj = ok ? exp2f(sc - m) : 0.f;
  float l = pj;
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) l += __shfl_xor_sync(0xffffffffu, l, s);
  if (lane == 0) s_red[4 + warp] = l;
  s_score[tid] = pj;  // every thread rewrites only its own entry, which nobody else reads before the barrier
  __syncthreads();
  l = (s_red[4] + s_red[5]) + (s_red[6] + s_red[7]);

  // output: the same half-warp per V row layout; each lane keeps kVec columns
  float of[kVec];
#pragma unroll
  for (int i = 0; i < kVec; ++i) of[i] = 0.f;
  const __nv_bfloat16* vbase = p.v + (size_t)b * p.v_sb + (size_t)h * p.v_sh;
#pragma unroll 4
  for (int it = 0; it < 16; ++it) {
    const int r = warp * 32 + it * 2 + sub;
    const float w = s_score[r];
    if (w != 0.f) {
      const __nv_bfloat16* vrow = vbase + (size_t)(tile * kTile + r) * p.v_st + l16 * kVec;
      if (kVec == 8) {
        const uint4 raw = *reinterpret_cast<const uint4*>(vrow);
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(h2[i]);
          of[2 * i] = fmaf(w, f.x, of[2 * i]);
          of[2 * i + 1] = fmaf(w, f.y, of[2 * i + 1]);
        }
      } else {
        const uint2 raw = *reinterpret_cast<const uint2*>(vrow);
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const float2 f = __bfloat1622float2(h2[i]);
          of[2 * i] = fmaf(w, f.x, of[2 * i]);
          of[2 * i + 1] = fmaf(w, f.y, of[2 * i + 1]);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kVec; ++i) of[i] += __shfl_xor_sync(0xffffffffu, of[i], 16);  // the two half-warps of a warp
  if (sub == 0) {
#pragma unroll
    for (int i = 0; i < kVec; ++i) s_o[warp][l16 * kVec + i] = of[i];
  }
  __syncthreads();
  if (tid < D) part[2 + tid] = (s_o[0][tid] + s_o[1][tid]) + (s_o[2][tid] + s_o[3][tid]);
  if (tid == 0) { part[0] = m; part[1] = l; }
}

template <int D>
__global__ void __launch_bounds__(D) decode_combine_kernel(const DecodeParams p) {
  const int h = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
  const float* part = p.part + ((size_t)b * p.H + h) * p.NB * (2 + D);
  float m = -CUDART_INF_F;
  for (int t = 0; t < p.NB; ++t) m = fmaxf(m, part[(size_t)t * (2 + D)]);
  float l = 0.f, o = 0.f;
  if (m > -CUDART_INF_F) {
    for (int t = 0; t < p.NB; ++t) {
      const float mt = part[(size_t)t * (2 + D)];
      if (mt == -CUDART_INF_F) continue;
      const float w = exp2f(mt - m);
      l = fmaf(w, part[(size_t)t * (2 + D) + 1], l);
      o = fmaf(w, part[(size_t)t * (2 + D) + 2 + d], o);
    }
  }
  p.out[(size_t)b * p.o_sb + (size_t)h * p.o_sh + d] = __float2bfloat16(l > 0.f ? o / l : 0.f);
  if (d == 0) p.lse[(size_t)b * p.H + h] = l > 0.f ? (m + log2f(l)) * 0.6931471805599453f : -CUDART_INF_F;
}

size_t decode_workspace_bytes(int B, int H, int Tk, int D) {
  const size_t nb = (size_t)((Tk + kTile - 1) / kTile);
  return plan_align((size_t)B * H * nb * (2 + D) * sizeof(float));
}

int launch_decode(const void* q, const void* k, const void* v, const int64_t* sq, const int64_t* sk, const int64_t* sv, int B, int H,
                  int Tk, int D, float scale, MaskArgs M, const int32_t* q_pos, void* out, const int64_t* so, float* lse,
                  void* workspace, cudaStream_t stream) {
  DecodeParams p;
  p.q = static_cast<const __nv_bfloat16*>(q); p.k = static_cast<const __nv_bfloat16*>(k); p.v = static_cast<const __nv_bfloat16*>(v);
  p.q_sb = sq[0]; p.q_sh = sq[1];
  p.k_sb = sk[0]; p.k_sh = sk[1]; p.k_st = sk[2];
  p.v_sb = sv[0]; p.v_sh = sv[1]; p.v_st = sv[2];
  p.mask = M; p.q_pos = q_pos;
  p.part = static_cast<float*>(workspace);
  p.out = static_cast<__nv_bfloat16*>(out); p.o_sb = so[0]; p.o_sh = so[1];
  p.lse = lse;
  p.B = B; p.H = H; p.Tk = Tk; p.NB = (Tk + kTile - 1) / kTile;
  p.scale_log2 = scale * 1.4426950408889634f;
  const dim3 grid(p.NB, H, B);
  if (D == 128) {
    decode_partial_kernel<128><<<grid, 128, 0, stream>>>(p);
    decode_combine_kernel<128><<<dim3(H, B), 128, 0, stream>>>(p);
  } else if (D == 64) {
    decode_partial_kernel<64><<<grid, 128, 0, stream>>>(p);
    decode_combine_kernel<64><<<dim3(H, B), 64, 0, stream>>>(p);
  } else {
    return -142;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -141;
}

}  // namespace ts2ts
