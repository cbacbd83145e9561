// Masked flash-attention backward for sm_100a.
//
// Three kernels:
//   bwd_prep     delta[q] = sum_d O[q,d] dO[q,d],  lse2[q] = LSE[q] * log2(e)   (fp32, padded to whole tiles)
//   attn_bwd     one CTA per 128-key tile of one (batch, head); walks the non-skipped query tiles of the
//                transposed block list.  Per query tile, with everything transposed so that a thread owns a key row:
//                  tcgen05  S^T = K Q^T,  dP^T = V dO^T                      (fp32 in tensor memory)
//                  4 warps  P^T = exp2(scale S^T - lse2[q]) under the mask,  dS^T = P^T (dP^T - delta[q]);
//                           both written as bf16 over the S^T / dP^T columns, dS^T also to shared memory
//                  tcgen05  dV += P^T dO,  dK += dS^T Q   (A operand from tensor memory, B MN-major from smem)
//                           dQ  = dS K                    (A = dS^T tile read MN-major, B = K MN-major)
//                  4 warps  dQ tile -> fp32 red.global.add into the dQ accumulator
//                dK (scaled) and dV leave through shared memory and TMA stores at the end.
//   dq_convert   dQ accumulator (fp32, already scaled) -> bf16 dq
//
// Computes what the reference gets from autograd of PyTorch FlexAttention
// (torch/_higher_order_ops/flex_attention.py:947-1075): P = exp(S - LSE), dV = P^T dO, dP = dO V^T,
// dS = P (dP - delta), dQ = scale dS K, dK = scale dS^T Q.  Rows whose LSE is -inf get zero gradients.
#include "plan.h"
#include "profile.h"
#include "ptx.cuh"
#include "tma_host.h"

#include <math_constants.h>

namespace ts2ts {

struct BwdParams {
  PlanView plan;
  MaskArgs mask;
  const float* lse2;     // [B,H,Tp]
  const float* delta;    // [B,H,Tp]
  float* dq_acc;         // [B,H,Tp,D]
  __nv_bfloat16* dk;     // for the empty-list path only
  __nv_bfloat16* dv;
  int64_t dk_s[3], dv_s[3];
  int H, Tp;
  float scale, scale_log2;
};

constexpr int kBwdThreads = 192;

template <int D>
struct BwdSmem {
  static constexpr int kSub = D / 64;
  static constexpr int kTileBytes = kTile * D * 2;
  static constexpr int kDsBytes = kTile * kTile * 2;
  static constexpr int kBytes = 4 * kTileBytes + kDsBytes + 1024;
  // tensor-memory columns
  static constexpr int kDV = 0, kDK = D, kST = 2 * D, kDPT = 2 * D + 128;
};

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// 128-bit mask of the query rows of tile `qb` that may read key (doc, column class), before causality.
__device__ __forceinline__ void allowed_rows(const PlanView& P, const MaskArgs& M, int b, int qb, int kvdoc, int kvcol,
                                             uint32_t (&bits)[4]) {
  bits[0] = bits[1] = bits[2] = bits[3] = 0u;
  const int n = P.run_cnt[(size_t)b * P.NB + qb];
  const Run* runs = P.runs + ((size_t)b * P.NB + qb) * kTile;
  const int n_valid = min(kTile, P.T - qb * kTile);
  const bool col_ok = M.link != nullptr && kvcol >= 0 && kvcol < 64 * M.W;
  const int64_t* link_b = col_ok ? M.link + (size_t)b * M.R * M.W + (kvcol >> 6) : nullptr;
  for (int r = 0; r < n; ++r) {
    const int4 raw = __ldg(reinterpret_cast<const int4*>(runs + r));
    const int start = raw.x, doc = raw.y, row = raw.z;
    const int end = (r + 1 < n) ? __ldg(&runs[r + 1].start) : n_valid;
    bool ok = doc == kvdoc;
    if (!ok && col_ok && row >= 0 && row < M.R)
      ok = (static_cast<unsigned long long>(__ldg(link_b + (size_t)row * M.W)) >> (kvcol & 63)) & 1ull;
    if (ok) {
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const int lo = max(start - 32 * w, 0), hi = min(end - 32 * w, 32);
        if (hi > lo) bits[w] |= (hi - lo == 32 ? 0xffffffffu : ((1u << (hi - lo)) - 1u)) << lo;
      }
    }
  }
}

template <int D>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapDO,
                const __grid_constant__ CUtensorMap mapDK, const __grid_constant__ CUtensorMap mapDV, const BwdParams p) {
  using Cfg = BwdSmem<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = smem + Cfg::kTileBytes;
  uint8_t* sQ = smem + 2 * Cfg::kTileBytes;
  uint8_t* sDO = smem + 3 * Cfg::kTileBytes;
  uint8_t* sDS = smem + 4 * Cfg::kTileBytes;
  __shared__ uint64_t bar_kv, bar_qdo, bar_st, bar_pds, bar_g, bar_dqr, bar_epi;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_word;
  __shared__ __align__(16) float s_lse2[kTile];
  __shared__ __align__(16) float s_delta[kTile];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const PlanView& P = p.plan;
  const int NB = P.NB;
  const int rank = blockIdx.x % NB;
  const int bh = blockIdx.x / NB;
  const int h = bh % p.H, b = bh / p.H;
  const int kb = P.bwd_order[(size_t)b * NB + rank];
  const int n = P.bwd_cnt[(size_t)b * NB + kb];
  const int32_t* list = P.bwd_idx + ((size_t)b * NB + kb) * NB;

  if (n == 0) {
    if (tid < kTile) {
      const int kv = kb * kTile + tid;
      if (kv < P.T) {
        __nv_bfloat16* a = p.dk + (size_t)b * p.dk_s[0] + (size_t)h * p.dk_s[1] + (size_t)kv * p.dk_s[2];
        __nv_bfloat16* c = p.dv + (size_t)b * p.dv_s[0] + (size_t)h * p.dv_s[1] + (size_t)kv * p.dv_s[2];
        for (int i = 0; i < D; i += 8) {
          *reinterpret_cast<uint4*>(a + i) = make_uint4(0, 0, 0, 0);
          *reinterpret_cast<uint4*>(c + i) = make_uint4(0, 0, 0, 0);
        }
      }
    }
    return;
  }

  if (tid == 0) {
    abort_word = 0;
    mbar_init(&bar_kv, 1);
    mbar_init(&bar_qdo, 1);
    mbar_init(&bar_st, 1);
    mbar_init(&bar_pds, kTile);
    mbar_init(&bar_g, 1);
    mbar_init(&bar_dqr, kTile);
    mbar_init(&bar_epi, kTile);
    fence_mbar_init();
  }
  __syncthreads();
  if (warp == 5) {
    tmem_alloc(&tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  const uint32_t tDV = tmem + Cfg::kDV, tDK = tmem + Cfg::kDK, tST = tmem + Cfg::kST, tDPT = tmem + Cfg::kDPT;
  // dQ (128 q rows x D) is produced in 64-column parts into the halves of the S^T / dP^T regions that the
  // bf16 overlays leave free.
  const uint32_t tDQ0 = tST + 64, tDQ1 = tDPT + 64;

  if (warp == 4) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&mapQ); tma_prefetch_desc(&mapK); tma_prefetch_desc(&mapV); tma_prefetch_desc(&mapDO);
      mbar_expect_tx(&bar_kv, 2 * Cfg::kTileBytes);
      for (int s = 0; s < Cfg::kSub; ++s) {
        tma_load_4d(sK + s * 16384, &mapK, &bar_kv, s * 64, kb * kTile, h, b);
        tma_load_4d(sV + s * 16384, &mapV, &bar_kv, s * 64, kb * kTile, h, b);
      }
      for (int i = 0; i < n; ++i) {
        const int qb = list[i] & ~kFullBit;
        if (i > 0 && !mbar_wait(&bar_g, (i - 1) & 1, &abort_word, 11)) break;  // Q / dO of the previous tile consumed
        mbar_expect_tx(&bar_qdo, 2 * Cfg::kTileBytes + 2 * kTile * 4);
        for (int s = 0; s < Cfg::kSub; ++s) {
          tma_load_4d(sQ + s * 16384, &mapQ, &bar_qdo, s * 64, qb * kTile, h, b);
          tma_load_4d(sDO + s * 16384, &mapDO, &bar_qdo, s * 64, qb * kTile, h, b);
        }
        const size_t stat = ((size_t)b * p.H + h) * p.Tp + (size_t)qb * kTile;
        bulk_load(s_lse2, p.lse2 + stat, kTile * 4, &bar_qdo);
        bulk_load(s_delta, p.delta + stat, kTile * 4, &bar_qdo);
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_st = make_idesc_bf16(128, 128, false, false);   // K-major x K-major
      constexpr uint32_t idesc_g = make_idesc_bf16(128, D, false, true);       // TMEM A x MN-major B
      constexpr uint32_t idesc_dq = make_idesc_bf16(128, 64, true, true);      // MN-major A x MN-major B
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aQ = smem_u32(sQ), aDO = smem_u32(sDO), aDS = smem_u32(sDS);
      bool ok = mbar_wait(&bar_kv, 0, &abort_word, 21);
      for (int i = 0; i < n && ok; ++i) {
        if (!mbar_wait(&bar_qdo, i & 1, &abort_word, 22)) break;
        if (i > 0 && !mbar_wait(&bar_dqr, (i - 1) & 1, &abort_word, 23)) break;  // S^T / dP^T columns free again
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          mma_ss(tST, make_smem_desc(aK + off, 16, 1024), make_smem_desc(aQ + off, 16, 1024), idesc_st, kk > 0);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          mma_ss(tDPT, make_smem_desc(aV + off, 16, 1024), make_smem_desc(aDO + off, 16, 1024), idesc_st, kk > 0);
        }
        mma_commit(&bar_st);
        if (!mbar_wait(&bar_pds, i & 1, &abort_word, 24)) break;
        tc_fence_after();
        const uint32_t acc = i > 0 ? 1u : 0u;
#pragma unroll
        for (int kk = 0; kk < kTile / 16; ++kk)   // dV += P^T dO      (K = query index)
          mma_ts(tDV, tST + kk * 8, make_smem_desc(aDO + kk * 2048, 16384, 1024), idesc_g, acc | (kk > 0));
#pragma unroll
        for (int kk = 0; kk < kTile / 16; ++kk)   // dK += dS^T Q
          mma_ts(tDK, tDPT + kk * 8, make_smem_desc(aQ + kk * 2048, 16384, 1024), idesc_g, acc | (kk > 0));
#pragma unroll
        for (int part = 0; part < Cfg::kSub; ++part) {  // dQ[:, 64 part ..] = dS K[:, 64 part ..]   (K = key index)
          const uint32_t td = part == 0 ? tDQ0 : tDQ1;
#pragma unroll
          for (int kk = 0; kk < kTile / 16; ++kk)
            mma_ss(td, make_smem_desc(aDS + kk * 2048, 16384, 1024), make_smem_desc(aK + part * 16384 + kk * 2048, 16384, 1024),
                   idesc_dq, kk > 0);
        }
        mma_commit(&bar_g);
      }
    }
  } else {
    // ------------------------------------------------------------------ compute warps
    const int kv = kb * kTile + tid;
    const bool kv_valid = kv < P.T;
    const int kvdoc = kv_valid ? p.mask.doc[(size_t)b * P.T + kv] : INT32_MIN;
    const int kvcol = kv_valid ? p.mask.col[(size_t)b * P.T + kv] : -1;
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    const size_t row_base = ((size_t)b * p.H + h) * p.Tp;
    bool ok = true;
    for (int i = 0; i < n; ++i) {
      const int entry = list[i];
      const int qb = entry & ~kFullBit;
      const bool is_full = (entry & kFullBit) != 0;
      uint32_t bits[4] = {0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu};
      if (!is_full) {
        allowed_rows(P, p.mask, b, qb, kvdoc, kvcol, bits);
        if (!kv_valid) bits[0] = bits[1] = bits[2] = bits[3] = 0u;
        if (kb == qb) {  // causal inside the diagonal tile: query rows tid..127
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            const int lo = tid - 32 * w;
            bits[w] &= lo <= 0 ? 0xffffffffu : (lo >= 32 ? 0u : ~((1u << lo) - 1u));
          }
        }
      }
      // S^T done implies Q, dO, lse2 and delta of this tile have landed (the MMA warp waited for them)
      if (!(ok = mbar_wait(&bar_qdo, i & 1, &abort_word, 30))) break;
      if (!(ok = mbar_wait(&bar_st, i & 1, &abort_word, 31))) break;
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t s[32], dp[32];
        tmem_ld32(tST + lane_base + c * 32, s);
        tmem_ld32(tDPT + lane_base + c * 32, dp);
        tmem_ld_wait();
        const uint32_t bw = bits[c];
        uint32_t pk[16], dsk[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          const int q0 = c * 32 + e;
          float p0 = fast_exp2(fmaf(__uint_as_float(s[e]), p.scale_log2, -s_lse2[q0]));
          float p1 = fast_exp2(fmaf(__uint_as_float(s[e + 1]), p.scale_log2, -s_lse2[q0 + 1]));
          p0 = ((bw >> e) & 1u) ? p0 : 0.f;
          p1 = ((bw >> (e + 1)) & 1u) ? p1 : 0.f;
          const float d0 = p0 * (__uint_as_float(dp[e]) - s_delta[q0]);
          const float d1 = p1 * (__uint_as_float(dp[e + 1]) - s_delta[q0 + 1]);
          pk[e >> 1] = pack_bf16(p0, p1);
          dsk[e >> 1] = pack_bf16(d0, d1);
        }
        tmem_st16(tST + lane_base + c * 16, pk);
        tmem_st16(tDPT + lane_base + c * 16, dsk);
        // dS^T row `tid`, query columns [32c, 32c+32): 64 bytes = four 16-byte chunks of sub-tile c/2
#pragma unroll
        for (int g = 0; g < 4; ++g)
          *reinterpret_cast<uint4*>(sDS + (c >> 1) * 16384 + sw128_offset(tid, (c & 1) * 4 + g)) =
              make_uint4(dsk[g * 4 + 0], dsk[g * 4 + 1], dsk[g * 4 + 2], dsk[g * 4 + 3]);
      }
      tmem_st_wait();
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(&bar_pds);
      // ---- dQ tile: thread = query row now
      if (!(ok = mbar_wait(&bar_g, i & 1, &abort_word, 32))) break;
      tc_fence_after();
      float* dst = p.dq_acc + (row_base + (size_t)qb * kTile + tid) * D;
#pragma unroll
      for (int part = 0; part < Cfg::kSub; ++part) {
        const uint32_t td = part == 0 ? tDQ0 : tDQ1;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t r[32];
          tmem_ld32(td + lane_base + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; e += 4)
            red_add_v4(dst + part * 64 + c * 32 + e, __uint_as_float(r[e]) * p.scale, __uint_as_float(r[e + 1]) * p.scale,
                       __uint_as_float(r[e + 2]) * p.scale, __uint_as_float(r[e + 3]) * p.scale);
        }
      }
      tc_fence_before();
      mbar_arrive(&bar_dqr);
    }
    // ---- epilogue: dV, scale * dK -> bf16 -> swizzled smem (Q / dO buffers are free) -> TMA stores
    if (ok) {
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        const uint32_t tsrc = which == 0 ? tDV : tDK;
        uint8_t* stage = which == 0 ? sQ : sDO;
        const float f = which == 0 ? 1.f : p.scale;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(tsrc + lane_base + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 v;
            v.x = pack_bf16(__uint_as_float(r[g * 8 + 0]) * f, __uint_as_float(r[g * 8 + 1]) * f);
            v.y = pack_bf16(__uint_as_float(r[g * 8 + 2]) * f, __uint_as_float(r[g * 8 + 3]) * f);
            v.z = pack_bf16(__uint_as_float(r[g * 8 + 4]) * f, __uint_as_float(r[g * 8 + 5]) * f);
            v.w = pack_bf16(__uint_as_float(r[g * 8 + 6]) * f, __uint_as_float(r[g * 8 + 7]) * f);
            const int chunk = c * 4 + g;
            *reinterpret_cast<uint4*>(stage + (chunk >> 3) * 16384 + sw128_offset(tid, chunk & 7)) = v;
          }
        }
      }
      fence_async_smem();
      mbar_arrive(&bar_epi);
    }
    if (tid == 0 && ok && mbar_wait(&bar_epi, 0, &abort_word, 33)) {
      for (int s = 0; s < Cfg::kSub; ++s) {
        tma_store_4d(&mapDV, sQ + s * 16384, s * 64, kb * kTile, h, b);
        tma_store_4d(&mapDK, sDO + s * 16384, s * 64, kb * kTile, h, b);
      }
      tma_store_commit();
      tma_store_wait_all();
    }
  }

  tc_fence_before();
  __syncthreads();
  if (abort_word != 0) {
    if (tid == 0) atomicCAS(P.status, 0, 2000 + abort_word);
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  if (warp == 5) tmem_dealloc(tmem, 512);
}

// One warp per (b, h, t): delta and lse2.  Rows t >= T of the padded arrays get lse2 = +inf (P = 0) and delta = 0.
template <int D>
__global__ void __launch_bounds__(256) bwd_prep_kernel(const __nv_bfloat16* out, const __nv_bfloat16* dout, const float* lse,
                                                       int64_t o_sb, int64_t o_sh, int64_t o_st, int64_t d_sb, int64_t d_sh,
                                                       int64_t d_st, int B, int H, int T, int Tp, float* lse2, float* delta) {
  const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= (int64_t)B * H * Tp) return;
  const int t = (int)(row % Tp);
  const int64_t bh = row / Tp;
  const int h = (int)(bh % H), b = (int)(bh / H);
  float acc = 0.f, l2 = CUDART_INF_F;
  if (t < T) {
    const __nv_bfloat16* o = out + b * o_sb + h * o_sh + (int64_t)t * o_st;
    const __nv_bfloat16* d = dout + b * d_sb + h * d_sh + (int64_t)t * d_st;
    constexpr int kPer = D / 32;  // 2 or 4 elements per lane
#pragma unroll
    for (int i = 0; i < kPer; i += 2) {
      const __nv_bfloat162 ov = *reinterpret_cast<const __nv_bfloat162*>(o + lane * kPer + i);
      const __nv_bfloat162 dv = *reinterpret_cast<const __nv_bfloat162*>(d + lane * kPer + i);
      acc += __bfloat162float(ov.x) * __bfloat162float(dv.x) + __bfloat162float(ov.y) * __bfloat162float(dv.y);
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
    const float l = lse[bh * T + t];
    l2 = (l == -CUDART_INF_F) ? CUDART_INF_F : l * 1.4426950408889634f;
  }
  if (lane == 0) {
    lse2[row] = l2;
    delta[row] = acc;
  }
}

template <int D>
__global__ void __launch_bounds__(256) dq_convert_kernel(const float* acc, __nv_bfloat16* dq, int64_t sb, int64_t sh, int64_t st,
                                                         int B, int H, int T, int Tp) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // one thread per 8 elements
  constexpr int kPerRow = D / 8;
  const int64_t total = (int64_t)B * H * T * kPerRow;
  if (idx >= total) return;
  const int c = (int)(idx % kPerRow);
  const int64_t rt = idx / kPerRow;
  const int t = (int)(rt % T);
  const int64_t bh = rt / T;
  const int h = (int)(bh % H), b = (int)(bh / H);
  const float4* src = reinterpret_cast<const float4*>(acc + ((bh * Tp + t) * D + c * 8));
  const float4 a = src[0], e = src[1];
  uint4 v;
  v.x = pack_bf16(a.x, a.y); v.y = pack_bf16(a.z, a.w); v.z = pack_bf16(e.x, e.y); v.w = pack_bf16(e.z, e.w);
  *reinterpret_cast<uint4*>(dq + b * sb + h * sh + (int64_t)t * st + c * 8) = v;
}

size_t bwd_workspace_bytes(int B, int H, int T, int D) {
  const size_t Tp = (size_t)((T + kTile - 1) / kTile) * kTile;
  const size_t rows = (size_t)B * H * Tp;
  return plan_align(rows * 4) * 2 + plan_align(rows * D * 4);
}

template <int D>
static int launch_bwd_t(const void* q, const void* k, const void* v, const void* out, const void* dout, const float* lse,
                        const int64_t* sq, const int64_t* sk, const int64_t* sv, const int64_t* so, const int64_t* sdo, int B,
                        int H, int T, float scale, PlanView P, MaskArgs M, void* dq, void* dk, void* dv, const int64_t* sdq,
                        const int64_t* sdk, const int64_t* sdv, void* workspace, cudaStream_t stream) {
  const int Tp = P.NB * kTile;
  const size_t rows = (size_t)B * H * Tp;
  char* ws = static_cast<char*>(workspace);
  float* lse2 = reinterpret_cast<float*>(ws);
  float* delta = reinterpret_cast<float*>(ws + plan_align(rows * 4));
  float* dq_acc = reinterpret_cast<float*>(ws + 2 * plan_align(rows * 4));
  CUtensorMap mq, mk, mv, mdo, mdk, mdv;
  int r;
  if ((r = make_tile_map(&mq, q, 2, B, H, T, D, sq[0], sq[1], sq[2], kTile, 64))) return r;
  if ((r = make_tile_map(&mk, k, 2, B, H, T, D, sk[0], sk[1], sk[2], kTile, 64))) return r;
  if ((r = make_tile_map(&mv, v, 2, B, H, T, D, sv[0], sv[1], sv[2], kTile, 64))) return r;
  if ((r = make_tile_map(&mdo, dout, 2, B, H, T, D, sdo[0], sdo[1], sdo[2], kTile, 64))) return r;
  if ((r = make_tile_map(&mdk, dk, 2, B, H, T, D, sdk[0], sdk[1], sdk[2], kTile, 64))) return r;
  if ((r = make_tile_map(&mdv, dv, 2, B, H, T, D, sdv[0], sdv[1], sdv[2], kTile, 64))) return r;
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return -120;
  if (!attr_done[dev]) {
    if (cudaFuncSetAttribute(attn_bwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem<D>::kBytes) != cudaSuccess)
      return -120;
    attr_done[dev] = true;
  }
  cudaMemsetAsync(dq_acc, 0, rows * D * 4, stream);
  bwd_prep_kernel<D><<<(unsigned)((rows + 7) / 8), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(dout), lse, so[0], so[1], so[2], sdo[0], sdo[1],
      sdo[2], B, H, T, Tp, lse2, delta);
  BwdParams p;
  p.plan = P; p.mask = M; p.lse2 = lse2; p.delta = delta; p.dq_acc = dq_acc;
  p.dk = static_cast<__nv_bfloat16*>(dk); p.dv = static_cast<__nv_bfloat16*>(dv);
  for (int i = 0; i < 3; ++i) { p.dk_s[i] = sdk[i]; p.dv_s[i] = sdv[i]; }
  p.H = H; p.Tp = Tp; p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  {
    ProfileScope timed(1, stream);
    attn_bwd_kernel<D><<<(unsigned)B * H * P.NB, kBwdThreads, BwdSmem<D>::kBytes, stream>>>(mq, mk, mv, mdo, mdk, mdv, p);
  }
  const int64_t n8 = (int64_t)B * H * T * (D / 8);
  dq_convert_kernel<D><<<(unsigned)((n8 + 255) / 256), 256, 0, stream>>>(dq_acc, static_cast<__nv_bfloat16*>(dq), sdq[0], sdq[1],
                                                                         sdq[2], B, H, T, Tp);
  return cudaGetLastError() == cudaSuccess ? 0 : -121;
}

int launch_bwd(const void* q, const void* k, const void* v, const void* out, const void* dout, const float* lse, const int64_t* sq,
               const int64_t* sk, const int64_t* sv, const int64_t* so, const int64_t* sdo, int B, int H, int T, int D, float scale,
               PlanView P, MaskArgs M, void* dq, void* dk, void* dv, const int64_t* sdq, const int64_t* sdk, const int64_t* sdv,
               void* workspace, cudaStream_t stream) {
  if (D == 128)
    return launch_bwd_t<128>(q, k, v, out, dout, lse, sq, sk, sv, so, sdo, B, H, T, scale, P, M, dq, dk, dv, sdq, sdk, sdv, workspace, stream);
  if (D == 64)
    return launch_bwd_t<64>(q, k, v, out, dout, lse, sq, sk, sv, so, sdo, B, H, T, scale, P, M, dq, dk, dv, sdq, sdk, sdv, workspace, stream);
  return -122;
}

}  // namespace ts2ts
