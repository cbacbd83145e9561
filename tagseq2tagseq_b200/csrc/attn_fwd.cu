// Masked flash-attention forward for sm_100a.
//
// One CTA owns one 128-row query tile of one (batch, head) and walks the
// non-skipped key tiles listed for it in the block plan.  Per key tile:
//   TMA       K, V tiles -> shared memory (128-byte swizzle)
//   tcgen05   S = Q K^T           (bf16 x bf16 -> fp32 in tensor memory)
//   softmax   4 warps, one thread per query row: tcgen05.ld of the row's 128 scores once into
//             registers, mask (partial tiles only, by bit tests against a per-row 128-bit column
//             mask built from the tile's runs), online softmax in base 2 (row maximum and sum
//             need no exchange between threads), P -> bf16 -> tcgen05.st over the first 64
//             score columns
//   tcgen05   O += P V            (P read from tensor memory, V MN-major from smem)
// The accumulator is rescaled lazily: only when a row's running maximum grows
// by more than 2^8, so most tiles never touch O in the softmax warps.
//
// Roles: warps 0-3 softmax / epilogue (setmaxnreg 216), warp 4 TMA producer, warp 5 MMA
// issuer (40 registers; warps 6-7 only complete the warpgroup for setmaxnreg).
// Shared memory 3 tiles (Q, K, V) so two CTAs fit on one SM and overlap one
// another's softmax and MMA phases; 256 TMEM columns per CTA (S/P 128, O <=128).
//
// Computes what the reference obtains from PyTorch FlexAttention's forward
// (model/modules/layer.py:33 via tunalab FlexSelfAttention; semantics in
// torch/_higher_order_ops/flex_attention.py:218-287): O = softmax(scale QK^T +
// mask) V, LSE in natural log, a fully masked row gives O = 0 and LSE = -inf.
#include "plan.h"
#include "profile.h"
#include "ptx.cuh"
#include "tma_host.h"

#include <math_constants.h>
#ifdef TS2TS_TRACE
#include <stdio.h>
#include <stdlib.h>
#endif

namespace ts2ts {

struct FwdParams {
  PlanView plan;
  MaskArgs mask;
  float* lse;            // [B,H,T]
  __nv_bfloat16* out;    // for the empty-list path only
  int64_t o_sb, o_sh, o_st;
  int H;
  float scale_log2;      // softmax scale * log2(e)
#ifdef TS2TS_TRACE
  long long* trace;
  unsigned trace_block;
#endif
};

#ifdef TS2TS_TRACE
#define FTRACE(role, step, ev) do { if (p.trace && blockIdx.x == p.trace_block) { \
  p.trace[(((role) * 64 + ((step) & 63)) * 8 + (ev))] = clock64(); } } while (0)
#else
#define FTRACE(role, step, ev) do { } while (0)
#endif

constexpr int kFwdThreads = 256;  // warps 0-3 softmax (thread = query row), 4 TMA producer, 5 MMA issuer, 6-7 idle
constexpr int kFwdProducerWarp = 4, kFwdMmaWarp = 5;
template <uint32_t N> __device__ __forceinline__ void fwd_reg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <uint32_t N> __device__ __forceinline__ void fwd_reg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }
constexpr float kRescaleThreshold = 8.0f;

template <int D>
struct FwdSmem {
  static constexpr int kSub = D / 64;
  static constexpr int kTileBytes = kTile * D * 2;
  // + alignment slack; never less than 100 KB so that at most two CTAs (2 x 256 TMEM columns) share an SM
  static constexpr int kBytes = (3 * kTileBytes + 1024) > 100 * 1024 ? (3 * kTileBytes + 1024) : 100 * 1024;
};

// 128-bit mask of the key columns of tile `kb` that query (doc, row class) may read, before causality.
__device__ __forceinline__ void allowed_columns(const PlanView& P, const MaskArgs& M, int b, int kb, int mydoc, int myrow,
                                                uint32_t (&bits)[4]) {
  bits[0] = bits[1] = bits[2] = bits[3] = 0u;
  const int n = P.run_cnt[(size_t)b * P.NB + kb];
  const Run* runs = P.runs + ((size_t)b * P.NB + kb) * kTile;
  const int n_valid = min(kTile, P.T - kb * kTile);
  const int64_t* link_row = (M.link != nullptr && myrow >= 0 && myrow < M.R) ? M.link + ((size_t)b * M.R + myrow) * M.W : nullptr;
  for (int r = 0; r < n; ++r) {
    const int4 raw = __ldg(reinterpret_cast<const int4*>(runs + r));
    const int start = raw.x, doc = raw.y, col = raw.w;
    const int end = (r + 1 < n) ? __ldg(&runs[r + 1].start) : n_valid;
    bool ok = doc == mydoc;
    if (!ok && link_row != nullptr && col >= 0 && col < 64 * M.W)
      ok = (static_cast<unsigned long long>(__ldg(link_row + (col >> 6))) >> (col & 63)) & 1ull;
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
__global__ void __launch_bounds__(kFwdThreads, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapO, const FwdParams p) {
  using Cfg = FwdSmem<D>;
  extern __shared__ uint8_t smem_raw[];
  // Plain pointer arithmetic (no round trip through an integer) keeps the shared address space visible to the
  // compiler, so every access below becomes a shared-memory instruction instead of a generic one.
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* sQ = smem;
  uint8_t* sK = smem + Cfg::kTileBytes;
  uint8_t* sV = smem + 2 * Cfg::kTileBytes;
  __shared__ uint64_t bar_q, bar_k, bar_v, bar_s, bar_p, bar_o, bar_epi;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_word;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const PlanView& P = p.plan;
  const int NB = P.NB;
  const int rank = blockIdx.x % NB;
  const int bh = blockIdx.x / NB;
  const int h = bh % p.H, b = bh / p.H;
  const int qb = P.fwd_order[(size_t)b * NB + rank];
  const int n = P.fwd_cnt[(size_t)b * NB + qb];
  const int32_t* list = P.fwd_idx + ((size_t)b * NB + qb) * NB;

  if (n == 0) {  // no readable key tile: defined result, nothing to compute
    if (tid < kTile) {
      const int q = qb * kTile + tid;
      if (q < P.T) {
        __nv_bfloat16* o = p.out + (size_t)b * p.o_sb + (size_t)h * p.o_sh + (size_t)q * p.o_st;
        for (int i = 0; i < D; i += 8) *reinterpret_cast<uint4*>(o + i) = make_uint4(0, 0, 0, 0);
        p.lse[((size_t)b * p.H + h) * P.T + q] = -CUDART_INF_F;
      }
    }
    return;
  }

  if (tid == 0) {
    abort_word = 0;
    mbar_init(&bar_q, 1);
    mbar_init(&bar_k, 1);
    mbar_init(&bar_v, 1);
    mbar_init(&bar_s, 1);
    mbar_init(&bar_p, kTile);
    mbar_init(&bar_o, 1);
    mbar_init(&bar_epi, kTile);
    fence_mbar_init();
  }
  __syncthreads();
  if (warp == kFwdMmaWarp) {
    tmem_alloc(&tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  const uint32_t tS = tmem;         // S fp32 [128 lanes x 128 cols]; P bf16 overlays cols [0,64)
  const uint32_t tO = tmem + 128;   // O fp32 [128 lanes x D cols]

  if (warp >= 4) {
    fwd_reg_dec<40>();
  }
  if (warp == kFwdProducerWarp) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&mapQ); tma_prefetch_desc(&mapK); tma_prefetch_desc(&mapV);
      mbar_expect_tx(&bar_q, Cfg::kTileBytes);
      for (int s = 0; s < Cfg::kSub; ++s) tma_load_4d(sQ + s * 16384, &mapQ, &bar_q, s * 64, qb * kTile, h, b);
      for (int j = 0; j < n; ++j) {
        const int kb = list[j] & ~kFullBit;
        if (j > 0 && !mbar_wait(&bar_s, (j - 1) & 1, &abort_word, 11)) break;  // S(j-1) done: K buffer free
        mbar_expect_tx(&bar_k, Cfg::kTileBytes);
        for (int s = 0; s < Cfg::kSub; ++s) tma_load_4d(sK + s * 16384, &mapK, &bar_k, s * 64, kb * kTile, h, b);
        if (j > 0 && !mbar_wait(&bar_o, (j - 1) & 1, &abort_word, 12)) break;  // PV(j-1) done: V buffer free
        mbar_expect_tx(&bar_v, Cfg::kTileBytes);
        for (int s = 0; s < Cfg::kSub; ++s) tma_load_4d(sV + s * 16384, &mapV, &bar_v, s * 64, kb * kTile, h, b);
      }
    }
  } else if (warp == kFwdMmaWarp) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(128, D, false, true);
      // descriptor halves: K-major operands (Q, K) step 32 B inside a 128-byte row and 16 KB between the two
      // 64-column halves; the MN-major operand (V) steps 16 key rows = 2048 B
      constexpr uint32_t hi_k = desc_hi(1024);
      const uint32_t q_lo = desc_lo(smem_u32(sQ), 16), k_lo = desc_lo(smem_u32(sK), 16), v_lo = desc_lo(smem_u32(sV), 16384);
      // Shared-memory accesses of this thread (barrier waits included) queue behind the MMAs it has issued and only
      // proceed once the tensor pipe has accepted those, so the wait for the next K tile (normally long complete)
      // sits two MMAs before the end of the PV group: the pipe stays fed while the wait runs.
      bool ok = mbar_wait(&bar_q, 0, &abort_word, 21) && mbar_wait(&bar_k, 0, &abort_word, 22);
      for (int j = 0; j < n && ok; ++j) {
#ifdef TS2TS_STRICT_ORDER
        if (j > 0 && !mbar_wait(&bar_o, (j - 1) & 1, &abort_word, 23)) break;  // P(j-1) consumed before S is overwritten
#endif
        // S(j) overwrites the columns that P(j-1) occupies; its reader, PV(j-1), was issued by this thread just
        // before and the tensor pipe executes this thread's MMAs in issue order.
        tc_fence_after();
        FTRACE(0, j, 0);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = ((kk >> 2) * 16384 + (kk & 3) * 32) >> 4;
          mma_ss2(tS, q_lo + off, hi_k, k_lo + off, hi_k, idesc_s, kk > 0);
        }
        mma_commit(&bar_s);
        FTRACE(0, j, 1);
        if (!mbar_wait(&bar_v, j & 1, &abort_word, 24)) break;
        if (!mbar_wait(&bar_p, j & 1, &abort_word, 25)) break;
        tc_fence_after();
        FTRACE(0, j, 2);
        constexpr int kSplit = kTile / 16 - 2;
#pragma unroll
        for (int kk = 0; kk < kSplit; ++kk)
          mma_ts2(tO, tS + kk * 8, v_lo + kk * (2048 >> 4), hi_k, idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
        if (j + 1 < n && !mbar_wait(&bar_k, (j + 1) & 1, &abort_word, 22)) break;
#pragma unroll
        for (int kk = kSplit; kk < kTile / 16; ++kk)
          mma_ts2(tO, tS + kk * 8, v_lo + kk * (2048 >> 4), hi_k, idesc_pv, 1u);
        mma_commit(&bar_o);
        FTRACE(0, j, 3);
      }
    }
  } else if (warp < 4) {
    // ------------------------------------------------------------------ softmax + epilogue: thread = query row
    // One thread owns a whole score row: the row maximum and sum need no exchange between threads and the 128
    // scores are read from tensor memory once and stay in registers between the two sweeps.
    fwd_reg_inc<216>();
    const int row = tid;
    const int q = qb * kTile + row;
    const bool q_valid = q < P.T;
    const int mydoc = q_valid ? p.mask.doc[(size_t)b * P.T + q] : INT32_MIN;
    const int myrow = q_valid ? p.mask.row[(size_t)b * P.T + q] : -1;
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    const uint32_t tSr = tS + lane_base;
    const uint32_t tOr = tO + lane_base;
    float m_used = -CUDART_INF_F, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n; ++j) {
      const int entry = list[j];
      const int kb = entry & ~kFullBit;
      const bool is_full = (entry & kFullBit) != 0;
      uint32_t bits[4] = {0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu};
      if (!is_full) {
        allowed_columns(P, p.mask, b, kb, mydoc, myrow, bits);
        if (kb == qb) {  // causal inside the diagonal tile: columns 0..row
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            const int hi = row + 1 - 32 * w;
            bits[w] &= hi >= 32 ? 0xffffffffu : (hi <= 0 ? 0u : ((1u << hi) - 1u));
          }
        }
      }
      if (tid == 0) FTRACE(1, j, 0);
      if (!(ok = mbar_wait(&bar_s, j & 1, &abort_word, 31))) break;
      tc_fence_after();
      if (tid == 0) FTRACE(1, j, 1);
      uint32_t sv[4][32];
      tmem_ld32(tSr, sv[0]);
      tmem_ld32(tSr + 32, sv[1]);
      tmem_ld32(tSr + 64, sv[2]);
      tmem_ld32(tSr + 96, sv[3]);
      tmem_ld_wait();
      // sweep 1: row maximum (eight independent running maxima keep the dependency chain short)
      float mx8[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) mx8[i] = -CUDART_INF_F;
      if (is_full) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 16; ++i) mx8[i & 7] = fmax3(mx8[i & 7], __uint_as_float(sv[c][i]), __uint_as_float(sv[c][i + 16]));
      } else {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 16; ++i)
            mx8[i & 7] = fmax3(mx8[i & 7], ((bits[c] >> i) & 1u) ? __uint_as_float(sv[c][i]) : -CUDART_INF_F,
                               ((bits[c] >> (i + 16)) & 1u) ? __uint_as_float(sv[c][i + 16]) : -CUDART_INF_F);
      }
      float mx = fmax3(fmax3(mx8[0], mx8[1], mx8[2]), fmax3(mx8[3], mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7]));
      if (tid == 0) FTRACE(1, j, 2);
      mx *= p.scale_log2;  // scale > 0, so max commutes with the scaling
      const float m_new = fmaxf(m_used, mx);
      const bool need = m_new > m_used + kRescaleThreshold || (m_used == -CUDART_INF_F && m_new > -CUDART_INF_F);
      if (__any_sync(0xffffffffu, need)) {
        const float factor = need ? fast_exp2(m_used - m_new) : 1.f;  // exp2(-inf) = 0 on the first real tile
        if (j > 0) {
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t r[32];
            tmem_ld32(tOr + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * factor);
            tmem_st32(tOr + c * 32, r);
          }
        }
        l *= factor;
        if (need) m_used = m_new;
      }
      if (tid == 0) FTRACE(1, j, 3);
      const float m_safe = m_used == -CUDART_INF_F ? 0.f : m_used;
      // sweep 2: P = exp2(s - m), row sum (four independent sums), bf16 pack over the first 64 score columns
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0 = fast_exp2(fmaf(__uint_as_float(sv[c][i]), p.scale_log2, -m_safe));
          float p1 = fast_exp2(fmaf(__uint_as_float(sv[c][i + 1]), p.scale_log2, -m_safe));
          if (!is_full) {
            p0 = ((bits[c] >> i) & 1u) ? p0 : 0.f;
            p1 = ((bits[c] >> (i + 1)) & 1u) ? p1 : 0.f;
          }
          sum4[(i >> 1) & 3] += p0 + p1;
          pk[i >> 1] = pack_bf16(p0, p1);
        }
        tmem_st16(tSr + c * 16, pk);
      }
      l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      if (tid == 0) FTRACE(1, j, 4);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bar_p);
      if (tid == 0) FTRACE(1, j, 5);
    }
    // ---- epilogue: O / l -> bf16 -> swizzled smem (Q buffer, free after the last S) -> TMA store
    if (ok) ok = mbar_wait(&bar_o, (n - 1) & 1, &abort_word, 32);
    tc_fence_after();
    if (ok) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(tOr + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 v;
          v.x = pack_bf16(__uint_as_float(r[g * 8 + 0]) * inv, __uint_as_float(r[g * 8 + 1]) * inv);
          v.y = pack_bf16(__uint_as_float(r[g * 8 + 2]) * inv, __uint_as_float(r[g * 8 + 3]) * inv);
          v.z = pack_bf16(__uint_as_float(r[g * 8 + 4]) * inv, __uint_as_float(r[g * 8 + 5]) * inv);
          v.w = pack_bf16(__uint_as_float(r[g * 8 + 6]) * inv, __uint_as_float(r[g * 8 + 7]) * inv);
          const int chunk = c * 4 + g;  // 16-byte chunk index inside the output row
          *reinterpret_cast<uint4*>(sQ + (chunk >> 3) * 16384 + sw128_offset(row, chunk & 7)) = v;
        }
      }
      if (q_valid) p.lse[((size_t)b * p.H + h) * P.T + q] = l > 0.f ? (m_used + log2f(l)) * 0.6931471805599453f : -CUDART_INF_F;
      fence_async_smem();
      mbar_arrive(&bar_epi);
    }
    if (tid == 0 && ok && mbar_wait(&bar_epi, 0, &abort_word, 33)) {
      for (int s = 0; s < Cfg::kSub; ++s) tma_store_4d(&mapO, sQ + s * 16384, s * 64, qb * kTile, h, b);
      tma_store_commit();
      tma_store_wait_all();
    }
  }

  tc_fence_before();
  __syncthreads();
  if (abort_word != 0) {
    // Let loads that were issued but never consumed land before the CTA's shared memory is released.
    if (tid == 0) atomicCAS(P.status, 0, 1000 + abort_word);
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  if (warp == kFwdMmaWarp) tmem_dealloc(tmem, 256);
}

// Host launcher.  Tensor strides are in elements; the last dimension is contiguous.
template <int D>
static int launch_fwd_t(const void* q, const void* k, const void* v, void* out, float* lse, const int64_t* sq,
                        const int64_t* sk, const int64_t* sv, const int64_t* so, int B, int H, int T, float scale,
                        PlanView P, MaskArgs M, cudaStream_t stream) {
  CUtensorMap mq, mk, mv, mo;
  int r;
  if ((r = make_tile_map(&mq, q, 2, B, H, T, D, sq[0], sq[1], sq[2], kTile, 64))) return r;
  if ((r = make_tile_map(&mk, k, 2, B, H, T, D, sk[0], sk[1], sk[2], kTile, 64))) return r;
  if ((r = make_tile_map(&mv, v, 2, B, H, T, D, sv[0], sv[1], sv[2], kTile, 64))) return r;
  if ((r = make_tile_map(&mo, out, 2, B, H, T, D, so[0], so[1], so[2], kTile, 64))) return r;
  FwdParams p;
  p.plan = P; p.mask = M; p.lse = lse; p.out = static_cast<__nv_bfloat16*>(out);
  p.o_sb = so[0]; p.o_sh = so[1]; p.o_st = so[2];
  p.H = H; p.scale_log2 = scale * 1.4426950408889634f;
#ifdef TS2TS_TRACE
  static long long* trace_buf = nullptr;
  if (!trace_buf) cudaMalloc(&trace_buf, 3 * 64 * 8 * sizeof(long long));
  cudaMemsetAsync(trace_buf, 0, 3 * 64 * 8 * sizeof(long long), stream);
  p.trace = trace_buf;
  p.trace_block = getenv("TS2TS_TRACE_BLOCK") ? (unsigned)atoi(getenv("TS2TS_TRACE_BLOCK")) : 0u;
#endif
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return -110;
  if (!attr_done[dev]) {
    if (cudaFuncSetAttribute(attn_fwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdSmem<D>::kBytes) != cudaSuccess)
      return -110;
    attr_done[dev] = true;
  }
  const unsigned grid = (unsigned)B * H * P.NB;
  {
    ProfileScope timed(0, stream);
    attn_fwd_kernel<D><<<grid, kFwdThreads, FwdSmem<D>::kBytes, stream>>>(mq, mk, mv, mo, p);
  }
#ifdef TS2TS_TRACE
  {
    static long long host[3 * 64 * 8];
    cudaStreamSynchronize(stream);
    cudaMemcpy(host, trace_buf, sizeof(host), cudaMemcpyDeviceToHost);
    FILE* f = fopen(getenv("TS2TS_FTRACE_FILE") ? getenv("TS2TS_FTRACE_FILE") : "ftrace.txt", "w");
    if (f) {
      for (int r = 0; r < 3; ++r)
        for (int u = 0; u < 64; ++u) {
          fprintf(f, "%d %d", r, u);
          for (int e = 0; e < 8; ++e) fprintf(f, " %lld", host[(r * 64 + u) * 8 + e]);
          fprintf(f, "\n");
        }
      fclose(f);
    }
  }
#endif
  return cudaGetLastError() == cudaSuccess ? 0 : -111;
}

int launch_fwd(const void* q, const void* k, const void* v, void* out, float* lse, const int64_t* sq, const int64_t* sk,
               const int64_t* sv, const int64_t* so, int B, int H, int T, int D, float scale, PlanView P, MaskArgs M,
               cudaStream_t stream) {
  if (D == 128) return launch_fwd_t<128>(q, k, v, out, lse, sq, sk, sv, so, B, H, T, scale, P, M, stream);
  if (D == 64) return launch_fwd_t<64>(q, k, v, out, lse, sq, sk, sv, so, B, H, T, scale, P, M, stream);
  return -112;
}

}  // namespace ts2ts
