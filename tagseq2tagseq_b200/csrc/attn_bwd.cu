// Masked flash-attention backward for sm_100a.
//
// Three kernels:
//   bwd_prep     delta[q] = sum_d O[q,d] dO[q,d],  lse2[q] = LSE[q] * log2(e)   (fp32, padded to whole tiles)
//   attn_bwd     one CTA per 128-key tile of one (batch, head); walks the non-skipped 128-query tiles of the
//                transposed block list.  Everything is transposed so that a tensor-memory lane is a key row:
//                  tcgen05  S^T = K Q^T,  dP^T = V dO^T            [128 keys x 128 queries, fp32 in TMEM, N = 128]
//                  warps 0-7 (two threads per key row, 64 queries each), in two phases:
//                           P^T = exp2(scale S^T - lse2[q]) under the mask, as soon as S^T is complete, written as
//                           bf16 over the S^T columns just read; then, once dP^T is complete and in two halves of 64
//                           queries, dS^T = P^T (dP^T - delta[q]) as bf16 next to P^T and to shared memory
//                  tcgen05  dV += P^T dO,  dK += dS^T Q           (A from TMEM, B MN-major from smem; issued per
//                           half, so the first half's MMAs overlap the second half's dS^T arithmetic)
//                           S^T of the NEXT tile, so that its exponentials run under the MMAs that follow
//                           dQ^T = K^T dS^T                       [D x 128 queries over the consumed dP^T columns]
//                           dP^T of the next tile once dQ^T has been read out
//                  warps 8-11 (thread = head-dim lane)  dQ^T -> scaled fp32, 32 queries at a time, through two
//                           private shared-memory boxes per warp -> TMA reduce-adds into the dQ accumulator
//                Q tiles are double-buffered in shared memory, dO has one buffer that is reloaded between the dV MMAs of
//                a tile and dP^T of the next.  dK (scaled) and dV leave through shared memory and TMA stores at the end.
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

// A debug build may name a private header that defines the hooks below to record clock64() stamps.
#ifdef TS2TS_BWD_TRACE_HEADER
#include TS2TS_BWD_TRACE_HEADER
#else
#define TS2TS_BWD_TRACE_FIELDS
#define TRACE(role, step, ev) do { } while (0)
#define BTRACE_ACC_DECL
#define BTRACE_ACC(k) do { } while (0)
#define BTRACE_ACC_DUMP() do { } while (0)
#define BTRACE_ATTACH(params, stream) do { } while (0)
#define BTRACE_DUMP(stream) do { } while (0)
#endif

#ifndef TS2TS_BWD_GROUP_MB
// Q/dO bytes of the heads whose CTAs are interleaved in the launch order.  Measured on the 32k masks in the
// seconds-long benchmark loop: 32 MB (one head at 32k, three at 16k) gives the best whole-step rate, 2-3 % above 64 MB
// and 16 MB; 136 MB is 4 % slower and all heads 10 % slower (Q / dO fall out of L2).
#define TS2TS_BWD_GROUP_MB 32
#endif

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
  int head_group;        // heads whose CTAs are interleaved in the launch order
  float scale, scale_log2;
  TS2TS_BWD_TRACE_FIELDS
};

constexpr int kBwdThreads = 512;  // warps 0-7 exp/dS, 8-11 dQ reduction, 12 TMA producer, 13 MMA issuer, 14-15 idle
constexpr int kSubQ = 64;         // query columns per compute half
constexpr int kRunSlotsB = 4;     // runs of a partial query tile that the producer copies to shared memory
#ifndef TS2TS_BWD_X2
#define TS2TS_BWD_X2 1
#endif
#ifndef TS2TS_BWD_LD2
#define TS2TS_BWD_LD2 0
#endif
#ifndef TS2TS_BWD_ELECT
#define TS2TS_BWD_ELECT 1
#endif
#ifndef TS2TS_BWD_DQ_FIRST
#define TS2TS_BWD_DQ_FIRST 1
#endif
#ifndef TS2TS_BWD_SPLIT_ST
#define TS2TS_BWD_SPLIT_ST 1  // S^T of the next tile in two 64-query halves, the first right behind the first half of dV / dK
#endif

template <int D>
struct BwdSmem {
  static constexpr int kSub = D / 64;
  static constexpr int kTileBytes = kTile * D * 2;
  static constexpr int kDsBytes = kTile * kTile * 2;  // dS^T: two halves of [128 key rows x 128 B]
  static constexpr int kStageBytes = 4 * 2 * 4096;     // dQ staging: per reduction warp two boxes of [32 queries x 32 floats]
  // K, V, two Q stages, one dO buffer, dS^T, the dQ staging boxes, then row statistics, barriers and flags; plus
  // alignment slack.  The kernel declares no static shared memory, so the dynamic region normally starts 1024-byte
  // aligned and the slack stays unused; if it ever does not fit, the kernel reports status 2900 instead of running.
  static constexpr int kTiles = 5 * kTileBytes + kDsBytes + kStageBytes;
  static constexpr int kSmall = 4 * kTile * 4 + 16 * 8 + 16 + 2 * kRunSlotsB * 16 + 16;  // statistics, barriers, flags, staged runs
  static constexpr int kSlack = 512;
  static constexpr int kBytes = kTiles + kSmall + kSlack;
  // tensor-memory columns: dV, dK accumulators, S^T (later P^T / dS^T), dP^T (later dQ^T)
  static constexpr int kDV = 0, kDK = D, kST = 2 * D, kDPT = 2 * D + 128;
};

template <uint32_t N> __device__ __forceinline__ void reg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <uint32_t N> __device__ __forceinline__ void reg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }

// What a backward thread knows about its key: document, column class, and how it looks up "may row class r read my
// column class": 0 = never (no links, or the key has no class), 1 = words of the transposed table kept in registers
// (R <= 256), 2 = words of the transposed table read from global memory, 3 = the untransposed table (no transposed
// one was built).
struct KeyCtx {
  int kvdoc, kvcol, mode;
  unsigned long long lt0, lt1, lt2, lt3;
  const unsigned long long* lt_row;
  const int64_t* link_col;  // &link[b][0][kvcol >> 6]
};
__device__ __forceinline__ bool row_class_allowed(const KeyCtx& k, const MaskArgs& M, int row) {
  if (k.mode == 0 || row < 0 || row >= M.R) return false;
  unsigned long long w;
  if (k.mode == 1) {
    const int wi = row >> 6;
    w = wi == 0 ? k.lt0 : wi == 1 ? k.lt1 : wi == 2 ? k.lt2 : k.lt3;
    return (w >> (row & 63)) & 1ull;
  }
  if (k.mode == 2) return (__ldg(k.lt_row + (row >> 6)) >> (row & 63)) & 1ull;
  return (static_cast<unsigned long long>(__ldg(k.link_col + (size_t)row * M.W)) >> (k.kvcol & 63)) & 1ull;
}
// 128-bit mask of the query rows of tile `qb` that may read this thread's key, before causality.  The first
// kRunSlotsB runs come from shared memory (`staged`), further ones from the plan in global memory.
__device__ __forceinline__ void allowed_rows(const PlanView& P, const MaskArgs& M, int b, int qb, const KeyCtx& k,
                                             const int4* staged, int n, uint32_t (&bits)[4]) {
  bits[0] = bits[1] = bits[2] = bits[3] = 0u;
  const Run* runs = P.runs + ((size_t)b * P.NB + qb) * kTile;
  const int n_valid = min(kTile, P.T - qb * kTile);
  auto get_run = [&](int r) { return r < kRunSlotsB ? staged[r] : __ldg(reinterpret_cast<const int4*>(runs + r)); };
  int4 cur = n > 0 ? get_run(0) : make_int4(0, 0, 0, 0);
  uint32_t lo[4];
  prefix_mask(cur.x, lo);
  for (int r = 0; r < n; ++r) {
    const int4 nx = r + 1 < n ? get_run(r + 1) : make_int4(n_valid, 0, 0, 0);
    uint32_t hi[4];
    prefix_mask(nx.x, hi);  // the run covers rows [cur.x, nx.x)
    if (cur.y == k.kvdoc || row_class_allowed(k, M, cur.z)) {
#pragma unroll
      for (int w = 0; w < 4; ++w) bits[w] |= hi[w] & ~lo[w];
    }
#pragma unroll
    for (int w = 0; w < 4; ++w) lo[w] = hi[w];
    cur = nx;
  }
}

// The per-tile arithmetic of a compute thread, 32 query columns at a time, in two phases so that the first can run
// while the tensor core still works on dQ^T of the previous tile and dP^T of this one:
//   p_chunk   P^T = exp2(scale S^T - lse2) under the mask, packed to bf16 pairs (the MMA operand, also kept in
//             registers for the second phase)
//   ds_chunk  dS^T = P^T (dP^T - delta), from the bf16 P^T, packed to bf16 pairs
// The row statistics of the 32 queries are read from shared memory; every lane of a warp reads the same addresses.
// `nl2` / `ndl` hold the NEGATED statistics (-lse2, -delta), so that both phases are one packed multiply-add /
// add per two queries (fp32x2 instructions; a 16-byte shared-memory load yields two ready operand pairs).
// mode: 0 = every query allowed, 1 = test the bits of `bw`, 2 = no query allowed (nothing is computed).
__device__ __forceinline__ void p_chunk(const uint32_t (&s)[32], const float* nl2, uint32_t bw, int mode, float scale_log2,
                                        uint32_t (&pk)[16]) {
  if (mode == 2) {
#pragma unroll
    for (int e = 0; e < 16; ++e) pk[e] = 0u;
    return;
  }
  const unsigned long long scale2 = pack_f32x2(scale_log2, scale_log2);
#pragma unroll
  for (int e = 0; e < 32; e += 4) {
    const ulonglong2 n4 = *reinterpret_cast<const ulonglong2*>(nl2 + e);
    float x0, x1, x2, x3;
#if TS2TS_BWD_X2
    unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(s[e + 0]), __uint_as_float(s[e + 1])), scale2, n4.x), x0, x1);
    unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(s[e + 2]), __uint_as_float(s[e + 3])), scale2, n4.y), x2, x3);
#else
    {
      float n0, n1, n2, n3;
      unpack_f32x2(n4.x, n0, n1); unpack_f32x2(n4.y, n2, n3);
      x0 = fmaf(__uint_as_float(s[e + 0]), scale_log2, n0); x1 = fmaf(__uint_as_float(s[e + 1]), scale_log2, n1);
      x2 = fmaf(__uint_as_float(s[e + 2]), scale_log2, n2); x3 = fmaf(__uint_as_float(s[e + 3]), scale_log2, n3);
    }
#endif
    float p0 = fast_exp2(x0), p1 = fast_exp2(x1), p2 = fast_exp2(x2), p3 = fast_exp2(x3);
    if (mode == 1) {
      p0 = ((bw >> (e + 0)) & 1u) ? p0 : 0.f;
      p1 = ((bw >> (e + 1)) & 1u) ? p1 : 0.f;
      p2 = ((bw >> (e + 2)) & 1u) ? p2 : 0.f;
      p3 = ((bw >> (e + 3)) & 1u) ? p3 : 0.f;
    }
    pk[(e >> 1) + 0] = pack_bf16(p0, p1);
    pk[(e >> 1) + 1] = pack_bf16(p2, p3);
  }
}
__device__ __forceinline__ void ds_chunk(const uint32_t (&pk)[16], const uint32_t (&dp)[32], const float* ndl, int mode,
                                         uint32_t (&dsk)[16]) {
  if (mode == 2) {
#pragma unroll
    for (int e = 0; e < 16; ++e) dsk[e] = 0u;
    return;
  }
#pragma unroll
  for (int e = 0; e < 32; e += 4) {
    const ulonglong2 d4 = *reinterpret_cast<const ulonglong2*>(ndl + e);
    const uint32_t a = pk[(e >> 1) + 0], c = pk[(e >> 1) + 1];
    const unsigned long long p01 = pack_f32x2(__uint_as_float(a << 16), __uint_as_float(a & 0xffff0000u));
    const unsigned long long p23 = pack_f32x2(__uint_as_float(c << 16), __uint_as_float(c & 0xffff0000u));
    float r0, r1, r2, r3;
#if TS2TS_BWD_X2
    unpack_f32x2(mul_f32x2(p01, add_f32x2(pack_f32x2(__uint_as_float(dp[e + 0]), __uint_as_float(dp[e + 1])), d4.x)), r0, r1);
    unpack_f32x2(mul_f32x2(p23, add_f32x2(pack_f32x2(__uint_as_float(dp[e + 2]), __uint_as_float(dp[e + 3])), d4.y)), r2, r3);
#else
    {
      float n0, n1, n2, n3, q0, q1, q2, q3;
      unpack_f32x2(d4.x, n0, n1); unpack_f32x2(d4.y, n2, n3);
      unpack_f32x2(p01, q0, q1); unpack_f32x2(p23, q2, q3);
      r0 = q0 * (__uint_as_float(dp[e + 0]) + n0); r1 = q1 * (__uint_as_float(dp[e + 1]) + n1);
      r2 = q2 * (__uint_as_float(dp[e + 2]) + n2); r3 = q3 * (__uint_as_float(dp[e + 3]) + n3);
    }
#endif
    dsk[(e >> 1) + 0] = pack_bf16(r0, r1);
    dsk[(e >> 1) + 1] = pack_bf16(r2, r3);
  }
}

template <int D>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapDO,
                const __grid_constant__ CUtensorMap mapDK, const __grid_constant__ CUtensorMap mapDV,
                const __grid_constant__ CUtensorMap mapDQ, const BwdParams p) {
  using Cfg = BwdSmem<D>;
  extern __shared__ uint8_t smem_raw[];
  // Plain pointer arithmetic (no round trip through an integer) keeps the shared address space visible to the
  // compiler, so every access below becomes a shared-memory instruction instead of a generic one.
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* sK = smem;
  uint8_t* sV = smem + Cfg::kTileBytes;           // must follow sK directly (dQ^T operand padding for D = 64)
  uint8_t* sQ = smem + 2 * Cfg::kTileBytes;       // two stages, Cfg::kTileBytes each
  uint8_t* sDO = smem + 4 * Cfg::kTileBytes;      // one buffer: reloaded between the dV MMAs of a tile and dP^T of the next
  uint8_t* sDS = smem + 5 * Cfg::kTileBytes;      // dS^T, halves of 16 KB
  uint8_t* sStage = sDS + Cfg::kDsBytes;          // dQ staging boxes
  float (*s_lse2)[kTile] = reinterpret_cast<float (*)[kTile]>(smem + Cfg::kTiles);
  float (*s_delta)[kTile] = reinterpret_cast<float (*)[kTile]>(smem + Cfg::kTiles + 2 * kTile * 4);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kTiles + 4 * kTile * 4);
  uint64_t& bar_kv = bars[0];
  uint64_t* bar_q_full = bars + 1;     // [2] Q, lse2, delta of a stage landed
  uint64_t& bar_do_full = bars[3];     // dO of the tile landed
  uint64_t& bar_gd = bars[4];          // dV / dK MMAs of the tile completed: its Q stage and the dO buffer may be reloaded
  uint64_t& bar_st = bars[5];          // S^T and dP^T of the tile are in tensor memory
  uint64_t* bar_pds = bars + 6;        // [2] P^T / dS^T of a 64-query half written
  uint64_t& bar_g = bars[8];           // gradient MMAs of the tile completed (dQ^T readable)
  uint64_t& bar_dqr = bars[9];         // dQ^T read out of tensor memory
  uint64_t& bar_epi = bars[10];
  uint64_t* bar_s = bars + 12;         // [2] S^T of a 64-query half of the tile is in tensor memory (dP^T may still be running)
  uint32_t& tmem_slot = *reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_ptr = reinterpret_cast<volatile int*>(reinterpret_cast<uint8_t*>(bars + 16) + 4);
  int* abort_w = const_cast<int*>(abort_ptr);
  int4* s_runs = reinterpret_cast<int4*>(bars + 18);                  // [2 stages][kRunSlotsB] first runs of a partial query tile
  int* s_nruns = reinterpret_cast<int*>(s_runs + 2 * kRunSlotsB);     // [2] its number of runs
  {  // uniform across the grid: refuse a plan that was not built for this (B, T), or a misplaced shared-memory window
    int bad = 0;
    const int32_t* stw = p.plan.status;
    if (stw[kStampMagic] != kPlanMagic || stw[kStampB] != p.plan.B || stw[kStampT] != p.plan.T) bad = 2901;
    else if (smem + Cfg::kTiles + Cfg::kSmall > smem_raw + Cfg::kBytes) bad = 2900;
    if (bad) {
      if (threadIdx.x == 0) atomicCAS(p.plan.status, 0, bad);
      return;
    }
  }

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const PlanView& P = p.plan;
  const int NB = P.NB;
  // Launch order (the hardware starts CTAs by ascending blockIdx): batch elements one after the other; inside one,
  // groups of G heads; inside a group all heads' heaviest kv tiles first, then their second heaviest, and so on.  The
  // group bounds the Q / dO working set that has to stay in L2, and the long CTAs of the last group still start well
  // before the end of the launch instead of running alone at its tail.
  const int per_b = p.H * NB, G = p.head_group;
  const int b = blockIdx.x / per_b;
  const int r1 = blockIdx.x - b * per_b;
  const int grp = r1 / (G * NB);
  const int r2 = r1 - grp * G * NB;
  const int gsize = min(G, p.H - grp * G);
  const int rank = r2 / gsize;
  const int h = grp * G + (r2 - rank * gsize);
  const int kb = min(max(P.bwd_order[(size_t)b * NB + rank], 0), NB - 1);
  const int n = min(max(P.bwd_cnt[(size_t)b * NB + kb], 0), NB);
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
    *abort_ptr = 0;
    mbar_init(&bar_kv, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar_q_full[i], 1);
      mbar_init(&bar_pds[i], TS2TS_BWD_ELECT ? 8 : 2 * kTile);  // one arrival per compute warp
    }
    mbar_init(&bar_do_full, 1);
    mbar_init(&bar_gd, 1);
    mbar_init(&bar_st, 1);
    mbar_init(&bar_g, 1);
    mbar_init(&bar_dqr, kTile);
    mbar_init(&bar_epi, 2 * kTile);
    mbar_init(&bar_s[0], 1);
    mbar_init(&bar_s[1], 1);
    fence_mbar_init();
  }
  __syncthreads();
  if (warp == 13) {
    tmem_alloc(&tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  const uint32_t tDV = tmem + Cfg::kDV, tDK = tmem + Cfg::kDK, tST = tmem + Cfg::kST, tDPT = tmem + Cfg::kDPT;
  // S^T columns [64s + 32h, +32) are read by the compute thread (row, h) in half s and overwritten by it with
  // P^T bf16 [.., +16) and dS^T bf16 [.. + 16, +16) for its 32 queries.

  if (warp >= 12) {
    reg_dec<88>();
    if (warp == 12 && lane == 0) {
      // ---------------------------------------------------------------- TMA producer
      tma_prefetch_desc(&mapQ); tma_prefetch_desc(&mapK); tma_prefetch_desc(&mapV); tma_prefetch_desc(&mapDO);
      mbar_expect_tx(&bar_kv, 2 * Cfg::kTileBytes);
      for (int s = 0; s < Cfg::kSub; ++s) {
        tma_load_4d(sK + s * 16384, &mapK, &bar_kv, s * 64, kb * kTile, h, b);
        tma_load_4d(sV + s * 16384, &mapV, &bar_kv, s * 64, kb * kTile, h, b);
      }
      auto load_q = [&](int i) {  // Q tile and row statistics of tile i into stage i & 1
        const int entry = list[i];
        const int qb = min(entry & ~kFullBit, NB - 1);
        const int st = i & 1;
        if (!(entry & kFullBit)) {
          // partial tile: its first runs travel with the stage (the arrive below publishes these plain stores)
          const size_t tq = (size_t)b * NB + qb;
          const int4* src = reinterpret_cast<const int4*>(P.runs + tq * kTile);
          const int4 r0 = __ldg(src), r1 = __ldg(src + 1), r2 = __ldg(src + 2), r3 = __ldg(src + 3);
          s_nruns[st] = min(max(__ldg(&P.run_cnt[tq]), 0), kTile);
          s_runs[st * kRunSlotsB + 0] = r0; s_runs[st * kRunSlotsB + 1] = r1;
          s_runs[st * kRunSlotsB + 2] = r2; s_runs[st * kRunSlotsB + 3] = r3;
        }
        mbar_expect_tx(&bar_q_full[st], Cfg::kTileBytes + 2 * kTile * 4);
        for (int s = 0; s < Cfg::kSub; ++s)
          tma_load_4d(sQ + st * Cfg::kTileBytes + s * 16384, &mapQ, &bar_q_full[st], s * 64, qb * kTile, h, b);
        const size_t stat = ((size_t)b * p.H + h) * p.Tp + (size_t)qb * kTile;
        bulk_load(s_lse2[st], p.lse2 + stat, kTile * 4, &bar_q_full[st]);
        bulk_load(s_delta[st], p.delta + stat, kTile * 4, &bar_q_full[st]);
      };
      auto load_do = [&](int i) {
        const int qb = list[i] & ~kFullBit;
        mbar_expect_tx(&bar_do_full, Cfg::kTileBytes);
        for (int s = 0; s < Cfg::kSub; ++s) tma_load_4d(sDO + s * 16384, &mapDO, &bar_do_full, s * 64, qb * kTile, h, b);
      };
      load_q(0);
      load_do(0);
      if (n > 1) load_q(1);
      for (int i = 0; i + 1 < n; ++i) {
        if (!mbar_wait(&bar_gd, i & 1, abort_w, 11)) break;  // dV / dK MMAs of tile i done: dO and Q stage i & 1 are free
        load_do(i + 1);
        if (i + 2 < n) load_q(i + 2);
      }
    } else if (warp == 13 && lane == 0) {
      // ---------------------------------------------------------------- MMA issuer
      constexpr uint32_t idesc_st = make_idesc_bf16(128, 128, false, false);  // K-major x K-major
      constexpr uint32_t idesc_g = make_idesc_bf16(128, D, false, true);      // TMEM A x MN-major B, N = D
      constexpr uint32_t idesc_dq = make_idesc_bf16(128, 128, true, true);    // MN-major A x MN-major B
      // Descriptor halves (see desc_lo / desc_hi): `hi` is shared by every operand (SBO = 1024); K-major operands
      // carry LBO 16, MN-major ones LBO 16384 (distance between the two 64-element halves of the MN extent).
      constexpr uint32_t hi = desc_hi(1024);
      const uint32_t k_kmaj = desc_lo(smem_u32(sK), 16), v_kmaj = desc_lo(smem_u32(sV), 16);
      const uint32_t q_kmaj = desc_lo(smem_u32(sQ), 16), do_kmaj = desc_lo(smem_u32(sDO), 16);
      const uint32_t q_mn = desc_lo(smem_u32(sQ), 16384), do_mn = desc_lo(smem_u32(sDO), 16384);
      const uint32_t k_mn = desc_lo(smem_u32(sK), 16384), ds_mn = desc_lo(smem_u32(sDS), 16384);
      // Shared-memory accesses of this thread (barrier waits included) queue behind the MMAs it has issued and only
      // proceed once the tensor pipe has accepted those, so every wait whose barrier is normally complete already
      // is placed one or two MMAs before the end of a group: the pipe stays fed while the wait runs.
      auto issue_st = [&](uint32_t stage) {  // S^T = K Q^T, then tell the compute warps
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = ((kk >> 2) * 16384 + (kk & 3) * 32) >> 4;
          mma_ss2(tST, k_kmaj + off, hi, q_kmaj + stage + off, hi, idesc_st, kk > 0);
        }
        mma_commit(&bar_s[0]);
        mma_commit(&bar_s[1]);
      };
      constexpr uint32_t idesc_st64 = make_idesc_bf16(128, 64, false, false);
      auto issue_st_half = [&](uint32_t stage, int hq) {  // S^T[:, 64 hq, +64) = K Q[64 hq, +64)^T  (N = 64)
        const uint32_t rows = (uint32_t)hq * (kSubQ * 128) >> 4;  // 64 query rows x 128 B of the K-major Q tile
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = ((kk >> 2) * 16384 + (kk & 3) * 32) >> 4;
          mma_ss2(tST + 64 * hq, k_kmaj + off, hi, q_kmaj + stage + rows + off, hi, idesc_st64, kk > 0);
        }
        mma_commit(&bar_s[hq]);
      };
      auto issue_dpt = [&]() {  // dP^T = V dO^T
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = ((kk >> 2) * 16384 + (kk & 3) * 32) >> 4;
          mma_ss2(tDPT, v_kmaj + off, hi, do_kmaj + off, hi, idesc_st, kk > 0);
        }
        mma_commit(&bar_st);
      };
      auto issue_dqt = [&]() {  // dQ^T = K^T dS^T   (K = 128 keys; M = D, padded to 128 lanes when D = 64)
#pragma unroll
        for (int kk = 0; kk < kTile / 16; ++kk) mma_ss2(tDPT, k_mn + kk * 128, hi, ds_mn + kk * 128, hi, idesc_dq, kk > 0);
        mma_commit(&bar_g);
      };
      // Order per tile i: dV/dK(i) half 0, half 1 | S^T(i+1) | dQ^T(i) | (dQ^T(i) read out) dP^T(i+1).
      // S^T of the next tile goes first so that the compute warps can do the exponentials of tile i+1 while the
      // tensor core is busy with dQ^T(i), its read-out and dP^T(i+1).  S^T(i+1) overwrites the P^T / dS^T columns of
      // tile i; their readers, the dV / dK MMAs of tile i, were issued before it by this thread and the tensor pipe
      // executes one thread's MMAs in issue order.
      bool ok = mbar_wait(&bar_kv, 0, abort_w, 21) && mbar_wait(&bar_q_full[0], 0, abort_w, 22);
      if (ok) {
        tc_fence_after();
        issue_st(0u);
        ok = mbar_wait(&bar_do_full, 0, abort_w, 27);
        if (ok) issue_dpt();
      }
      for (int i = 0; i < n && ok; ++i) {
        const int st = i & 1;
        const uint32_t stage = ((uint32_t)st * Cfg::kTileBytes) >> 4;
        const uint32_t next = ((uint32_t)(st ^ 1) * Cfg::kTileBytes) >> 4;
        const bool more = i + 1 < n;
        bool fail = false;
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          if (!mbar_wait(&bar_pds[s], i & 1, abort_w, 24)) { fail = true; break; }
          tc_fence_after();
          TRACE(0, i, 3 + s);
          const uint32_t half_rows = (uint32_t)s * (kSubQ * 128) >> 4;  // 64 query rows x 128 B
          const uint32_t acc = (i > 0 || s > 0) ? 1u : 0u;
#pragma unroll
          for (int kk = 0; kk < kSubQ / 16; ++kk)  // dV += P^T dO   (K = 64 queries of this half)
            mma_ts2(tDV, tST + 64 * s + (kk >> 1) * 32 + (kk & 1) * 8, do_mn + half_rows + kk * 128, hi, idesc_g, kk > 0 ? 1u : acc);
#pragma unroll
          for (int kk = 0; kk < kSubQ / 16; ++kk)  // dK += dS^T Q
            mma_ts2(tDK, tST + 64 * s + (kk >> 1) * 32 + 16 + (kk & 1) * 8, q_mn + stage + half_rows + kk * 128, hi, idesc_g, kk > 0 ? 1u : acc);
#if TS2TS_BWD_SPLIT_ST && !defined(TS2TS_STRICT_ORDER)
          if (s == 0 && more) {
            // The first half of S^T(i+1) overwrites the P^T / dS^T columns of half 0 of tile i, whose readers were
            // issued just above: it runs while the compute warps still work on half 1, so that their exponentials of
            // tile i+1 can start the moment they are done with tile i.
            if (!mbar_wait(&bar_q_full[st ^ 1], ((i + 1) >> 1) & 1, abort_w, 22)) { fail = true; break; }
            tc_fence_after();
            issue_st_half(next, 0);
          }
#endif
        }
        if (fail) break;
        mma_commit(&bar_gd);
#ifdef TS2TS_STRICT_ORDER
        issue_dqt();
        TRACE(0, i, 5);
        if (more) {
          if (!mbar_wait(&bar_q_full[st ^ 1], ((i + 1) >> 1) & 1, abort_w, 22)) break;
          if (!mbar_wait(&bar_g, i & 1, abort_w, 26)) break;  // every MMA of tile i complete before S^T(i+1) is issued
          tc_fence_after();
          issue_st(next);
        }
#else
#if TS2TS_BWD_SPLIT_ST && TS2TS_BWD_DQ_FIRST
        issue_dqt();  // its read-out by the reduction warps then overlaps the second half of S^T(i+1)
        TRACE(0, i, 5);
#endif
        if (more) {
#if TS2TS_BWD_SPLIT_ST
          issue_st_half(next, 1);
#else
          if (!mbar_wait(&bar_q_full[st ^ 1], ((i + 1) >> 1) & 1, abort_w, 22)) break;
          tc_fence_after();
          issue_st(next);
#endif
          TRACE(0, i, 0);
        }
#if !(TS2TS_BWD_SPLIT_ST && TS2TS_BWD_DQ_FIRST)
        issue_dqt();
        TRACE(0, i, 5);
#endif
#endif
        if (more) {
          if (!mbar_wait(&bar_dqr, i & 1, abort_w, 23)) break;  // dQ^T(i) read out of the columns dP^T(i+1) overwrites
          if (!mbar_wait(&bar_do_full, (i + 1) & 1, abort_w, 27)) break;
          tc_fence_after();
          TRACE(0, i, 1);
          issue_dpt();
          TRACE(0, i, 2);
        }
      }
    }
  } else if (warp < 8) {
    // ------------------------------------------------------------------ exp / dS warps: thread = (key row, 32 of 64 queries)
#if TS2TS_BWD_LD2
    // register pool: 256 x 128 (these warps keep the launch value) + 128 x 168 + 128 x 88 = 512 x 128
#else
    reg_dec<120>();
#endif
    const int row = tid & (kTile - 1), half = tid >> 7;
    const int kv = kb * kTile + row;
    const bool kv_valid = kv < P.T;
    KeyCtx key;
    key.kvdoc = kv_valid ? p.mask.doc[(size_t)b * P.T + kv] : INT32_MIN;
    key.kvcol = kv_valid ? p.mask.col[(size_t)b * P.T + kv] : -1;
    key.mode = 0;
    key.lt0 = key.lt1 = key.lt2 = key.lt3 = 0ull;
    key.lt_row = nullptr;
    key.link_col = nullptr;
    if (p.mask.link != nullptr && key.kvcol >= 0 && key.kvcol < 64 * p.mask.W) {
      const int t_rows = P.status[kLinkTRows];
      if (t_rows == p.mask.R && key.kvcol < kLinkTMaxCols) {
        key.lt_row = P.link_t + ((size_t)b * kLinkTMaxCols + key.kvcol) * kLinkTWords;
        if (t_rows <= 256) {
          key.mode = 1;
          key.lt0 = __ldg(key.lt_row);
          if (t_rows > 64) key.lt1 = __ldg(key.lt_row + 1);
          if (t_rows > 128) key.lt2 = __ldg(key.lt_row + 2);
          if (t_rows > 192) key.lt3 = __ldg(key.lt_row + 3);
        } else {
          key.mode = 2;
        }
      } else {
        key.mode = 3;
        key.link_col = p.mask.link + (size_t)b * p.mask.R * p.mask.W + (key.kvcol >> 6);
      }
    }
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    bool ok = true;
    BTRACE_ACC_DECL
    for (int i = 0; i < n && ok; ++i) {
      const int st = i & 1;
      const int entry = list[i];
      const int qb = min(entry & ~kFullBit, NB - 1);
      const bool masked = (entry & kFullBit) == 0;
      if (!(ok = mbar_wait(&bar_q_full[st], (i >> 1) & 1, abort_w, 30))) break;  // Q, -lse2, -delta and staged runs of this tile landed
      uint32_t bits[4] = {0, 0, 0, 0};
      if (masked) {
        allowed_rows(P, p.mask, b, qb, key, s_runs + st * kRunSlotsB, s_nruns[st], bits);
        if (!kv_valid) bits[0] = bits[1] = bits[2] = bits[3] = 0u;
        if (kb == qb) {  // causal inside the diagonal tile: query rows row..127
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            const int lo = row - 32 * w;
            bits[w] &= lo <= 0 ? 0xffffffffu : (lo >= 32 ? 0u : ~((1u << lo) - 1u));
          }
        }
      }
      // per 32-query chunk of this thread, uniform over the warp: 0 all allowed, 1 test bits, 2 nothing allowed
      int mode[2] = {0, 0};
      uint32_t bw2[2] = {0xffffffffu, 0xffffffffu};
      if (masked) {
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          bw2[s] = s == 0 ? (half == 0 ? bits[0] : bits[1]) : (half == 0 ? bits[2] : bits[3]);
          mode[s] = __all_sync(0xffffffffu, bw2[s] == 0u) ? 2 : (__all_sync(0xffffffffu, bw2[s] == 0xffffffffu) ? 0 : 1);
        }
      }
      if (masked) BTRACE_ACC(0); else BTRACE_ACC(1);
      // ---- phase 1: exponentials, as soon as the half of S^T is complete
      if (!(ok = mbar_wait(&bar_s[0], i & 1, abort_w, 35))) break;
      tc_fence_after();
      BTRACE_ACC(2);
      if (tid == 0) TRACE(1, i, 0);
      uint32_t pk[2][16];
      {
        uint32_t sv[2][32];
#if TS2TS_BWD_LD2
        tmem_ld32(tST + lane_base + 32 * half, sv[0]);
        tmem_ld32(tST + lane_base + 64 + 32 * half, sv[1]);
        tmem_ld_wait();
#endif
#pragma unroll
        for (int s = 0; s < 2; ++s) {
#if !TS2TS_BWD_LD2
          if (s == 1) {
            if (!(ok = mbar_wait(&bar_s[1], i & 1, abort_w, 36))) break;
            tc_fence_after();
          }
          tmem_ld32(tST + lane_base + 64 * s + 32 * half, sv[s]);
          tmem_ld_wait();
#endif
          p_chunk(sv[s], s_lse2[st] + s * kSubQ + 32 * half, bw2[s], mode[s], p.scale_log2, pk[s]);
          tmem_st16(tST + lane_base + 64 * s + 32 * half, pk[s]);
        }
      }
      if (!ok) break;
      if (tid == 0) TRACE(1, i, 1);
      BTRACE_ACC(3);
      // ---- phase 2: dS^T, once dP^T is complete
      if (!(ok = mbar_wait(&bar_st, i & 1, abort_w, 31))) break;
      tc_fence_after();
      BTRACE_ACC(4);
      if (tid == 0) TRACE(1, i, 2);
      {
        uint32_t dp[2][32];
#if TS2TS_BWD_LD2
        tmem_ld32(tDPT + lane_base + 32 * half, dp[0]);
        tmem_ld32(tDPT + lane_base + 64 + 32 * half, dp[1]);
        tmem_ld_wait();
#endif
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          const uint32_t col = lane_base + 64 * s + 32 * half;
#if !TS2TS_BWD_LD2
          tmem_ld32(tDPT + col, dp[s]);
          tmem_ld_wait();
#endif
          uint32_t dsk[16];
          ds_chunk(pk[s], dp[s], s_delta[st] + s * kSubQ + 32 * half, mode[s], dsk);
          tmem_st16(tST + col + 16, dsk);
          // dS^T row `row`, queries [64 s + 32 half, +32): four 16-byte chunks of the 128-byte row of half s
          uint8_t* ds_row = sDS + s * 16384;
#pragma unroll
          for (int g = 0; g < 4; ++g)
            *reinterpret_cast<uint4*>(ds_row + sw128_offset(row, 4 * half + g)) = make_uint4(dsk[g * 4 + 0], dsk[g * 4 + 1], dsk[g * 4 + 2], dsk[g * 4 + 3]);
          tmem_st_wait();
          fence_async_smem();
          tc_fence_before();
#if TS2TS_BWD_ELECT
          __syncwarp();
          if (lane == 0) mbar_arrive(&bar_pds[s]);
#else
          mbar_arrive(&bar_pds[s]);
#endif
          if (tid == 0) TRACE(1, i, 3 + 4 * s);
        }
      }
      BTRACE_ACC(5);
    }
    // ---- epilogue: dV (query-half 0 threads) and scale * dK (half 1) -> bf16 -> swizzled smem -> TMA stores.
    //      dV goes through the Q stage the last tile did not use, dK through the dO buffer (its last readers, the
    //      dV MMAs of the last tile, completed before bar_g).
    const int est = n & 1;
    if (ok) ok = mbar_wait(&bar_g, (n - 1) & 1, abort_w, 32);
    tc_fence_after();
    uint8_t* out_dv = sQ + est * Cfg::kTileBytes;
    uint8_t* out_dk = sDO;
    if (ok) {
      const uint32_t tsrc = half == 0 ? tDV : tDK;
      uint8_t* stage = half == 0 ? out_dv : out_dk;
      const float f = half == 0 ? 1.f : p.scale;
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
          *reinterpret_cast<uint4*>(stage + (chunk >> 3) * 16384 + sw128_offset(row, chunk & 7)) = v;
        }
      }
      fence_async_smem();
      mbar_arrive(&bar_epi);
    }
    if (tid == 0 && ok && mbar_wait(&bar_epi, 0, abort_w, 33)) {
      for (int s = 0; s < Cfg::kSub; ++s) {
        tma_store_4d(&mapDV, out_dv + s * 16384, s * 64, kb * kTile, h, b);
        tma_store_4d(&mapDK, out_dk + s * 16384, s * 64, kb * kTile, h, b);
      }
      tma_store_commit();
      tma_store_wait_all();
    }
    BTRACE_ACC(6);
    if ((tid & 127) == 0) BTRACE_ACC_DUMP();
  } else {
    // ------------------------------------------------------------------ dQ reduction warps 8-11, thread = head-dim lane
    reg_inc<168>();
    const int dlane = tid - 2 * kTile;  // 0..127 = TMEM lane = index into D
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    // Each warp owns the 32 head-dim lanes d/32 of the dQ tile and two private 128-byte-swizzled fp32 boxes of
    // [32 queries x 32 floats] in shared memory.  The tile leaves in four rounds of 32 queries: store a round into
    // one box, hand it to a TMA reduce-add, and store the next round into the other box while the first is read.
    // Nothing else in the CTA waits for these reads.
    const int box = dlane >> 5, chunk = (dlane & 31) >> 2, word = dlane & 3;
    const bool has_box = box * 32 < D;
    uint8_t* my_stage = sStage + (warp & 3) * 8192;
    bool ok = true;
    for (int i = 0; i < n; ++i) {
      const int qb = list[i] & ~kFullBit;
      if (!(ok = mbar_wait(&bar_g, i & 1, abort_w, 41))) break;
      tc_fence_after();
      if (tid == 2 * kTile) TRACE(2, i, 0);
      uint32_t r[2][64];
      tmem_ld64(tDPT + lane_base, r[0]);
      tmem_ld64(tDPT + lane_base + 64, r[1]);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(&bar_dqr);  // the dP^T / dQ^T columns may be overwritten once all four warps have arrived
      if (tid == 2 * kTile) TRACE(2, i, 1);
      if (!has_box) continue;
      if (tid == 2 * kTile) TRACE(2, i, 3);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        uint8_t* buf = my_stage + (k & 1) * 4096;
        // the box was last used two rounds ago: at most the previous round may still be reading
        if (lane == 0) tma_store_wait_read1();
        __syncwarp();
        uint8_t* base = buf + word * 4;
#pragma unroll
        for (int c = 0; c < 32; ++c)
          *reinterpret_cast<float*>(base + c * 128 + ((chunk ^ (c & 7)) << 4)) = __uint_as_float(r[k >> 1][32 * (k & 1) + c]) * p.scale;
        fence_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_reduce_add_4d(&mapDQ, buf, box * 32, qb * kTile + 32 * k, h, b);
          tma_store_commit();
        }
      }
      if (tid == 2 * kTile) TRACE(2, i, 4);
    }
    if (lane == 0 && has_box) tma_store_wait_all();
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_ptr != 0) {
    if (tid == 0) atomicCAS(P.status, 0, 2000 + *abort_ptr);
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  if (warp == 13) tmem_dealloc(tmem, 512);
}

// One warp per (b, h, t): the negated statistics -delta and -lse2.  Rows t >= T of the padded arrays get
// -lse2 = -inf (P = 0) and delta = 0.
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
  float acc = 0.f, l2 = CUDART_INF_F;  // stored negated below: -lse2 (so -inf where P must be 0) and -delta
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
    lse2[row] = -l2;
    delta[row] = -acc;
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
  CUtensorMap mq, mk, mv, mdo, mdk, mdv, mdq;
  int r;
  if ((r = cached_tile_map(&mq, q, 2, B, H, T, D, sq[0], sq[1], sq[2], kTile, 64))) return r;
  if ((r = cached_tile_map(&mk, k, 2, B, H, T, D, sk[0], sk[1], sk[2], kTile, 64))) return r;
  if ((r = cached_tile_map(&mv, v, 2, B, H, T, D, sv[0], sv[1], sv[2], kTile, 64))) return r;
  if ((r = cached_tile_map(&mdo, dout, 2, B, H, T, D, sdo[0], sdo[1], sdo[2], kTile, 64))) return r;
  if ((r = cached_tile_map(&mdk, dk, 2, B, H, T, D, sdk[0], sdk[1], sdk[2], kTile, 64))) return r;
  if ((r = cached_tile_map(&mdv, dv, 2, B, H, T, D, sdv[0], sdv[1], sdv[2], kTile, 64))) return r;
  if ((r = cached_tile_map(&mdq, dq_acc, 4, B, H, Tp, D, (int64_t)H * Tp * D, (int64_t)Tp * D, D, 32, 32))) return r;
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
  {  // heads per group: their Q and dO (2 x T x D bf16 each) stay within TS2TS_BWD_GROUP_MB, a quarter of the L2
    const long long qdo_bytes = 4ll * T * D;
    long long g = (static_cast<long long>(TS2TS_BWD_GROUP_MB) << 20) / (qdo_bytes > 0 ? qdo_bytes : 1);
    p.head_group = (int)(g < 1 ? 1 : (g > H ? H : g));
  }
  BTRACE_ATTACH(p, stream);
  {
    ProfileScope timed(1, stream);
    attn_bwd_kernel<D><<<(unsigned)B * H * P.NB, kBwdThreads, BwdSmem<D>::kBytes, stream>>>(mq, mk, mv, mdo, mdk, mdv, mdq, p);
  }
  const int64_t n8 = (int64_t)B * H * T * (D / 8);
  dq_convert_kernel<D><<<(unsigned)((n8 + 255) / 256), 256, 0, stream>>>(dq_acc, static_cast<__nv_bfloat16*>(dq), sdq[0], sdq[1],
                                                                         sdq[2], B, H, T, Tp);
  BTRACE_DUMP(stream);
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

// --------------------------------------------------------------------------------------------------------------
// Scratch that lives inside the library, for ts2ts_attn_bwd_noalloc (see include/ts2ts_attn.h).
//
// `g_static_scratch` is a device array.  Host code must not use the name as a pointer: on the host it is only a
// handle, and a kernel handed that handle would read or write unrelated memory.  The device address is asked for
// once per device with cudaGetSymbolAddress, with that device current, and cached.
constexpr size_t kStaticScratchBytes = size_t(64) << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

int bwd_static_scratch(void** ptr, size_t* bytes) {
  static void* cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -130;
  if (cached[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || p == nullptr) return -131;
    cached[dev] = p;
  }
  *ptr = cached[dev];
  *bytes = kStaticScratchBytes;
  return 0;
}

}  // namespace ts2ts
