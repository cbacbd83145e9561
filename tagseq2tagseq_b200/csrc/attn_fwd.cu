// Masked flash-attention forward for sm_100a.
//
// Persistent kernel, one CTA per SM.  A work item is a pair of adjacent 128-row query tiles (2p, 2p+1) of one
// (batch, head); CTAs draw items from a ticket counter in the order the pre-pass wrote (heads one after the
// other, inside a head the pairs with the most key tiles first), so the tiles that run at the same time share
// K/V in L2 and the long items start early.  Each query tile of the pair belongs to a "team":
//   softmax team t   4 warps, one thread per query row (setmaxnreg 216)
//   issuer t         1 thread issuing the team's tcgen05.mma
// and one producer thread feeds both teams with TMA.  Both teams walk the same ascending stream of key tiles (the
// union of their two lists; a team simply does nothing for a tile only the other one reads), so every K/V tile is
// brought into shared memory once per pair.  Per key tile and team:
//   tcgen05   S = Q K^T                       (bf16 x bf16 -> fp32, 128 columns of tensor memory)
//   softmax   the row's 128 scores are read into registers in one go and the S columns are handed back at
//             once, so that the issuer can compute S of the NEXT key tile while this one is being exponentiated;
//             mask (partial tiles only: one select per element against a per-row 128-bit column mask built from
//             the tile's runs; 32-column chunks that are masked for a whole warp are skipped), online softmax in
//             base 2, P -> bf16 -> shared memory (K-major, 128-byte swizzle)
//   tcgen05   O += P V                        (both operands from shared memory, V MN-major)
// The accumulator is rescaled lazily: only when a row's running maximum grows by more than 2^8.
// K/V tiles travel through one ring of shared-memory slots in the order K0, K1, V0, K2, V1, ... (K runs one tile
// ahead of V because S is computed one tile ahead of P V).  At the end of an item each softmax thread reads its
// row of O out of tensor memory, frees it for the next item and writes the normalised row straight to global
// memory, while the issuers already work on the next item.
//
// Tensor memory: S0 | S1 | O0 | O1 = 512 columns.  Shared memory at D = 128: Q0 Q1 (64 KB), P0 P1 (64 KB),
// three K/V slots (96 KB).
//
// Computes what the reference obtains from PyTorch FlexAttention's forward
// (model/modules/layer.py:33 via tunalab FlexSelfAttention; semantics in
// torch/_higher_order_ops/flex_attention.py:218-287): O = softmax(scale QK^T +
// mask) V, LSE in natural log, a fully masked row gives O = 0 and LSE = -inf.
#include "plan.h"
#include "profile.h"
#include "ptx.cuh"
#include "tma_host.h"

#include <limits.h>
#include <math_constants.h>

#include <type_traits>

// A debug build may name a private header that defines the three hooks below to record clock64() stamps.
#ifdef TS2TS_TRACE_HEADER
#include TS2TS_TRACE_HEADER
#else
#define TS2TS_TRACE_FIELDS
#define FTRACE(role, step, ev) do { } while (0)
#define FTRACE_SPAN(which) do { } while (0)
#define FTRACE_CTA(slot, value) do { } while (0)
#define FTRACE_ACC_DECL
#define FTRACE_ACC(k) do { } while (0)
#define FTRACE_ACC_DUMP(team) do { } while (0)
#define FTRACE_ATTACH(params, stream) do { } while (0)
#define FTRACE_DUMP(stream) do { } while (0)
#endif

#ifndef TS2TS_FWD_GROUP_MB
// K/V bytes of the heads whose work items are interleaved in the ticket order.  Measured on the 32k masks: 136 MB
// (8 heads) is 5-7 % faster than 64 MB on the two sparser masks, equal on the densest, 2 % slower on plain causal.
#define TS2TS_FWD_GROUP_MB 136
#endif

namespace ts2ts {

struct FwdParams {
  PlanView plan;
  MaskArgs mask;
  float* lse;            // [B,H,T]
  __nv_bfloat16* out;
  int64_t o_sb, o_sh, o_st;
  int H;
  int n_items;           // B * H * ceil(NB / 2)
  int head_group;        // heads whose items are interleaved in the ticket order
  float scale_log2;      // softmax scale * log2(e)
  TS2TS_TRACE_FIELDS
};

constexpr int kFwdThreads = 384;   // warps 0-3 softmax team 0, 4-7 team 1, 8-9 MMA issuers, 10 TMA producer, 11 idle
constexpr int kFwdIssuerWarp = 8;  // + team
constexpr int kFwdProducerWarp = 10;
constexpr int kFwdItemSlots = 2;
template <uint32_t N> __device__ __forceinline__ void fwd_reg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <uint32_t N> __device__ __forceinline__ void fwd_reg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }
constexpr float kRescaleThreshold = 8.0f;
#ifndef TS2TS_FWD_X2
#define TS2TS_FWD_X2 1
#endif
#ifndef TS2TS_FWD_DUAL
#define TS2TS_FWD_DUAL 1
#endif
constexpr int kRunSlots = 8;  // runs of a partial tile that travel through shared memory; further ones are read from global memory
// Barrier among the 128 threads of softmax team t (hardware barrier 1 + t; barrier 0 is __syncthreads).
__device__ __forceinline__ void team_sync(int t) {
  if (t == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
  else asm volatile("bar.sync 2, 128;" ::: "memory");
}

template <int D>
struct FwdSmem {
  static constexpr int kSub = D / 64;
  static constexpr int kTileBytes = kTile * D * 2;
  static constexpr int kPBytes = kTile * kTile * 2;
  static constexpr int kStages = D == 128 ? 3 : 6;
  static constexpr int kQ = 0;                               // two Q tiles
  static constexpr int kP = 2 * kTileBytes;                  // two P tiles
  static constexpr int kRing = kP + 2 * kPBytes;             // K/V slots
  static constexpr int kSmall = kRing + kStages * kTileBytes;
  static constexpr int kBars = 18 + 2 * kStages;
  static constexpr int kSmallBytes = kBars * 8 + 16 + 4 * kStages + 8 + 8 * kRunSlots * 16;  // barriers, words, run copies
  static constexpr int kBytes = kSmall + kSmallBytes + 1024;  // + alignment slack
};

// One work item, decoded from its ticket number by every role on its own.
struct FwdItem {
  int b, h, qb0;
  int n[2];
  const int32_t* list[2];
};
// Ticket order: batch elements one after the other; inside one, groups of G heads; inside a group all heads' heaviest
// pairs first, then their second heaviest, and so on.  The group bounds the K/V working set that has to stay in L2,
// and the long items of the last group still start well before the end of the launch.
__device__ __forceinline__ void decode_item(const PlanView& P, int H, int G, int code, FwdItem& it) {
  const int NP = (P.NB + 1) / 2;
  const int per_b = H * NP;
  it.b = code / per_b;
  const int r1 = code - it.b * per_b;
  const int g = r1 / (G * NP);
  const int r2 = r1 - g * G * NP;
  const int gsize = min(G, H - g * G);
  const int rank = r2 / gsize;
  it.h = g * G + (r2 - rank * gsize);
  const int pair = min(max(__ldg(&P.pair_order[(size_t)it.b * NP + rank]), 0), NP - 1);
  it.qb0 = 2 * pair;
  const size_t row0 = (size_t)it.b * P.NB + it.qb0;
  it.n[0] = min(max(__ldg(&P.fwd_cnt[row0]), 0), P.NB);
  it.list[0] = P.fwd_idx + row0 * P.NB;
  if (it.qb0 + 1 < P.NB) {
    it.n[1] = min(max(__ldg(&P.fwd_cnt[row0 + 1]), 0), P.NB);
    it.list[1] = it.list[0] + P.NB;
  } else {
    it.n[1] = 0;
    it.list[1] = it.list[0];
  }
}
// What a ring slot holds, written by the producer next to the slot.
enum : uint32_t {
  kRingTeam0 = 1u, kRingTeam1 = 2u,     // the tile is on the list of team 0 / 1
  kRingIsV = 4u,                        // V tile (else K)
  kRingFirst0 = 8u, kRingFirst1 = 16u,  // the team's first tile of the item
  kRingLast0 = 32u, kRingLast1 = 64u,   // the team's last tile of the item
  kRingEnd = 128u,                      // no more work
};
// Ascending merge of the two key-tile lists of an item.  next() returns the next key tile, -1 at the end, and
// -2 when an entry is not a tile number (the plan does not belong to this call); `info` gets the kRing* bits.
struct UnionWalk {
  const int32_t *l0, *l1;
  int n0, n1, i0, i1, NB;
  __device__ __forceinline__ void start(const FwdItem& it, int nb) {
    l0 = it.list[0]; l1 = it.list[1]; n0 = it.n[0]; n1 = it.n[1]; i0 = i1 = 0; NB = nb;
  }
  __device__ __forceinline__ int next(uint32_t& info) {
    const int a = i0 < n0 ? static_cast<int>(__ldg(l0 + i0) & ~kFullBit) : INT_MAX;
    const int c = i1 < n1 ? static_cast<int>(__ldg(l1 + i1) & ~kFullBit) : INT_MAX;
    const int kb = min(a, c);
    if (kb == INT_MAX) return -1;
    if (kb < 0 || kb >= NB) return -2;
    info = 0;
    if (a == kb) {
      info |= kRingTeam0 | (i0 == 0 ? kRingFirst0 : 0u) | (i0 == n0 - 1 ? kRingLast0 : 0u);
      ++i0;
    }
    if (c == kb) {
      info |= kRingTeam1 | (i1 == 0 ? kRingFirst1 : 0u) | (i1 == n1 - 1 ? kRingLast1 : 0u);
      ++i1;
    }
    return kb;
  }
};

template <int D>
__global__ void __launch_bounds__(kFwdThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapO, const FwdParams p) {
  using Cfg = FwdSmem<D>;
  constexpr int kStages = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  // Plain pointer arithmetic (no round trip through an integer) keeps the shared address space visible to the
  // compiler, so every access below becomes a shared-memory instruction instead of a generic one.
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* sQ = smem + Cfg::kQ;
  uint8_t* sP = smem + Cfg::kP;
  uint8_t* sRing = smem + Cfg::kRing;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kSmall);
  uint64_t* bar_item_full = bars;        // [2] the producer published a ticket
  uint64_t* bar_item_empty = bars + 2;   // [2] the eight softmax warps copied it
  uint64_t* bar_q_full = bars + 4;       // [team] Q tile landed
  uint64_t* bar_q_free = bars + 6;       // [team] last S of the item complete: the Q buffer may be reloaded
  uint64_t* bar_s = bars + 8;            // [team] S of the tile is in tensor memory
  uint64_t* bar_sfree = bars + 10;       // [team] S read into registers: its columns may be overwritten
  uint64_t* bar_p = bars + 12;           // [team] P of the tile is in shared memory
  uint64_t* bar_pv = bars + 14;          // [team] P V of the tile complete: P buffer free, O consistent
  uint64_t* bar_ofree = bars + 16;       // [team] O of the item read out of tensor memory
  uint64_t* bar_ring_full = bars + 18;   // [kStages] K or V tile landed in the slot
  uint64_t* bar_ring_free = bars + 18 + kStages;  // [kStages] both issuers are done with the slot
  int* s_item = reinterpret_cast<int*>(bars + Cfg::kBars);  // [2] ticket ring
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_item + 2);
  int* abort_w = s_item + 3;
  uint32_t* s_ring_info = reinterpret_cast<uint32_t*>(s_item + 4);  // [kStages] kRing* bits of what each slot holds
  int4* s_runs = reinterpret_cast<int4*>(reinterpret_cast<uint8_t*>(bars) + ((Cfg::kBars * 8 + 16 + 4 * kStages + 15) & ~15));  // [8 warps][kRunSlots]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const PlanView& P = p.plan;
  const int NB = P.NB;
  {  // uniform across the grid: refuse a plan that was not built for this (B, T), or a misplaced shared-memory window
    int bad = 0;
    if (P.status[kStampMagic] != kPlanMagic || P.status[kStampB] != P.B || P.status[kStampT] != P.T) bad = 1900;
    else if (smem + Cfg::kSmall + Cfg::kSmallBytes > smem_raw + Cfg::kBytes) bad = 1901;
    if (bad) {
      if (tid == 0) atomicCAS(P.status, 0, bad);
      return;
    }
  }

  if (tid == 0) {
    *abort_w = 0;
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar_item_full[i], 1);
      mbar_init(&bar_item_empty[i], 8);
      mbar_init(&bar_q_full[i], 1);
      mbar_init(&bar_q_free[i], 1);
      mbar_init(&bar_s[i], 1);
      mbar_init(&bar_sfree[i], 4);  // one arrival per softmax warp
      mbar_init(&bar_p[i], 4);
      mbar_init(&bar_pv[i], 1);
      mbar_init(&bar_ofree[i], 4);
    }
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&bar_ring_full[i], 1);
      mbar_init(&bar_ring_free[i], 2);
    }
    fence_mbar_init();
  }
  __syncthreads();
  if (warp == kFwdIssuerWarp) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  volatile int* abort_v = abort_w;
  if (tid == 0) FTRACE_SPAN(0);

  if (warp >= 8) {
    fwd_reg_dec<72>();  // register pool: 256 x 216 + 128 x 72 = 384 x 168
    if (warp == kFwdProducerWarp && lane == 0) {
      // ------------------------------------------------------------------ TMA producer
      // Walks the key-tile lists (the only role that reads them from global memory besides the softmax threads) and
      // tells the issuers through a word per ring slot what the slot holds and which team uses it.
      tma_prefetch_desc(&mapQ); tma_prefetch_desc(&mapK); tma_prefetch_desc(&mapV);
      uint32_t ring = 0;             // ring slots filled so far
      uint32_t q_loads[2] = {0, 0};  // Q tiles loaded so far, per team
      bool ok = true;
      auto fill = [&](const CUtensorMap* map, uint32_t info, int kb, int h, int b) {
        const uint32_t slot = ring % kStages, use = ring / kStages;
        if (use > 0 && !mbar_wait(&bar_ring_free[slot], (use - 1) & 1, abort_v, 11)) return false;
        s_ring_info[slot] = info;
        if (map != nullptr) {
          mbar_expect_tx(&bar_ring_full[slot], Cfg::kTileBytes);
          for (int s = 0; s < Cfg::kSub; ++s)
            tma_load_4d(sRing + slot * Cfg::kTileBytes + s * 16384, map, &bar_ring_full[slot], s * 64, kb * kTile, h, b);
        } else {
          mbar_arrive(&bar_ring_full[slot]);  // end marker: nothing to load
        }
        ++ring;
        return true;
      };
      for (uint32_t it = 0; ok; ++it) {
        const uint32_t is = it % kFwdItemSlots;
        if (it >= kFwdItemSlots && !mbar_wait(&bar_item_empty[is], (it / kFwdItemSlots - 1) & 1, abort_v, 12)) break;
        const int ticket = atomicAdd(&P.status[kFwdTicket], 1);
        const int code = ticket < p.n_items ? ticket : -1;
        s_item[is] = code;
        mbar_arrive(&bar_item_full[is]);
        if (code < 0) {
          fill(nullptr, kRingEnd, 0, 0, 0);
          break;
        }
        FwdItem item;
        decode_item(P, p.H, p.head_group, code, item);
        for (int t = 0; t < 2 && ok; ++t) {
          if (item.n[t] == 0) continue;
          if (q_loads[t] > 0 && !mbar_wait(&bar_q_free[t], (q_loads[t] - 1) & 1, abort_v, 13)) { ok = false; break; }
          mbar_expect_tx(&bar_q_full[t], Cfg::kTileBytes);
          for (int s = 0; s < Cfg::kSub; ++s)
            tma_load_4d(sQ + t * Cfg::kTileBytes + s * 16384, &mapQ, &bar_q_full[t], s * 64, (item.qb0 + t) * kTile, item.h, item.b);
          ++q_loads[t];
        }
        if (!ok) break;
        UnionWalk w;
        w.start(item, NB);
        uint32_t cur_info = 0, nxt_info = 0;
        int cur = w.next(cur_info);
        if (cur == -2) { atomicCAS(abort_w, 0, 14); break; }
        if (cur >= 0) ok = fill(&mapK, cur_info, cur, item.h, item.b);
        while (cur >= 0 && ok) {
          const int nxt = w.next(nxt_info);
          if (nxt == -2) { atomicCAS(abort_w, 0, 14); ok = false; break; }
          if (nxt >= 0) ok = fill(&mapK, nxt_info, nxt, item.h, item.b);
          if (ok) ok = fill(&mapV, cur_info | kRingIsV, cur, item.h, item.b);
          cur = nxt;
          cur_info = nxt_info;
        }
      }
    } else if ((warp == kFwdIssuerWarp || warp == kFwdIssuerWarp + 1) && lane == 0) {
      // ------------------------------------------------------------------ MMA issuer of team t
      // Takes the ring slots in order: waits until a slot is filled, uses it if the tile is on this team's list
      // (S = Q K^T for a K slot, O += P V for a V slot) and hands it back.  It reads shared memory only.
      const int t = warp - kFwdIssuerWarp;
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(128, D, false, true);
      // descriptor halves: K-major operands (Q, K, P) step 32 B inside a 128-byte row and 16 KB between two
      // 64-column halves; the MN-major operand (V) steps 16 key rows = 2048 B
      constexpr uint32_t hi_k = desc_hi(1024);
      const uint32_t q_lo = desc_lo(smem_u32(sQ + t * Cfg::kTileBytes), 16);
      const uint32_t p_lo = desc_lo(smem_u32(sP + t * Cfg::kPBytes), 16);
      const uint32_t k_ring_lo = desc_lo(smem_u32(sRing), 16), v_ring_lo = desc_lo(smem_u32(sRing), 16384);
      const uint32_t tS = tmem + t * kTile;
      const uint32_t tO = tmem + 2 * kTile + t * D;
      const uint32_t mine_bit = kRingTeam0 << t, first_bit = kRingFirst0 << t, last_bit = kRingLast0 << t;
      uint32_t n_s = 0;      // S tiles issued by this team so far
      uint32_t n_pv = 0;     // P V tiles issued so far
      uint32_t n_items = 0;  // items this team has started
      for (uint32_t ring = 0;; ++ring) {
        const uint32_t slot = ring % kStages, use = ring / kStages;
        if (!mbar_wait(&bar_ring_full[slot], use & 1, abort_v, 23)) break;
        const uint32_t info = s_ring_info[slot];
        if (info & kRingEnd) break;
        if (!(info & mine_bit)) {
          mbar_arrive(&bar_ring_free[slot]);
          continue;
        }
        if (!(info & kRingIsV)) {
          if ((info & first_bit) && !mbar_wait(&bar_q_full[t], n_items & 1, abort_v, 22)) break;
          if (info & first_bit) ++n_items;
          if (n_s > 0 && !mbar_wait(&bar_sfree[t], (n_s - 1) & 1, abort_v, 24)) break;
          tc_fence_after();
          FTRACE(2 * t, n_s, 0);
          const uint32_t k_lo = k_ring_lo + slot * (Cfg::kTileBytes >> 4);
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t off = ((kk >> 2) * 16384 + (kk & 3) * 32) >> 4;
            mma_ss2(tS, q_lo + off, hi_k, k_lo + off, hi_k, idesc_s, kk > 0);
          }
          mma_commit(&bar_s[t]);
          FTRACE(2 * t, n_s, 1);
          ++n_s;
          if (info & last_bit) mma_commit(&bar_q_free[t]);
          mma_commit(&bar_ring_free[slot]);
        } else {
          if (!mbar_wait(&bar_p[t], n_pv & 1, abort_v, 26)) break;
          // the first P V of an item overwrites O: the previous item's rows must have been read out
          // (n_items counts this item already, so the previous one is n_items - 2)
          if ((info & first_bit) && n_items > 1 && !mbar_wait(&bar_ofree[t], (n_items - 2) & 1, abort_v, 27)) break;
          tc_fence_after();
          FTRACE(2 * t, n_pv, 2);
          const uint32_t v_lo = v_ring_lo + slot * (Cfg::kTileBytes >> 4);
          const uint32_t acc0 = (info & first_bit) ? 0u : 1u;
#pragma unroll
          for (int kk = 0; kk < kTile / 16; ++kk) {
            const uint32_t off = ((kk >> 2) * 16384 + (kk & 3) * 32) >> 4;
            mma_ss2(tO, p_lo + off, hi_k, v_lo + kk * (2048 >> 4), hi_k, idesc_pv, kk > 0 ? 1u : acc0);
          }
          mma_commit(&bar_pv[t]);
          FTRACE(2 * t, n_pv, 3);
          ++n_pv;
          mma_commit(&bar_ring_free[slot]);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue: thread = query row of team t
    // One thread owns a whole score row: the row maximum and sum need no exchange between threads, and the 128
    // scores are read from tensor memory once and stay in registers, which frees the S columns for the next tile.
    fwd_reg_inc<216>();
    const int t = warp >> 2;
    const int row = tid & (kTile - 1);
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tSr = tmem + t * kTile + lane_base;
    const uint32_t tOr = tmem + 2 * kTile + t * D + lane_base;
    uint8_t* sPt = sP + t * Cfg::kPBytes;
    int4* my_runs = s_runs + warp * kRunSlots;  // this warp's copy of the current partial tile's first runs
    uint32_t n_tiles = 0;  // tiles this team has processed so far
    uint32_t n_epi = 0;    // items this team has finished
    FTRACE_ACC_DECL
    bool ok = true;
    for (uint32_t it = 0; ok; ++it) {
      const uint32_t is = it % kFwdItemSlots;
      if (!mbar_wait(&bar_item_full[is], (it / kFwdItemSlots) & 1, abort_v, 31)) break;
      const int code = s_item[is];
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar_item_empty[is]);
      if (code < 0) break;
      FwdItem item;
      decode_item(P, p.H, p.head_group, code, item);
      const int qb = item.qb0 + t;
      if (qb >= NB) continue;
      const int b = item.b, h = item.h;
      const int n = t == 0 ? item.n[0] : item.n[1];
      const int32_t* list = t == 0 ? item.list[0] : item.list[1];
      const int q = qb * kTile + row;
      const bool q_valid = q < P.T;
      if (n == 0) {  // no readable key tile: defined result, nothing to compute
        if (q_valid) {
          __nv_bfloat16* orow = p.out + (size_t)b * p.o_sb + (size_t)h * p.o_sh + (size_t)q * p.o_st;
          for (int i = 0; i < D; i += 8) *reinterpret_cast<uint4*>(orow + i) = make_uint4(0, 0, 0, 0);
          p.lse[((size_t)b * p.H + h) * P.T + q] = -CUDART_INF_F;
        }
        continue;
      }
      const int mydoc = q_valid ? p.mask.doc[(size_t)b * P.T + q] : INT32_MIN;
      const int myrow = q_valid ? p.mask.row[(size_t)b * P.T + q] : -1;
      // This row's link words stay in registers for the whole item when there are at most four of them (256 column
      // classes); a lookup is then a select, not a load.
      const int64_t* link_row = (p.mask.link != nullptr && myrow >= 0 && myrow < p.mask.R) ? p.mask.link + ((size_t)b * p.mask.R + myrow) * p.mask.W : nullptr;
      const bool link_regs = p.mask.W <= 4;
      unsigned long long lw0 = 0, lw1 = 0, lw2 = 0, lw3 = 0;
      if (link_row != nullptr && link_regs) {
        lw0 = static_cast<unsigned long long>(__ldg(link_row));
        if (p.mask.W > 1) lw1 = static_cast<unsigned long long>(__ldg(link_row + 1));
        if (p.mask.W > 2) lw2 = static_cast<unsigned long long>(__ldg(link_row + 2));
        if (p.mask.W > 3) lw3 = static_cast<unsigned long long>(__ldg(link_row + 3));
      }
      // List entries are fetched two tiles ahead and the runs of a partial tile one tile ahead (lanes 0-7 hold one run
      // each), so that their latency hides behind the sweeps of the tile before.
      int e_cur = ld_nc_i32_here(list);
      int e_nxt = n > 1 ? ld_nc_i32_here(list + 1) : 0;
      int4 r_pf = make_int4(0, 0, 0, 0);
      int n_pf = 0;
      auto prefetch_runs = [&](int entry) {
        if (entry & kFullBit) return;
        const int kbp = min(max(entry & ~kFullBit, 0), NB - 1);
        n_pf = ld_nc_i32_here(&P.run_cnt[(size_t)b * NB + kbp]);
        if (lane < kRunSlots) r_pf = ld_nc_v4_here(P.runs + ((size_t)b * NB + kbp) * kTile + lane);
      };
      prefetch_runs(e_cur);
      float m_used = -CUDART_INF_F, l = 0.f;
      FTRACE_ACC(0);
      for (int j = 0; j < n && ok; ++j) {
        const int entry = e_cur;
        e_cur = e_nxt;
#ifdef TS2TS_EXPERIMENT_NOLIST
        if (j + 2 < n) e_nxt = (j + 2) | (j + 2 < n - 1 ? kFullBit : 0);
#else
        if (j + 2 < n) e_nxt = ld_nc_i32_here(list + j + 2);
#endif
        const int kb = entry & ~kFullBit;
        if (kb < 0 || kb >= NB) { atomicCAS(abort_w, 0, 38); ok = false; break; }
        int n_runs = 0;
        if (!(entry & kFullBit)) {  // hand the prefetched runs to the whole warp
          __syncwarp();
          if (lane < kRunSlots) my_runs[lane] = r_pf;
          n_runs = min(n_pf, kTile);
          __syncwarp();
        }
        if (j + 1 < n) prefetch_runs(e_cur);
        FTRACE_ACC(7);
#if TS2TS_FWD_DUAL
        auto tile = [&](auto masked_tag) {
          constexpr bool kMasked = decltype(masked_tag)::value;
#else
        auto tile = [&](bool kMasked) {
#endif
        uint32_t bits[4] = {0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu};
        bool dead[4] = {false, false, false, false}, mixed[4] = {false, false, false, false};
        if (kMasked) {
          // 128-bit mask of the key columns this row may read, before causality: walk the tile's runs
          bits[0] = bits[1] = bits[2] = bits[3] = 0u;
          const Run* runs_g = P.runs + ((size_t)b * NB + kb) * kTile;
          const int n_valid = min(kTile, P.T - kb * kTile);
          auto get_run = [&](int r) {
            return r < kRunSlots ? my_runs[r] : __ldg(reinterpret_cast<const int4*>(runs_g + r));
          };
          int4 cur = n_runs > 0 ? get_run(0) : make_int4(0, 0, 0, 0);
          for (int r = 0; r < n_runs; ++r) {
            const int4 nx = r + 1 < n_runs ? get_run(r + 1) : make_int4(n_valid, 0, 0, 0);
            const int start = cur.x, doc = cur.y, col = cur.w, end = nx.x;
            bool allowed = doc == mydoc;
            if (!allowed && link_row != nullptr && col >= 0 && col < 64 * p.mask.W) {
              unsigned long long wbits;
              if (link_regs) {
                const int wi = col >> 6;
                wbits = wi == 0 ? lw0 : wi == 1 ? lw1 : wi == 2 ? lw2 : lw3;
              } else {
                wbits = static_cast<unsigned long long>(__ldg(link_row + (col >> 6)));
              }
              allowed = (wbits >> (col & 63)) & 1ull;
            }
            if (allowed) {
#pragma unroll
              for (int w = 0; w < 4; ++w) {
                const int lo = max(start - 32 * w, 0), hi = min(end - 32 * w, 32);
                if (hi > lo) bits[w] |= (hi - lo == 32 ? 0xffffffffu : ((1u << (hi - lo)) - 1u)) << lo;
              }
            }
            cur = nx;
          }
          if (kb == qb) {  // causal inside the diagonal tile: columns 0..row
#pragma unroll
            for (int w = 0; w < 4; ++w) {
              const int hi = row + 1 - 32 * w;
              bits[w] &= hi >= 32 ? 0xffffffffu : (hi <= 0 ? 0u : ((1u << hi) - 1u));
            }
          }
#pragma unroll
          for (int c = 0; c < 4; ++c) {  // per 32-column chunk, uniform over the warp: nothing / everything / some allowed
            dead[c] = __all_sync(0xffffffffu, bits[c] == 0u);
            mixed[c] = !dead[c] && !__all_sync(0xffffffffu, bits[c] == 0xffffffffu);
          }
        }
        if (kMasked) FTRACE_ACC(1); else FTRACE_ACC(5);
        if (row == 0) FTRACE(2 * t + 1, n_tiles, 0);
        if (!mbar_wait(&bar_s[t], n_tiles & 1, abort_v, 32)) return false;
        tc_fence_after();
        FTRACE_ACC(2);
        if (row == 0) FTRACE(2 * t + 1, n_tiles, 1);
        uint32_t sv[4][32];
        tmem_ld32(tSr, sv[0]);
        tmem_ld32(tSr + 32, sv[1]);
        tmem_ld32(tSr + 64, sv[2]);
        tmem_ld32(tSr + 96, sv[3]);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_sfree[t]);  // the issuer may now overwrite S with the next tile's scores
        if (row == 0) FTRACE(2 * t + 1, n_tiles, 2);
        // masked scores become -inf once; both sweeps below then need no mask (exp2(-inf) = 0)
#pragma unroll
        for (int c = 0; c < 4; ++c)
          if (kMasked && mixed[c]) {
#pragma unroll
            for (int i = 0; i < 32; ++i) sv[c][i] = ((bits[c] >> i) & 1u) ? sv[c][i] : 0xff800000u;
          }
        // sweep 1: row maximum (eight independent running maxima keep the dependency chain short)
        float mx8[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) mx8[i] = -CUDART_INF_F;
#pragma unroll
        for (int c = 0; c < 4; ++c)
          if (!kMasked || !dead[c]) {
#pragma unroll
            for (int i = 0; i < 16; ++i) mx8[i & 7] = fmax3(mx8[i & 7], __uint_as_float(sv[c][i]), __uint_as_float(sv[c][i + 16]));
          }
        float mx = fmax3(fmax3(mx8[0], mx8[1], mx8[2]), fmax3(mx8[3], mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7]));
        mx *= p.scale_log2;  // scale > 0, so max commutes with the scaling
        const float m_new = fmaxf(m_used, mx);
        const bool need = m_new > m_used + kRescaleThreshold || (m_used == -CUDART_INF_F && m_new > -CUDART_INF_F);
        const bool any_need = __any_sync(0xffffffffu, need);
        float factor = 1.f;
        if (any_need) {
          factor = need ? fast_exp2(m_used - m_new) : 1.f;  // exp2(-inf) = 0 on the first real tile
          l *= factor;
          if (need) m_used = m_new;
        }
        const float m_safe = m_used == -CUDART_INF_F ? 0.f : m_used;
        if (row == 0) FTRACE(2 * t + 1, n_tiles, 3);
        // sweep 2: P = exp2(s * scale - m) with packed fp32 arithmetic (two scores per instruction), row sum in
        // four partial sums, bf16 pack, P -> shared memory
        const unsigned long long scale2 = pack_f32x2(p.scale_log2, p.scale_log2), negm2 = pack_f32x2(-m_safe, -m_safe);
        unsigned long long sum2[2] = {0ull, 0ull};
        float sum4[4] = {0.f, 0.f, 0.f, 0.f};
        uint32_t pk[4][16];
        bool fine = true;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          if (!kMasked || !dead[c]) {
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
#if TS2TS_FWD_X2
              float x0, x1;
              unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(sv[c][i]), __uint_as_float(sv[c][i + 1])), scale2, negm2), x0, x1);
              const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
              sum2[(i >> 1) & 1] = add_f32x2(sum2[(i >> 1) & 1], pack_f32x2(p0, p1));
#else
              const float p0 = fast_exp2(fmaf(__uint_as_float(sv[c][i]), p.scale_log2, -m_safe));
              const float p1 = fast_exp2(fmaf(__uint_as_float(sv[c][i + 1]), p.scale_log2, -m_safe));
              sum4[(i >> 1) & 3] += p0 + p1;
#endif
              pk[c][i >> 1] = pack_bf16(p0, p1);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) pk[c][i] = 0u;
          }
          if (c == 1) {
            // P V of the previous tile must be complete before its P buffer is overwritten and before O is touched;
            // it was issued a whole sweep ago, so this wait normally falls through.
            if (row == 0) FTRACE(2 * t + 1, n_tiles, 4);
            if (n_tiles > 0) fine = mbar_wait(&bar_pv[t], (n_tiles - 1) & 1, abort_v, 33);
            if (j == 0 && n_epi > 0) {
              // the previous item's output left through this buffer: its TMA store must have read it
              if (row == 0) tma_store_wait_read0();
              team_sync(t);
            }
            if (row == 0) FTRACE(2 * t + 1, n_tiles, 5);
            if (any_need && j > 0) {
              tc_fence_after();
              const unsigned long long f2 = pack_f32x2(factor, factor);
#pragma unroll 1
              for (int cc = 0; cc < D / 32; ++cc) {
                uint32_t r[32];
                tmem_ld32(tOr + cc * 32, r);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                  float y0, y1;
                  unpack_f32x2(mul_f32x2(pack_f32x2(__uint_as_float(r[i]), __uint_as_float(r[i + 1])), f2), y0, y1);
                  r[i] = __float_as_uint(y0);
                  r[i + 1] = __float_as_uint(y1);
                }
                tmem_st32(tOr + cc * 32, r);
              }
              tmem_st_wait();
            }
          }
          if (c >= 1) {
#pragma unroll
            for (int cc = (c == 1 ? 0 : c); cc <= c; ++cc)
#pragma unroll
              for (int g = 0; g < 4; ++g)
                *reinterpret_cast<uint4*>(sPt + (cc >> 1) * 16384 + sw128_offset(row, (cc & 1) * 4 + g)) =
                    make_uint4(pk[cc][g * 4 + 0], pk[cc][g * 4 + 1], pk[cc][g * 4 + 2], pk[cc][g * 4 + 3]);
          }
        }
        if (!fine) return false;
        {
          float s0, s1, s2, s3;
          unpack_f32x2(sum2[0], s0, s1);
          unpack_f32x2(sum2[1], s2, s3);
          l += (s0 + s1) + (s2 + s3) + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
        }
        if (row == 0) FTRACE(2 * t + 1, n_tiles, 6);
        fence_async_smem();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_p[t]);
        if (row == 0) FTRACE(2 * t + 1, n_tiles, 7);
        if (kMasked) FTRACE_ACC(6); else FTRACE_ACC(3);
          return true;
        };
#if TS2TS_FWD_DUAL
        ok = (entry & kFullBit) ? tile(std::false_type{}) : tile(std::true_type{});
#else
        ok = tile(!(entry & kFullBit));
#endif
        ++n_tiles;
      }
      if (!ok) break;
      // ---- epilogue: O / l -> bf16 -> the team's P buffer (free after the last P V) -> TMA store
      if (!(ok = mbar_wait(&bar_pv[t], (n_tiles - 1) & 1, abort_v, 34))) break;
      tc_fence_after();
      {
        const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t o[32];
          tmem_ld32(tOr + c * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 v;
            v.x = pack_bf16(__uint_as_float(o[g * 8 + 0]) * inv, __uint_as_float(o[g * 8 + 1]) * inv);
            v.y = pack_bf16(__uint_as_float(o[g * 8 + 2]) * inv, __uint_as_float(o[g * 8 + 3]) * inv);
            v.z = pack_bf16(__uint_as_float(o[g * 8 + 4]) * inv, __uint_as_float(o[g * 8 + 5]) * inv);
            v.w = pack_bf16(__uint_as_float(o[g * 8 + 6]) * inv, __uint_as_float(o[g * 8 + 7]) * inv);
            const int chunk = c * 4 + g;  // 16-byte chunk index inside the output row
            *reinterpret_cast<uint4*>(sPt + (chunk >> 3) * 16384 + sw128_offset(row, chunk & 7)) = v;
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_ofree[t]);  // the next item's first P V may overwrite O
        if (q_valid) p.lse[((size_t)b * p.H + h) * P.T + q] = l > 0.f ? (m_used + log2f(l)) * 0.6931471805599453f : -CUDART_INF_F;
      }
      fence_async_smem();
      team_sync(t);
      if (row == 0) {
        for (int s = 0; s < Cfg::kSub; ++s) tma_store_4d(&mapO, sPt + s * 16384, s * 64, qb * kTile, h, b);
        tma_store_commit();
      }
      ++n_epi;
      FTRACE_ACC(4);
    }
    if (row == 0) tma_store_wait_all();  // the stores read this CTA's shared memory
    if (row == 0) FTRACE_CTA(2 + t, n_tiles);
    if (row == 0) FTRACE_ACC_DUMP(t);
  }

  tc_fence_before();
  __syncthreads();
  if (tid == 0) { FTRACE_SPAN(1); }
  if (*abort_v != 0) {
    // Let loads that were issued but never consumed land before the CTA's shared memory is released.
    if (tid == 0) atomicCAS(P.status, 0, 1000 + *abort_v);
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  if (warp == kFwdIssuerWarp) tmem_dealloc(tmem, 512);
  if (tid == 0) {  // the last CTA to leave puts the ticket counter back to zero for the next launch
    __threadfence();
    const int done = atomicAdd(&P.status[kFwdDone], 1);
    if (done == static_cast<int>(gridDim.x) - 1) {
      P.status[kFwdTicket] = 0;
      P.status[kFwdDone] = 0;
      __threadfence();
    }
  }
}

// Host launcher.  Tensor strides are in elements; the last dimension is contiguous.
template <int D>
static int launch_fwd_t(const void* q, const void* k, const void* v, void* out, float* lse, const int64_t* sq,
                        const int64_t* sk, const int64_t* sv, const int64_t* so, int B, int H, int T, float scale,
                        PlanView P, MaskArgs M, cudaStream_t stream) {
  CUtensorMap mq, mk, mv, mo;
  int r;
  if ((r = cached_tile_map(&mq, q, 2, B, H, T, D, sq[0], sq[1], sq[2], kTile, 64))) return r;
  if ((r = cached_tile_map(&mk, k, 2, B, H, T, D, sk[0], sk[1], sk[2], kTile, 64))) return r;
  if ((r = cached_tile_map(&mv, v, 2, B, H, T, D, sv[0], sv[1], sv[2], kTile, 64))) return r;
  if ((r = cached_tile_map(&mo, out, 2, B, H, T, D, so[0], so[1], so[2], kTile, 64))) return r;
  FwdParams p;
  p.plan = P; p.mask = M; p.lse = lse; p.out = static_cast<__nv_bfloat16*>(out);
  p.o_sb = so[0]; p.o_sh = so[1]; p.o_st = so[2];
  p.H = H; p.scale_log2 = scale * 1.4426950408889634f;
  const long long items = (long long)B * H * ((P.NB + 1) / 2);
  p.n_items = (int)items;
  {  // heads per group, from the K and V bytes of one head (2 x T x D bf16 each)
    const long long kv_bytes = 4ll * T * D;
    long long g = (static_cast<long long>(TS2TS_FWD_GROUP_MB) << 20) / (kv_bytes > 0 ? kv_bytes : 1);
    p.head_group = (int)(g < 1 ? 1 : (g > H ? H : g));
  }
  static bool attr_done[64] = {};
  static int sm_count[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return -110;
  if (!attr_done[dev]) {
    if (cudaFuncSetAttribute(attn_fwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdSmem<D>::kBytes) != cudaSuccess)
      return -110;
    if (cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sm_count[dev] <= 0) return -110;
    attr_done[dev] = true;
  }
  const unsigned grid = (unsigned)(items < sm_count[dev] ? items : sm_count[dev]);
  FTRACE_ATTACH(p, stream);
  {
    ProfileScope timed(0, stream);
    attn_fwd_kernel<D><<<grid, kFwdThreads, FwdSmem<D>::kBytes, stream>>>(mq, mk, mv, mo, p);
  }
  FTRACE_DUMP(stream);
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
