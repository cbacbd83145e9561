// Layout of the block plan: the device buffer that the pre-pass fills from the
// per-token mask inputs and that the attention kernels read.  One plan serves
// every head and every layer of a micro-batch (the reference builds one
// BlockMask per micro-batch and broadcasts it, block_mask_creator.py:132-139).
//
// All tiles are 128 tokens.  NB = ceil(T / 128).
#pragma once
#include <stddef.h>
#include <stdint.h>

namespace ts2ts {

constexpr int kTile = 128;

enum : uint8_t { kSkip = 0, kPartial = 1, kFull = 2 };

// A run is a maximal stretch of tokens inside one tile whose (doc id, row class,
// column class) triple is constant.  `start` is the offset inside the tile.
struct alignas(16) Run {
  int32_t start, doc, row, col;
};

constexpr uint32_t kFullBit = 1u << 30;  // set in merged list entries for full tiles

// Words of the status block.  Word 0 holds the first device error code.  The stamp is written by the pre-pass and
// compared by every attention kernel with its own B and T before it touches a list.  The ticket / done words are
// the work counters of the persistent attention kernels: a CTA draws work items from `ticket`; the last CTA to
// leave (counted in `done`) puts both back to zero, so launches that share a plan must be ordered on one stream.
enum : int {
  kStatusCode = 0, kStampMagic = 1, kStampB = 2, kStampT = 3,
  kFwdTicket = 8, kFwdDone = 9, kBwdTicket = 10, kBwdDone = 11,
  kLinkTRows = 12,  // > 0: link_t holds the transposed link bits of this many row classes
};
// Transposed link bits: word w of column class c holds, in bit r % 64, whether row class 64 w + r may read c.  A
// backward thread owns one key, i.e. one column class, and tests many row classes against it; with the transposed
// table its words are loaded once per CTA.  The table exists when R <= kLinkTMaxRows and 64 W <= kLinkTMaxCols.
constexpr int kLinkTMaxRows = 1024, kLinkTMaxCols = 1024, kLinkTWords = kLinkTMaxRows / 64;
constexpr int32_t kPlanMagic = 0x54533254;  // "TS2T"

struct PlanLayout {
  int B, T, NB;
  size_t status;      // int32[64]   see the kStatus* / kStamp* / k*Ticket words above
  size_t run_cnt;     // int32[B,NB]
  size_t runs;        // Run[B,NB,128]
  size_t state;       // uint8[B,NB,NB]   state[b,qb,kb]
  size_t fwd_cnt;     // int32[B,NB]      non-skipped kv tiles of q tile qb
  size_t fwd_idx;     // int32[B,NB,NB]   ascending kb, kFullBit set when full
  size_t bwd_cnt;     // int32[B,NB]      non-skipped q tiles of kv tile kb
  size_t bwd_idx;     // int32[B,NB,NB]   ascending qb, kFullBit set when full
  size_t fwd_order;   // int32[B,NB]      q tiles of batch b by descending fwd_cnt
  size_t bwd_order;   // int32[B,NB]      kv tiles of batch b by descending bwd_cnt
  size_t pair_cnt;    // int32[B,NP]      NP = ceil(NB/2): kv tiles that q tile 2p or 2p+1 reads (forward work items)
  size_t pair_order;  // int32[B,NP]      pairs of batch b by descending pair_cnt
  size_t link_t;      // uint64[B,kLinkTMaxCols,kLinkTWords]   transposed link bits (see kLinkTRows)
  size_t bytes;
};

inline size_t plan_align(size_t x) { return (x + 255) & ~size_t(255); }

inline PlanLayout plan_layout(int B, int T) {
  PlanLayout L;
  L.B = B;
  L.T = T;
  L.NB = (T + kTile - 1) / kTile;
  const size_t nb = (size_t)L.NB, b = (size_t)B;
  size_t off = 0;
  L.status = off;    off = plan_align(off + 64 * sizeof(int32_t));
  L.run_cnt = off;   off = plan_align(off + b * nb * sizeof(int32_t));
  L.runs = off;      off = plan_align(off + b * nb * kTile * sizeof(Run));
  L.state = off;     off = plan_align(off + b * nb * nb);
  L.fwd_cnt = off;   off = plan_align(off + b * nb * sizeof(int32_t));
  L.fwd_idx = off;   off = plan_align(off + b * nb * nb * sizeof(int32_t));
  L.bwd_cnt = off;   off = plan_align(off + b * nb * sizeof(int32_t));
  L.bwd_idx = off;   off = plan_align(off + b * nb * nb * sizeof(int32_t));
  L.fwd_order = off; off = plan_align(off + b * nb * sizeof(int32_t));
  L.bwd_order = off; off = plan_align(off + b * nb * sizeof(int32_t));
  const size_t np = (nb + 1) / 2;
  L.pair_cnt = off;   off = plan_align(off + b * np * sizeof(int32_t));
  L.pair_order = off; off = plan_align(off + b * np * sizeof(int32_t));
  L.link_t = off;     off = plan_align(off + b * kLinkTMaxCols * kLinkTWords * sizeof(uint64_t));
  L.bytes = off;
  return L;
}

// Device-side view (pointers resolved from the layout).
struct PlanView {
  int B, T, NB;
  int32_t* status;
  int32_t* run_cnt;
  Run* runs;
  uint8_t* state;
  int32_t* fwd_cnt;
  int32_t* fwd_idx;
  int32_t* bwd_cnt;
  int32_t* bwd_idx;
  int32_t* fwd_order;
  int32_t* bwd_order;
  int32_t* pair_cnt;
  int32_t* pair_order;
  unsigned long long* link_t;
};

inline PlanView plan_view(void* base, int B, int T) {
  PlanLayout L = plan_layout(B, T);
  char* p = static_cast<char*>(base);
  PlanView v;
  v.B = B; v.T = T; v.NB = L.NB;
  v.status = reinterpret_cast<int32_t*>(p + L.status);
  v.run_cnt = reinterpret_cast<int32_t*>(p + L.run_cnt);
  v.runs = reinterpret_cast<Run*>(p + L.runs);
  v.state = reinterpret_cast<uint8_t*>(p + L.state);
  v.fwd_cnt = reinterpret_cast<int32_t*>(p + L.fwd_cnt);
  v.fwd_idx = reinterpret_cast<int32_t*>(p + L.fwd_idx);
  v.bwd_cnt = reinterpret_cast<int32_t*>(p + L.bwd_cnt);
  v.bwd_idx = reinterpret_cast<int32_t*>(p + L.bwd_idx);
  v.fwd_order = reinterpret_cast<int32_t*>(p + L.fwd_order);
  v.bwd_order = reinterpret_cast<int32_t*>(p + L.bwd_order);
  v.pair_cnt = reinterpret_cast<int32_t*>(p + L.pair_cnt);
  v.pair_order = reinterpret_cast<int32_t*>(p + L.pair_order);
  v.link_t = reinterpret_cast<unsigned long long*>(p + L.link_t);
  return v;
}

// Per-token mask inputs of one call (device pointers; row/col may alias doc).
struct MaskArgs {
  const int32_t* doc;    // [B,T]
  const int32_t* row;    // [B,T] row class of a query token, <0 = none
  const int32_t* col;    // [B,T] column class of a key token, <0 = none
  const int64_t* link;   // [B,R,W] bit c of row r: row class r may read column class c; nullptr = no links
  int R, W;
};

}  // namespace ts2ts
