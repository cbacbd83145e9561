// Integer pre-pass: per-token doc ids / row classes / column classes / link bits
// -> 128x128 block map (skip / partial / full), ordered block lists and a
// heaviest-first tile order.  Replaces, in O(tiles x runs) integer work, what the
// reference obtains from torch's create_block_mask by materialising the dense
// T x T mask (called at block_mask_creator.py:132-139, cross_doc_mask.py:359-366;
// block sums at torch/nn/attention/flex_attention.py:1034-1084).
//
// A tile is cut into runs of constant (doc, row class, column class).  For a
// tile pair below the diagonal the number of allowed elements is
//   sum over (q-run i, kv-run j) of allowed(i, j) * len_i * len_j
// with allowed(i,j) = doc_i == doc_j  or  bit(link[row_i], col_j);  the pair is
// skipped when the sum is 0, full when it is 128*128 and partial otherwise.
// Tokens past T belong to no run, which reproduces torch's pad-with-False: a
// ragged last tile is never full.  A diagonal pair always holds its own
// diagonal (allowed) and the upper triangle (not allowed), so it is partial.
#include "plan.h"

#include <cuda_runtime.h>

namespace ts2ts {

__device__ __forceinline__ bool link_bit(const int64_t* link_b, int R, int W, int row, int col) {
  if (link_b == nullptr || row < 0 || row >= R || col < 0 || col >= 64 * W) return false;
  const unsigned long long w = static_cast<unsigned long long>(link_b[(size_t)row * W + (col >> 6)]);
  return (w >> (col & 63)) & 1ull;
}

// grid (NB, B), 128 threads: cut tile into runs.
__global__ void __launch_bounds__(128) runs_kernel(PlanView P, MaskArgs M) {
  const int tb = blockIdx.x, b = blockIdx.y, t = threadIdx.x;
  const int pos = tb * kTile + t;
  const bool valid = pos < P.T;
  const size_t base = (size_t)b * P.T;
  int d = 0, r = 0, c = 0;
  bool flag = false;
  if (valid) {
    d = M.doc[base + pos]; r = M.row[base + pos]; c = M.col[base + pos];
    if (t == 0) flag = true;
    else flag = d != M.doc[base + pos - 1] || r != M.row[base + pos - 1] || c != M.col[base + pos - 1];
  }
  __shared__ int warp_cnt[4];
  const unsigned bal = __ballot_sync(0xffffffffu, flag);
  const int lane = t & 31, w = t >> 5;
  if (lane == 0) warp_cnt[w] = __popc(bal);
  __syncthreads();
  int off = 0;
  for (int i = 0; i < w; ++i) off += warp_cnt[i];
  const int total = warp_cnt[0] + warp_cnt[1] + warp_cnt[2] + warp_cnt[3];
  if (flag) {
    const int idx = off + __popc(bal & ((1u << lane) - 1u));
    Run run; run.start = t; run.doc = d; run.row = r; run.col = c;
    P.runs[((size_t)b * P.NB + tb) * kTile + idx] = run;
  }
  if (t == 0) P.run_cnt[(size_t)b * P.NB + tb] = total;
}

// One thread per (kb, qb, b).
__global__ void __launch_bounds__(128) state_kernel(PlanView P, MaskArgs M) {
  const int kb = blockIdx.x * blockDim.x + threadIdx.x, qb = blockIdx.y, b = blockIdx.z;
  if (kb >= P.NB) return;
  uint8_t st = kSkip;
  const int nvq = min(kTile, P.T - qb * kTile);
  if (kb == qb) {
    st = nvq > 0 ? kPartial : kSkip;
  } else if (kb < qb) {
    const int64_t* link_b = M.link ? M.link + (size_t)b * M.R * M.W : nullptr;
    const Run* qr = P.runs + ((size_t)b * P.NB + qb) * kTile;
    const Run* kr = P.runs + ((size_t)b * P.NB + kb) * kTile;
    const int nq = P.run_cnt[(size_t)b * P.NB + qb], nk = P.run_cnt[(size_t)b * P.NB + kb];
    int count = 0;
    for (int j = 0; j < nk; ++j) {
      const Run kj = kr[j];
      const int lk = (j + 1 < nk ? kr[j + 1].start : kTile) - kj.start;  // kv tiles below the diagonal are complete
      for (int i = 0; i < nq; ++i) {
        const Run qi = qr[i];
        const int lq = (i + 1 < nq ? qr[i + 1].start : nvq) - qi.start;
        if (qi.doc == kj.doc || link_bit(link_b, M.R, M.W, qi.row, kj.col)) count += lq * lk;
      }
    }
    st = count == 0 ? kSkip : (count == kTile * kTile ? kFull : kPartial);
  }
  P.state[((size_t)b * P.NB + qb) * P.NB + kb] = st;
}

// One warp per line.  transposed == 0: line = q tile, scan kv tiles; 1: line = kv tile, scan q tiles.
// Writes the merged list used by the kernels and, when given, the separate partial / full lists in the
// BlockMask convention (ascending, entries past the count = -1).
struct ListOutputs {
  int32_t *part_cnt, *part_idx, *full_cnt, *full_idx;
};
__global__ void __launch_bounds__(128) lists_kernel(PlanView P, ListOutputs fwd_out, ListOutputs bwd_out) {
  const int transposed = blockIdx.z;  // 0: line = q tile, scan kv tiles; 1: line = kv tile, scan q tiles
  int32_t* part_cnt = transposed ? bwd_out.part_cnt : fwd_out.part_cnt;
  int32_t* part_idx = transposed ? bwd_out.part_idx : fwd_out.part_idx;
  int32_t* full_cnt = transposed ? bwd_out.full_cnt : fwd_out.full_cnt;
  int32_t* full_idx = transposed ? bwd_out.full_idx : fwd_out.full_idx;
  const int line = blockIdx.x * 4 + (threadIdx.x >> 5), b = blockIdx.y, lane = threadIdx.x & 31;
  if (line >= P.NB) return;
  const size_t lb = (size_t)b * P.NB + line;
  int32_t* m_idx = (transposed ? P.bwd_idx : P.fwd_idx) + lb * P.NB;
  int n_m = 0, n_p = 0, n_f = 0;
  for (int c0 = 0; c0 < P.NB; c0 += 32) {
    const int c = c0 + lane;
    uint8_t st = kSkip;
    if (c < P.NB) st = transposed ? P.state[((size_t)b * P.NB + c) * P.NB + line] : P.state[lb * P.NB + c];
    const unsigned bm = __ballot_sync(0xffffffffu, st != kSkip);
    const unsigned bp = __ballot_sync(0xffffffffu, st == kPartial);
    const unsigned bf = __ballot_sync(0xffffffffu, st == kFull);
    const unsigned below = (1u << lane) - 1u;
    if (st != kSkip) m_idx[n_m + __popc(bm & below)] = c | (st == kFull ? (int)kFullBit : 0);
    if (part_idx && st == kPartial) part_idx[lb * P.NB + n_p + __popc(bp & below)] = c;
    if (full_idx && st == kFull) full_idx[lb * P.NB + n_f + __popc(bf & below)] = c;
    n_m += __popc(bm); n_p += __popc(bp); n_f += __popc(bf);
  }
  for (int c = n_m + lane; c < P.NB; c += 32) m_idx[c] = -1;
  if (part_idx) for (int c = n_p + lane; c < P.NB; c += 32) part_idx[lb * P.NB + c] = -1;
  if (full_idx) for (int c = n_f + lane; c < P.NB; c += 32) full_idx[lb * P.NB + c] = -1;
  if (lane == 0) {
    (transposed ? P.bwd_cnt : P.fwd_cnt)[lb] = n_m;
    if (part_cnt) part_cnt[lb] = n_p;
    if (full_cnt) full_cnt[lb] = n_f;
  }
}

// Forward work items are pairs of adjacent q tiles (2p, 2p+1) that share one stream of K/V tiles: count the kv
// tiles at least one of the two reads.  One warp per (pair, b).
__global__ void __launch_bounds__(128) pair_count_kernel(PlanView P) {
  const int pr = blockIdx.x * 4 + (threadIdx.x >> 5), b = blockIdx.y, lane = threadIdx.x & 31;
  const int NP = (P.NB + 1) / 2;
  if (pr >= NP) return;
  const uint8_t* s0 = P.state + ((size_t)b * P.NB + 2 * pr) * P.NB;
  const uint8_t* s1 = (2 * pr + 1 < P.NB) ? s0 + P.NB : s0;
  int n = 0;
  for (int kb = lane; kb <= min(2 * pr + 1, P.NB - 1); kb += 32) n += (s0[kb] | s1[kb]) != kSkip;
  for (int sh = 16; sh > 0; sh >>= 1) n += __shfl_xor_sync(0xffffffffu, n, sh);
  if (lane == 0) P.pair_cnt[(size_t)b * NP + pr] = n;
}

// Heaviest-first order inside each batch element: rank by descending count, ties by index.
// which = 0: q tiles by fwd_cnt, 1: kv tiles by bwd_cnt, 2: q-tile pairs by pair_cnt.
__global__ void __launch_bounds__(256) order_kernel(PlanView P, int link_t_rows) {
  const int b = blockIdx.y, which = blockIdx.z;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i == 0 && b == 0 && which == 0) {  // this is the last launch of the pre-pass: stamp the plan (see plan.h)
    P.status[kStampMagic] = kPlanMagic;
    P.status[kStampB] = P.B;
    P.status[kStampT] = P.T;
    P.status[kLinkTRows] = link_t_rows;
  }
  const int n = which == 2 ? (P.NB + 1) / 2 : P.NB;
  if (i >= n) return;
  const int32_t* cnt = (which == 2 ? P.pair_cnt : which == 1 ? P.bwd_cnt : P.fwd_cnt) + (size_t)b * n;
  int32_t* order = (which == 2 ? P.pair_order : which == 1 ? P.bwd_order : P.fwd_order) + (size_t)b * n;
  const int ci = cnt[i];
  int rank = 0;
  for (int j = 0; j < n; ++j) {
    const int cj = cnt[j];
    rank += (cj > ci) || (cj == ci && j < i);
  }
  order[rank] = i;
}

// One thread per (word, column class, b): gathers 64 row classes' bits for one column class.
__global__ void __launch_bounds__(128) link_transpose_kernel(PlanView P, MaskArgs M) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x, w = blockIdx.y, b = blockIdx.z;
  if (c >= 64 * M.W) return;
  const int64_t* link_b = M.link + (size_t)b * M.R * M.W;
  unsigned long long out = 0ull;
  for (int r = 64 * w; r < min(64 * w + 64, M.R); ++r)
    out |= ((static_cast<unsigned long long>(link_b[(size_t)r * M.W + (c >> 6)]) >> (c & 63)) & 1ull) << (r - 64 * w);
  P.link_t[((size_t)b * kLinkTMaxCols + c) * kLinkTWords + w] = out;
}

// Per-token ids from a sorted table of segments: token t gets ids[j] for bounds[j] <= t < bounds[j + 1], and -1 before
// bounds[0] or from bounds[n_seg] on.  This is the device-side half of what the reference does with one slice
// assignment per grant (cross_doc_mask.py:277-294): the host only works out the few hundred segment boundaries.
__global__ void __launch_bounds__(256) segment_ids_kernel(const int32_t* __restrict__ bounds, const int32_t* __restrict__ ids,
                                                          int n_seg, int T, int32_t* __restrict__ out) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  int lo = 0, hi = n_seg + 1;  // first boundary > t, by bisection over bounds[0 .. n_seg]
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (__ldg(bounds + mid) <= t) lo = mid + 1; else hi = mid;
  }
  out[t] = (lo == 0 || lo > n_seg) ? -1 : __ldg(ids + lo - 1);
}

cudaError_t launch_segment_ids(const int32_t* bounds, const int32_t* ids, int n_seg, int T, int32_t* out, cudaStream_t stream) {
  segment_ids_kernel<<<(T + 255) / 256, 256, 0, stream>>>(bounds, ids, n_seg, T, out);
  return cudaGetLastError();
}

// Host entry: fills the plan; optional BlockMask-shaped outputs may be null.
cudaError_t launch_block_map(PlanView P, MaskArgs M, uint8_t* state_out, int32_t* kv_cnt, int32_t* kv_idx,
                             int32_t* full_cnt, int32_t* full_idx, int32_t* q_cnt, int32_t* q_idx, int32_t* full_q_cnt,
                             int32_t* full_q_idx, cudaStream_t stream) {
  if (P.NB == 0 || P.B == 0) return cudaSuccess;
  cudaMemsetAsync(P.status, 0, 64 * sizeof(int32_t), stream);
  runs_kernel<<<dim3(P.NB, P.B), 128, 0, stream>>>(P, M);
  state_kernel<<<dim3((P.NB + 127) / 128, P.NB, P.B), 128, 0, stream>>>(P, M);
  lists_kernel<<<dim3((P.NB + 3) / 4, P.B, 2), 128, 0, stream>>>(P, ListOutputs{kv_cnt, kv_idx, full_cnt, full_idx},
                                                                  ListOutputs{q_cnt, q_idx, full_q_cnt, full_q_idx});
  pair_count_kernel<<<dim3(((P.NB + 1) / 2 + 3) / 4, P.B), 128, 0, stream>>>(P);
  int link_t_rows = 0;
  if (M.link != nullptr && M.R > 0 && M.R <= kLinkTMaxRows && 64 * M.W <= kLinkTMaxCols) {
    link_t_rows = M.R;
    link_transpose_kernel<<<dim3((64 * M.W + 127) / 128, (M.R + 63) / 64, P.B), 128, 0, stream>>>(P, M);
  }
  order_kernel<<<dim3((P.NB + 255) / 256, P.B, 3), 256, 0, stream>>>(P, link_t_rows);
  if (state_out)
    cudaMemcpyAsync(state_out, P.state, (size_t)P.B * P.NB * P.NB, cudaMemcpyDeviceToDevice, stream);
  return cudaGetLastError();
}

}  // namespace ts2ts
