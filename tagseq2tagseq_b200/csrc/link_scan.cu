// Candidate markdown links of a token sequence, found on the device.
//
// Restates the scan of MarkdownLinkDetector.detect_links (model/graph_traversal/markdown_link_detector.py:57-108)
// without its per-token host round trips:
//   * every position holding the "](" token id is a candidate (`:69`);
//   * the opening "[" is the nearest of the given start ids among the 100 tokens before it (`:74-79`); none -> no link;
//   * the closing ")" is looked for in the next `window` tokens (`:88-99`).  The reference decodes a growing
//     window until the text contains ')'.  ')' is one ASCII byte and a byte-level BPE token keeps its bytes whatever
//     its neighbours are, so "the decoded window contains ')'" is the same as "one of its tokens has a ')' byte":
//     `close_flags[token]` (one byte per vocabulary entry, built once on the host) answers that per token.
// Output: for every candidate, in ascending order of position (the order in which the reference appends links),
// the triple (mid position, start position, position of the closing token).  Decoding the few target tokens and the
// "non-empty after strip" test (`:94-97`) stay on the host, which needs the strings anyway.
//
// Three kernels: a grid-wide scan (HBM-bound: each token is read once, 4 or 8 bytes; one block per 256 positions)
// that marks candidates in a dense int32[T] array and counts them per block, a single-block exclusive scan of the
// block counts, and a grid-wide ordered write-out.
#include "link_scan.h"

namespace ts2ts {

__device__ __forceinline__ long long load_token(const LinkScanArgs& a, int t) {
  return a.token_bytes == 8 ? static_cast<const long long*>(a.tokens)[t]
                            : static_cast<long long>(static_cast<const int*>(a.tokens)[t]);
}

constexpr int kScanBlock = 256;

// dense_close[t] = -1 (not a link) or the closing token's position; dense_start[t] = position of the opening bracket;
// block_count[b] = candidates among positions [256 b, 256 b + 256).
__global__ void __launch_bounds__(kScanBlock) link_scan_kernel(LinkScanArgs a, int32_t* dense_close, int32_t* dense_start,
                                                                 int32_t* block_count) {
  __shared__ int warp_hits[kScanBlock / 32];
  const int t = blockIdx.x * kScanBlock + threadIdx.x;
  int close = -1, start = -1;
  if (t < a.T && load_token(a, t) == a.mid_id) {
    const int lo = max(0, t - a.back_limit);
    for (int i = t - 1; i >= lo && start < 0; --i) {
      const long long tok = load_token(a, i);
      for (int s = 0; s < a.n_start; ++s)
        if (tok == a.start_ids[s]) start = i;
    }
    if (start >= 0) {
      const int hi = min(t + 1 + a.window, a.T);
      for (int j = t + 1; j < hi; ++j) {
        const long long tok = load_token(a, j);
        if (tok >= 0 && tok < a.vocab && a.close_flags[tok]) {
          close = j;
          break;
        }
      }
    }
  }
  if (t < a.T) {
    dense_close[t] = close;
    dense_start[t] = close >= 0 ? start : -1;
  }
  const unsigned ballot = __ballot_sync(0xffffffffu, close >= 0);
  if ((threadIdx.x & 31) == 0) warp_hits[threadIdx.x >> 5] = __popc(ballot);
  __syncthreads();
  if (threadIdx.x == 0) {
    int total = 0;
    for (int w = 0; w < kScanBlock / 32; ++w) total += warp_hits[w];
    block_count[blockIdx.x] = total;
  }
}

// Exclusive scan of the block counts in place (one block; nb <= 4096 for the largest supported T); *count = total.
__global__ void __launch_bounds__(1024) link_offsets_kernel(int32_t* block_count, int nb, int32_t* count) {
  __shared__ int warp_sums[32];
  __shared__ int base;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) base = 0;
  __syncthreads();
  for (int b0 = 0; b0 < nb; b0 += blockDim.x) {
    const int bi = b0 + tid;
    const int v = bi < nb ? block_count[bi] : 0;
    int incl = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int o = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += o;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    int before = 0;
    for (int w = 0; w < warp; ++w) before += warp_sums[w];
    if (bi < nb) block_count[bi] = base + before + incl - v;
    __syncthreads();
    if (tid == blockDim.x - 1) base += before + incl;
    __syncthreads();
  }
  if (tid == 0) *count = base;
}

// Ordered write-out: block b appends its candidates at offset block_offset[b] in position order.  Only the first
// max_links triples are stored.
__global__ void __launch_bounds__(kScanBlock) link_write_kernel(const int32_t* dense_close, const int32_t* dense_start,
                                                                  const int32_t* block_offset, int T, int32_t* out, int max_links) {
  __shared__ int warp_hits[kScanBlock / 32];
  const int t = blockIdx.x * kScanBlock + threadIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int close = t < T ? dense_close[t] : -1;
  const unsigned ballot = __ballot_sync(0xffffffffu, close >= 0);
  if (lane == 0) warp_hits[warp] = __popc(ballot);
  __syncthreads();
  if (close < 0) return;
  int slot = block_offset[blockIdx.x] + __popc(ballot & ((1u << lane) - 1u));
  for (int w = 0; w < warp; ++w) slot += warp_hits[w];
  if (slot < max_links) {
    out[3 * slot + 0] = t;
    out[3 * slot + 1] = dense_start[t];
    out[3 * slot + 2] = close;
  }
}

size_t link_scan_scratch_ints(int T) { return 2 * static_cast<size_t>(T) + (T + kScanBlock - 1) / kScanBlock + 1; }

cudaError_t launch_link_scan(const LinkScanArgs& a, int32_t* scratch, int32_t* out, int max_links, int32_t* count,
                             cudaStream_t stream) {
  const int nb = (a.T + kScanBlock - 1) / kScanBlock;
  int32_t* dense_close = scratch;
  int32_t* dense_start = scratch + a.T;
  int32_t* block_count = scratch + 2 * static_cast<size_t>(a.T);
  link_scan_kernel<<<nb, kScanBlock, 0, stream>>>(a, dense_close, dense_start, block_count);
  link_offsets_kernel<<<1, 1024, 0, stream>>>(block_count, nb, count);
  link_write_kernel<<<nb, kScanBlock, 0, stream>>>(dense_close, dense_start, block_count, a.T, out, max_links);
  return cudaGetLastError();
}

}  // namespace ts2ts
