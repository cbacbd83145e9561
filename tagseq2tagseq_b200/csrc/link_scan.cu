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
// Two kernels: a grid-wide scan (HBM-bound: each token is read once, 4 or 8 bytes) that marks candidates in a dense
// int32[T] array, and a single-block ordered compaction.
#include "link_scan.h"

namespace ts2ts {

__device__ __forceinline__ long long load_token(const LinkScanArgs& a, int t) {
  return a.token_bytes == 8 ? static_cast<const long long*>(a.tokens)[t]
                            : static_cast<long long>(static_cast<const int*>(a.tokens)[t]);
}

// dense[t] = -1 (not a link) or the closing token's position; start_pos[t] = position of the opening bracket.
__global__ void __launch_bounds__(256) link_scan_kernel(LinkScanArgs a, int32_t* dense_close, int32_t* dense_start) {
  for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < a.T; t += gridDim.x * blockDim.x) {
    int close = -1, start = -1;
    if (load_token(a, t) == a.mid_id) {
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
    dense_close[t] = close;
    dense_start[t] = close >= 0 ? start : -1;
  }
}

// One block walks the dense array in order and appends (mid, start, close) triples; *count receives the number of
// candidates found (it may exceed max_links: only the first max_links triples are stored).
__global__ void __launch_bounds__(1024) link_compact_kernel(const int32_t* dense_close, const int32_t* dense_start, int T,
                                                            int32_t* out, int max_links, int32_t* count) {
  __shared__ int warp_sums[32];
  __shared__ int base;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) base = 0;
  __syncthreads();
  for (int t0 = 0; t0 < T; t0 += blockDim.x) {
    const int t = t0 + tid;
    const int close = t < T ? dense_close[t] : -1;
    const unsigned hit = close >= 0 ? 1u : 0u;
    const unsigned ballot = __ballot_sync(0xffffffffu, hit);
    if (lane == 0) warp_sums[warp] = __popc(ballot);
    __syncthreads();
    int before = __popc(ballot & ((1u << lane) - 1u));
    for (int w = 0; w < warp; ++w) before += warp_sums[w];
    const int slot = base + before;
    if (hit && slot < max_links) {
      out[3 * slot + 0] = t;
      out[3 * slot + 1] = dense_start[t];
      out[3 * slot + 2] = close;
    }
    __syncthreads();
    if (tid == 0) {
      int total = 0;
      for (int w = 0; w < 32; ++w) total += warp_sums[w];
      base += total;
    }
    __syncthreads();
  }
  if (tid == 0) *count = base;
}

cudaError_t launch_link_scan(const LinkScanArgs& a, int32_t* scratch /* 2*T int32 */, int32_t* out, int max_links, int32_t* count,
                             cudaStream_t stream) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int blocks = max(1, min((a.T + 255) / 256, sms * 8));
  link_scan_kernel<<<blocks, 256, 0, stream>>>(a, scratch, scratch + a.T);
  link_compact_kernel<<<1, 1024, 0, stream>>>(scratch, scratch + a.T, a.T, out, max_links, count);
  return cudaGetLastError();
}

}  // namespace ts2ts
