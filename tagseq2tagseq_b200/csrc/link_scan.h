// Arguments of the markdown link scan (link_scan.cu), shared with the C-ABI layer.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace ts2ts {

constexpr int kMaxStartIds = 8;

struct LinkScanArgs {
  const void* tokens;   // int32 or int64 [T]
  int token_bytes;      // 4 or 8
  int T;
  long long mid_id;
  long long start_ids[kMaxStartIds];
  int n_start;
  const uint8_t* close_flags;  // [vocab]
  int vocab;
  int back_limit;       // 100 in the reference
  int window;
};

// `scratch` holds link_scan_scratch_ints(T) int32.  Launches on `stream`; returns the launch status.
size_t link_scan_scratch_ints(int T);
cudaError_t launch_link_scan(const LinkScanArgs& a, int32_t* scratch, int32_t* out, int max_links, int32_t* count,
                             cudaStream_t stream);

}  // namespace ts2ts
