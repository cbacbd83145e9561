// Optional CUDA-event bracketing of the main kernels (see ts2ts_profile_enable in include/ts2ts_attn.h).
#pragma once
#include <cuda_runtime.h>

namespace ts2ts {

struct ProfileSlot {
  bool enabled = false;
  bool recorded[2] = {false, false};
  cudaEvent_t start[2] = {nullptr, nullptr};
  cudaEvent_t stop[2] = {nullptr, nullptr};
};

ProfileSlot& profile_slot();  // one per device, defined in api.cu

struct ProfileScope {
  ProfileSlot& s;
  int which;
  cudaStream_t stream;
  ProfileScope(int which_, cudaStream_t st) : s(profile_slot()), which(which_), stream(st) {
    if (s.enabled) cudaEventRecord(s.start[which], stream);
  }
  ~ProfileScope() {
    if (s.enabled) {
      cudaEventRecord(s.stop[which], stream);
      s.recorded[which] = true;
    }
  }
};

}  // namespace ts2ts
