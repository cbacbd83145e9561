// Test-only library (libts2ts_selftest.so): one kernel that exercises the bounded mbarrier wait of ptx.cuh on a
// barrier nobody ever arrives on.  It is compiled with a small TS2TS_SPIN_LIMIT so that the wait gives up after
// microseconds, records its code exactly as the attention kernels do (status word 0 of a plan-shaped buffer, set
// once with atomicCAS) and returns normally.  Nothing in libts2ts_attn.so links or calls this file: the product
// kernels cannot reach it, and it issues no TMA copy and no tensor-core instruction that could still be in
// flight when the wait ends.
#ifndef TS2TS_SPIN_LIMIT
#define TS2TS_SPIN_LIMIT 4096u
#endif
#include "../../include/ts2ts_selftest.h"
#include "ptx.cuh"

namespace ts2ts {

__global__ void __launch_bounds__(32) wait_runs_out_kernel(int32_t* status, int32_t code, long long* cycles) {
  __shared__ uint64_t bar;
  __shared__ int abort_word;
  if (threadIdx.x == 0) {
    abort_word = 0;
    mbar_init(&bar, 1);
    fence_mbar_init();
  }
  __syncwarp();
  if (threadIdx.x == 0) {
    const long long t0 = clock64();
    const bool completed = mbar_wait(&bar, 0, &abort_word, code);  // phase 0 never completes
    const bool second = mbar_wait(&bar, 0, &abort_word, code + 1);  // later waits must return at once
    if (!completed && !second) atomicCAS(status, 0, 1000 + abort_word);
    if (cycles != nullptr) *cycles = clock64() - t0;
  }
}

}  // namespace ts2ts

extern "C" int ts2ts_selftest_bounded_wait(int32_t* status, int32_t code, long long* cycles, void* stream) {
  if (status == nullptr || code <= 0 || code >= 1000) return -1;
  ts2ts::wait_runs_out_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(status, code, cycles);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" unsigned ts2ts_selftest_spin_limit(void) { return TS2TS_SPIN_LIMIT; }
