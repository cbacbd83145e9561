// Host-side construction of TMA tensor maps.  The driver entry point
// cuTensorMapEncodeTiled is resolved at run time through the CUDA runtime, so
// the library links against nothing but the (static) runtime and loads on a
// machine without a driver.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <mutex>

namespace ts2ts {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess)
    return nullptr;
  fn = reinterpret_cast<EncodeTiledFn>(p);
  return fn;
}

// Tensor [B,H,T,D] with D contiguous and element strides (sb, sh, st); tile = box_rows tokens x box_cols
// elements of one (b,h), written to shared memory with the 128-byte swizzle.  `elem_bytes` is 2 (bf16)
// or 4 (fp32); box_cols * elem_bytes must be 128.  Rows past T read as zero and are not written.
// Returns 0 on success.
inline int make_tile_map(CUtensorMap* out, const void* base, int elem_bytes, int64_t B, int64_t H, int64_t T, int64_t D,
                         int64_t sb, int64_t sh, int64_t st, int box_rows, int box_cols) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return -100;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) return -101;
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)T, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)st * elem_bytes, (cuuint64_t)sh * elem_bytes, (cuuint64_t)sb * elem_bytes};
  for (int i = 0; i < 3; ++i)
    if (strides[i] % 16 != 0) return -102;
  cuuint32_t box[4] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = enc(out, dt, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -103;
}

// The same map through a small per-process cache: a training step calls the attention entry points once per layer
// with the same few (pointer, shape, strides) combinations, and encoding a map costs a driver call each time.
// The map is copied out, so a later request that recycles the cache entry cannot change what a caller holds.
constexpr int kMapCacheSize = 64;
struct MapKey {
  const void* base;
  int64_t v[9];
  int dev;
};
inline int cached_tile_map(CUtensorMap* out, const void* base, int elem_bytes, int64_t B, int64_t H, int64_t T, int64_t D,
                           int64_t sb, int64_t sh, int64_t st, int box_rows, int box_cols) {
  struct Entry { MapKey key; CUtensorMap map; bool used; };
  static Entry cache[kMapCacheSize];
  static int next = 0;
  static std::mutex mu;
  MapKey key;
  memset(&key, 0, sizeof(key));
  key.base = base;
  const int64_t vals[9] = {elem_bytes, B, H, T, D, sb, sh, st, (int64_t)box_rows * 65536 + box_cols};
  for (int i = 0; i < 9; ++i) key.v[i] = vals[i];
  cudaGetDevice(&key.dev);
  std::lock_guard<std::mutex> lock(mu);
  for (int i = 0; i < kMapCacheSize; ++i)
    if (cache[i].used && memcmp(&cache[i].key, &key, sizeof(key)) == 0) {
      *out = cache[i].map;
      return 0;
    }
  Entry& e = cache[next];
  const int r = make_tile_map(&e.map, base, elem_bytes, B, H, T, D, sb, sh, st, box_rows, box_cols);
  if (r) {
    e.used = false;
    return r;
  }
  e.key = key;
  e.used = true;
  *out = e.map;
  next = (next + 1) % kMapCacheSize;
  return 0;
}

}  // namespace ts2ts
