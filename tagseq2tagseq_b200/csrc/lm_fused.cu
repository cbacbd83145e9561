// Memory-bound pieces of the decoder layer around the attention operator, one pass over HBM each: residual add +
// RMSNorm, rotary embedding applied in place to the q and k parts of the packed QKV projection, SwiGLU, and the
// cross-entropy of the output head.  They stand where the reference's training step has its fused modules
// (model/modules/layer.py:20-35: RMSNorm, rotary attention, SwiGLU; model/modules/training_module.py:205: fused
// linear + cross-entropy loss) and only exist so that the training-step benchmark measures the attention kernels and
// the GEMMs rather than chains of element-wise launches.  All arithmetic is fp32; bf16 only in memory.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

namespace ts2ts {
namespace {

constexpr int kMaxVec = 4;  // float4 per thread and row in the wide variant: C <= 16 * blockDim.x

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Block-wide reductions; `red` holds 32 floats; every thread receives the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  return warp_sum(lane < nw ? red[lane] : 0.f);
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  return warp_max(lane < nw ? red[lane] : -CUDART_INF_F);
}

__device__ __forceinline__ float4 bf16x4_to_float4(uint2 raw) {
  const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  const float2 a = __bfloat1622float2(lo), b = __bfloat1622float2(hi);
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ uint2 float4_to_bf16x4(float4 v) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 r;
  r.x = *reinterpret_cast<const uint32_t*>(&lo);
  r.y = *reinterpret_cast<const uint32_t*>(&hi);
  return r;
}
__device__ __forceinline__ void bf16x8_to_float(uint4 raw, float (&f)[8]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
    f[2 * i] = a.x;
    f[2 * i + 1] = a.y;
  }
}
__device__ __forceinline__ uint4 float_to_bf16x8(const float (&f)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 p = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&p);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// ---------------------------------------------------------------------------------------------- residual add + RMSNorm
// x_out = x_in + a (a may be null), h = x_out * rstd * w with rstd = 1 / sqrt(mean(x_out^2) + eps).  One block per row.
template <int NV>  // float4 per thread and row: 1 when C <= 4 * blockDim.x, else kMaxVec
__global__ void add_rmsnorm_fwd_kernel(const float* __restrict__ x_in, const __nv_bfloat16* __restrict__ a, const float* __restrict__ w,
                                       float* x_out, __nv_bfloat16* __restrict__ h, float* __restrict__ rstd, int C, float eps) {
  __shared__ float red[32];
  const size_t base = (size_t)blockIdx.x * C;
  float4 v[NV];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (threadIdx.x + i * blockDim.x) * 4;
    if (c < C) {
      float4 x = *reinterpret_cast<const float4*>(x_in + base + c);
      if (a != nullptr) {
        const float4 d = bf16x4_to_float4(*reinterpret_cast<const uint2*>(a + base + c));
        x.x += d.x; x.y += d.y; x.z += d.z; x.w += d.w;
      }
      *reinterpret_cast<float4*>(x_out + base + c) = x;
      v[i] = x;
      ss += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
    }
  }
  ss = block_sum(ss, red);
  const float r = rsqrtf(ss / (float)C + eps);
  if (threadIdx.x == 0) rstd[blockIdx.x] = r;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (threadIdx.x + i * blockDim.x) * 4;
    if (c < C) {
      const float4 g = *reinterpret_cast<const float4*>(w + c);
      const float4 x = v[i];
      *reinterpret_cast<uint2*>(h + base + c) = float4_to_bf16x4(make_float4(x.x * r * g.x, x.y * r * g.y, x.z * r * g.z, x.w * r * g.w));
    }
  }
}

// Gradient of the pair above.  With xh = x_out * rstd and g = dh * w:
//   d(x_out) = dx_up + rstd * (g - xh * mean(g * xh)),  dw = sum over rows of dh * xh.
// d(x_out) is the gradient of both x_in and a (written in fp32 and, when da is given, in bf16).  Blocks walk the rows
// with a stride, keep their share of dw in registers and write it to row blockIdx.x of dw_part [gridDim.x, C] at the
// end (atomics on the C addresses of one dw vector serialise a thousand blocks); a second kernel adds the rows up.
template <int NV>
__global__ void add_rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dh, const float* __restrict__ dx_up, const float* __restrict__ x,
                                       const float* __restrict__ w, const float* __restrict__ rstd, float* __restrict__ dx,
                                       __nv_bfloat16* __restrict__ da, float* __restrict__ dw_part, int N, int C) {
  __shared__ float red[32];
  float4 wv[NV], acc[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (threadIdx.x + i * blockDim.x) * 4;
    wv[i] = c < C ? *reinterpret_cast<const float4*>(w + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  for (int row = blockIdx.x; row < N; row += gridDim.x) {
    const size_t base = (size_t)row * C;
    const float r = rstd[row];
    float4 xh[NV], g[NV];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = (threadIdx.x + i * blockDim.x) * 4;
      if (c < C) {
        const float4 xv = *reinterpret_cast<const float4*>(x + base + c);
        const float4 d = bf16x4_to_float4(*reinterpret_cast<const uint2*>(dh + base + c));
        xh[i] = make_float4(xv.x * r, xv.y * r, xv.z * r, xv.w * r);
        g[i] = make_float4(d.x * wv[i].x, d.y * wv[i].y, d.z * wv[i].z, d.w * wv[i].w);
        dot += g[i].x * xh[i].x + g[i].y * xh[i].y + g[i].z * xh[i].z + g[i].w * xh[i].w;
        acc[i].x += d.x * xh[i].x; acc[i].y += d.y * xh[i].y; acc[i].z += d.z * xh[i].z; acc[i].w += d.w * xh[i].w;
      }
    }
    dot = block_sum(dot, red) / (float)C;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = (threadIdx.x + i * blockDim.x) * 4;
      if (c < C) {
        float4 o = make_float4(r * (g[i].x - xh[i].x * dot), r * (g[i].y - xh[i].y * dot), r * (g[i].z - xh[i].z * dot),
                               r * (g[i].w - xh[i].w * dot));
        if (dx_up != nullptr) {
          const float4 u = *reinterpret_cast<const float4*>(dx_up + base + c);
          o.x += u.x; o.y += u.y; o.z += u.z; o.w += u.w;
        }
        *reinterpret_cast<float4*>(dx + base + c) = o;
        if (da != nullptr) *reinterpret_cast<uint2*>(da + base + c) = float4_to_bf16x4(o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (threadIdx.x + i * blockDim.x) * 4;
    if (c < C) *reinterpret_cast<float4*>(dw_part + (size_t)blockIdx.x * C + c) = acc[i];
  }
}
// dw[c] += sum over the rows of dw_part[rows, C].
__global__ void column_sum_kernel(const float* __restrict__ part, float* dw, int rows, int C) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  int r = 0;
  for (; r + 3 < rows; r += 4) {
    s0 += part[(size_t)r * C + c];
    s1 += part[(size_t)(r + 1) * C + c];
    s2 += part[(size_t)(r + 2) * C + c];
    s3 += part[(size_t)(r + 3) * C + c];
  }
  for (; r < rows; ++r) s0 += part[(size_t)r * C + c];
  dw[c] += (s0 + s1) + (s2 + s3);
}

// ---------------------------------------------------------------------------------------------- rotary embedding
// In place on the q (part 0) and k (part 1) slices of qkv [B,T,3,H,D]: pairs (i, i + D/2),
//   y1 = x1 cos - sign * x2 sin,  y2 = x2 cos + sign * x1 sin;  sign = -1 turns a gradient back (the inverse rotation).
// cos / sin are fp32 [T, D/2].  One thread rotates eight pairs.
__global__ void rope_qk_kernel(__nv_bfloat16* qkv, const float* __restrict__ cs, const float* __restrict__ sn, int T, int H, int D,
                               int64_t n_threads, float sign) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_threads) return;
  const int vec_per_head = D / 16;  // groups of eight pairs
  int64_t r = idx;
  const int i8 = (int)(r % vec_per_head); r /= vec_per_head;
  const int h = (int)(r % H); r /= H;
  const int part = (int)(r % 2); r /= 2;
  const int t = (int)(r % T);
  const int64_t b = r / T;
  __nv_bfloat16* lo = qkv + ((((b * T + t) * 3 + part) * H + h) * (int64_t)D + i8 * 8);
  __nv_bfloat16* hi = lo + D / 2;
  float x1[8], x2[8], c[8], s[8];
  bf16x8_to_float(*reinterpret_cast<const uint4*>(lo), x1);
  bf16x8_to_float(*reinterpret_cast<const uint4*>(hi), x2);
  const float* cp = cs + (size_t)t * (D / 2) + i8 * 8;
  const float* sp = sn + (size_t)t * (D / 2) + i8 * 8;
  *reinterpret_cast<float4*>(c) = *reinterpret_cast<const float4*>(cp);
  *reinterpret_cast<float4*>(c + 4) = *reinterpret_cast<const float4*>(cp + 4);
  *reinterpret_cast<float4*>(s) = *reinterpret_cast<const float4*>(sp);
  *reinterpret_cast<float4*>(s + 4) = *reinterpret_cast<const float4*>(sp + 4);
  float y1[8], y2[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    y1[i] = x1[i] * c[i] - sign * x2[i] * s[i];
    y2[i] = x2[i] * c[i] + sign * x1[i] * s[i];
  }
  *reinterpret_cast<uint4*>(lo) = float_to_bf16x8(y1);
  *reinterpret_cast<uint4*>(hi) = float_to_bf16x8(y2);
}

// ---------------------------------------------------------------------------------------------- SwiGLU
// gu [N, 2F]: gate in the first F columns, up in the last F (torch.chunk(2, dim=-1));  act = silu(gate) * up.
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ act, int F, int64_t n_vec) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_vec) return;
  const int per_row = F / 8;
  const int64_t row = idx / per_row;
  const int c = (int)(idx % per_row) * 8;
  float g[8], u[8], o[8];
  bf16x8_to_float(*reinterpret_cast<const uint4*>(gu + row * 2 * F + c), g);
  bf16x8_to_float(*reinterpret_cast<const uint4*>(gu + row * 2 * F + F + c), u);
#pragma unroll
  for (int i = 0; i < 8; ++i) o[i] = g[i] / (1.f + __expf(-g[i])) * u[i];
  *reinterpret_cast<uint4*>(act + row * F + c) = float_to_bf16x8(o);
}
// d gate = dact * up * s * (1 + gate * (1 - s)),  d up = dact * gate * s,  s = sigmoid(gate).
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dact,
                                  __nv_bfloat16* __restrict__ dgu, int F, int64_t n_vec) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_vec) return;
  const int per_row = F / 8;
  const int64_t row = idx / per_row;
  const int c = (int)(idx % per_row) * 8;
  float g[8], u[8], d[8], dg[8], du[8];
  bf16x8_to_float(*reinterpret_cast<const uint4*>(gu + row * 2 * F + c), g);
  bf16x8_to_float(*reinterpret_cast<const uint4*>(gu + row * 2 * F + F + c), u);
  bf16x8_to_float(*reinterpret_cast<const uint4*>(dact + row * F + c), d);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float s = 1.f / (1.f + __expf(-g[i]));
    dg[i] = d[i] * u[i] * s * (1.f + g[i] * (1.f - s));
    du[i] = d[i] * g[i] * s;
  }
  *reinterpret_cast<uint4*>(dgu + row * 2 * F + c) = float_to_bf16x8(dg);
  *reinterpret_cast<uint4*>(dgu + row * 2 * F + F + c) = float_to_bf16x8(du);
}

// ---------------------------------------------------------------------------------------------- cross-entropy
// One block per row of logits [N, V] (bf16, V a multiple of 8).  Forward: lse = log sum exp, loss = lse - logit[target].
__global__ void ce_fwd_kernel(const __nv_bfloat16* __restrict__ logits, const int64_t* __restrict__ target, float* __restrict__ lse,
                              float* __restrict__ loss, int V) {
  __shared__ float red[32];
  const __nv_bfloat16* row = logits + (size_t)blockIdx.x * V;
  float m = -CUDART_INF_F, s = 0.f;
  for (int c = threadIdx.x * 8; c < V; c += blockDim.x * 8) {
    float f[8];
    bf16x8_to_float(*reinterpret_cast<const uint4*>(row + c), f);
    float mx = f[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) mx = fmaxf(mx, f[i]);
    const float m_new = fmaxf(m, mx);
    if (m_new == -CUDART_INF_F) continue;  // nothing but -inf so far: contributes nothing, and -inf - -inf is no number
    float add = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) add += __expf(f[i] - m_new);
    s = s * __expf(m - m_new) + add;
    m = m_new;
  }
  const float m_all = block_max(m, red);
  const float s_all = block_sum(m == -CUDART_INF_F ? 0.f : s * __expf(m - m_all), red);
  if (threadIdx.x == 0) {
    const float l = m_all + logf(s_all);
    const int64_t tg = target[blockIdx.x];
    lse[blockIdx.x] = l;
    loss[blockIdx.x] = (tg >= 0 && tg < V) ? l - __bfloat162float(row[tg]) : 0.f;
  }
}
// Backward, in place: logits <- (softmax - onehot(target)) * gscale[0] * inv_n.  Rows whose target is out of range
// contributed no loss and get a zero gradient.
__global__ void ce_bwd_kernel(__nv_bfloat16* logits, const int64_t* __restrict__ target, const float* __restrict__ lse,
                              const float* __restrict__ gscale, float inv_n, int V) {
  __nv_bfloat16* row = logits + (size_t)blockIdx.x * V;
  const int64_t tg = target[blockIdx.x];
  const bool live = tg >= 0 && tg < V;
  const float l = lse[blockIdx.x], g = live ? gscale[0] * inv_n : 0.f;
  for (int c = threadIdx.x * 8; c < V; c += blockDim.x * 8) {
    float f[8];
    bf16x8_to_float(*reinterpret_cast<const uint4*>(row + c), f);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = (__expf(f[i] - l) - ((int64_t)(c + i) == tg ? 1.f : 0.f)) * g;
    *reinterpret_cast<uint4*>(row + c) = float_to_bf16x8(f);
  }
}

int norm_threads(int C) {
  int t = (C / 4 + kMaxVec - 1) / kMaxVec;  // threads needed with kMaxVec float4 each
  t = ((t + 31) / 32) * 32;
  // prefer one float4 per thread while the block stays within 1024 threads
  const int one = ((C / 4 + 31) / 32) * 32;
  return one <= 1024 ? one : t;
}

}  // namespace

cudaError_t launch_add_rmsnorm_fwd(const float* x_in, const void* a, const float* w, float* x_out, void* h, float* rstd, int N, int C,
                                   float eps, cudaStream_t stream) {
  const int threads = norm_threads(C);
  if (C <= 4 * threads)
    add_rmsnorm_fwd_kernel<1><<<N, threads, 0, stream>>>(x_in, static_cast<const __nv_bfloat16*>(a), w, x_out, static_cast<__nv_bfloat16*>(h),
                                                         rstd, C, eps);
  else
    add_rmsnorm_fwd_kernel<kMaxVec><<<N, threads, 0, stream>>>(x_in, static_cast<const __nv_bfloat16*>(a), w, x_out,
                                                               static_cast<__nv_bfloat16*>(h), rstd, C, eps);
  return cudaGetLastError();
}

// Blocks of the backward kernel = rows of its dw_part workspace.
int add_rmsnorm_bwd_blocks(int64_t N, int C) {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    sms = n;
  }
  const int threads = norm_threads(C);
  const int per_sm = 2048 / threads;  // as many resident blocks as the thread limit allows
  const int64_t cap = (int64_t)sms * per_sm;
  return (int)(N < cap ? N : cap);
}

cudaError_t launch_add_rmsnorm_bwd(const void* dh, const float* dx_up, const float* x, const float* w, const float* rstd, float* dx,
                                   void* da, float* dw, float* dw_part, int N, int C, cudaStream_t stream) {
  const int grid = add_rmsnorm_bwd_blocks(N, C);
  const int threads = norm_threads(C);
  if (C <= 4 * threads)
    add_rmsnorm_bwd_kernel<1><<<grid, threads, 0, stream>>>(static_cast<const __nv_bfloat16*>(dh), dx_up, x, w, rstd, dx,
                                                            static_cast<__nv_bfloat16*>(da), dw_part, N, C);
  else
    add_rmsnorm_bwd_kernel<kMaxVec><<<grid, threads, 0, stream>>>(static_cast<const __nv_bfloat16*>(dh), dx_up, x, w, rstd, dx,
                                                                  static_cast<__nv_bfloat16*>(da), dw_part, N, C);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  column_sum_kernel<<<(C + 127) / 128, 128, 0, stream>>>(dw_part, dw, grid, C);
  return cudaGetLastError();
}

cudaError_t launch_rope_qk(void* qkv, const float* cs, const float* sn, int B, int T, int H, int D, float sign, cudaStream_t stream) {
  const int64_t n = (int64_t)B * T * 2 * H * (D / 16);
  const int threads = 256;
  rope_qk_kernel<<<(unsigned)((n + threads - 1) / threads), threads, 0, stream>>>(static_cast<__nv_bfloat16*>(qkv), cs, sn, T, H, D, n, sign);
  return cudaGetLastError();
}

cudaError_t launch_swiglu_fwd(const void* gu, void* act, int64_t N, int F, cudaStream_t stream) {
  const int64_t n = N * (F / 8);
  const int threads = 256;
  swiglu_fwd_kernel<<<(unsigned)((n + threads - 1) / threads), threads, 0, stream>>>(static_cast<const __nv_bfloat16*>(gu),
                                                                                     static_cast<__nv_bfloat16*>(act), F, n);
  return cudaGetLastError();
}

cudaError_t launch_swiglu_bwd(const void* gu, const void* dact, void* dgu, int64_t N, int F, cudaStream_t stream) {
  const int64_t n = N * (F / 8);
  const int threads = 256;
  swiglu_bwd_kernel<<<(unsigned)((n + threads - 1) / threads), threads, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(gu), static_cast<const __nv_bfloat16*>(dact), static_cast<__nv_bfloat16*>(dgu), F, n);
  return cudaGetLastError();
}

cudaError_t launch_ce_fwd(const void* logits, const int64_t* target, float* lse, float* loss, int N, int V, cudaStream_t stream) {
  ce_fwd_kernel<<<N, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(logits), target, lse, loss, V);
  return cudaGetLastError();
}

cudaError_t launch_ce_bwd(void* logits, const int64_t* target, const float* lse, const float* gscale, float inv_n, int N, int V,
                          cudaStream_t stream) {
  ce_bwd_kernel<<<N, 256, 0, stream>>>(static_cast<__nv_bfloat16*>(logits), target, lse, gscale, inv_n, V);
  return cudaGetLastError();
}

}  // namespace ts2ts
