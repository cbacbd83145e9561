// extern "C" surface of libts2ts_attn.so: argument checks, then kernel launches on the caller's stream.
// Declarations and the contract of every entry point are in include/ts2ts_attn.h.
#include "../../include/ts2ts_attn.h"
#include "../../include/ts2ts_lm.h"

#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdio.h>

#include "link_scan.h"
#include "plan.h"
#include "profile.h"

namespace ts2ts {
cudaError_t launch_block_map(PlanView P, MaskArgs M, uint8_t* state_out, int32_t* kv_cnt, int32_t* kv_idx, int32_t* full_cnt,
                             int32_t* full_idx, int32_t* q_cnt, int32_t* q_idx, int32_t* full_q_cnt, int32_t* full_q_idx,
                             cudaStream_t stream);
int launch_fwd(const void* q, const void* k, const void* v, void* out, float* lse, const int64_t* sq, const int64_t* sk,
               const int64_t* sv, const int64_t* so, int B, int H, int T, int D, float scale, PlanView P, MaskArgs M,
               cudaStream_t stream);
cudaError_t launch_segment_ids(const int32_t* bounds, const int32_t* ids, int n_seg, int T, int32_t* out, cudaStream_t stream);
size_t bwd_workspace_bytes(int B, int H, int T, int D);
int launch_bwd(const void* q, const void* k, const void* v, const void* out, const void* dout, const float* lse, const int64_t* sq,
               const int64_t* sk, const int64_t* sv, const int64_t* so, const int64_t* sdo, int B, int H, int T, int D, float scale,
               PlanView P, MaskArgs M, void* dq, void* dk, void* dv, const int64_t* sdq, const int64_t* sdk, const int64_t* sdv,
               void* workspace, cudaStream_t stream);
int bwd_static_scratch(void** ptr, size_t* bytes);
cudaError_t launch_add_rmsnorm_fwd(const float* x_in, const void* a, const float* w, float* x_out, void* h, float* rstd, int N, int C,
                                   float eps, cudaStream_t stream);
cudaError_t launch_add_rmsnorm_bwd(const void* dh, const float* dx_up, const float* x, const float* w, const float* rstd, float* dx,
                                   void* da, float* dw, float* dw_part, int N, int C, cudaStream_t stream);
int add_rmsnorm_bwd_blocks(int64_t N, int C);
cudaError_t launch_rope_qk(void* qkv, const float* cs, const float* sn, int B, int T, int H, int D, float sign, cudaStream_t stream);
cudaError_t launch_swiglu_fwd(const void* gu, void* act, int64_t N, int F, cudaStream_t stream);
cudaError_t launch_swiglu_bwd(const void* gu, const void* dact, void* dgu, int64_t N, int F, cudaStream_t stream);
cudaError_t launch_ce_fwd(const void* logits, const int64_t* target, float* lse, float* loss, int N, int V, cudaStream_t stream);
cudaError_t launch_ce_bwd(void* logits, const int64_t* target, const float* lse, const float* gscale, float inv_n, int N, int V,
                          cudaStream_t stream);
size_t decode_workspace_bytes(int B, int H, int Tk, int D);
int launch_decode(const void* q, const void* k, const void* v, const int64_t* sq, const int64_t* sk, const int64_t* sv, int B, int H,
                  int Tk, int D, float scale, MaskArgs M, const int32_t* q_pos, void* out, const int64_t* so, float* lse,
                  void* workspace, cudaStream_t stream);

}  // namespace ts2ts

namespace ts2ts {
ProfileSlot& profile_slot() {
  static ProfileSlot slots[64];
  int dev = 0;
  cudaGetDevice(&dev);
  return slots[(dev >= 0 && dev < 64) ? dev : 0];
}
}  // namespace ts2ts

using namespace ts2ts;

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

constexpr int kMaxT = 1 << 20;

bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

int check_shape(int B, int H, int T, int D) {
  if (B <= 0 || H <= 0 || T <= 0) return fail(-1, "B, H and T must be positive (got B=%d H=%d T=%d)", B, H, T);
  if (T > kMaxT) return fail(-1, "T=%d exceeds the supported maximum %d", T, kMaxT);
  if (D != 64 && D != 128) return fail(-2, "head dimension must be 64 or 128 (got %d)", D);
  if ((long long)B * H * ((T + kTile - 1) / kTile) > 0x7fffffffLL) return fail(-1, "too many tiles for one launch");
  return 0;
}

int check_tensor(const char* name, const void* p, const int64_t* s) {
  if (p == nullptr || s == nullptr) return fail(-3, "%s: null pointer", name);
  if (!aligned(p, 16)) return fail(-4, "%s: base address must be 16-byte aligned", name);
  for (int i = 0; i < 3; ++i)
    if (s[i] <= 0 || (s[i] * 2) % 16 != 0) return fail(-5, "%s: stride %d = %lld elements is not a positive multiple of 8", name, i, (long long)s[i]);
  return 0;
}

int check_mask(const int32_t* doc, const int64_t* link, int R, int W) {
  if (doc == nullptr) return fail(-6, "doc_ids is null");
  if (link != nullptr && (R <= 0 || W <= 0)) return fail(-6, "link_bits given with R=%d W=%d", R, W);
  if (link == nullptr && (R != 0 || W != 0)) return fail(-6, "R and W must be 0 when link_bits is null");
  return 0;
}

int check_plan(const void* plan, size_t plan_bytes, int B, int T) {
  if (plan == nullptr || !aligned(plan, 256)) return fail(-7, "plan must be a 256-byte aligned device buffer");
  if (plan_bytes < plan_layout(B, T).bytes) return fail(-7, "plan buffer too small: %zu < %zu", plan_bytes, plan_layout(B, T).bytes);
  return 0;
}

MaskArgs mask_args(const int32_t* doc, const int32_t* row, const int32_t* col, const int64_t* link, int R, int W) {
  MaskArgs m;
  m.doc = doc;
  m.row = row ? row : doc;
  m.col = col ? col : doc;
  m.link = link;
  m.R = R;
  m.W = W;
  return m;
}

}  // namespace

extern "C" {

int ts2ts_version(void) { return 1000; }

const char* ts2ts_last_error_string(void) { return g_err; }

size_t ts2ts_plan_bytes(int B, int T) {
  if (B <= 0 || T <= 0 || T > kMaxT) return 0;
  return plan_layout(B, T).bytes;
}

int ts2ts_block_map(const int32_t* doc_ids, const int32_t* q_row_ids, const int32_t* kv_col_ids, const int64_t* link_bits, int B,
                    int T, int R, int W, void* plan, size_t plan_bytes, uint8_t* state, int32_t* kv_cnt, int32_t* kv_idx,
                    int32_t* full_cnt, int32_t* full_idx, int32_t* q_cnt, int32_t* q_idx, int32_t* full_q_cnt,
                    int32_t* full_q_idx, void* stream) {
  int r;
  if (B <= 0 || T <= 0 || T > kMaxT) return fail(-1, "B and T must be positive, T <= %d (got B=%d T=%d)", kMaxT, B, T);
  if ((r = check_mask(doc_ids, link_bits, R, W))) return r;
  if ((r = check_plan(plan, plan_bytes, B, T))) return r;
  PlanView P = plan_view(plan, B, T);
  cudaError_t e = launch_block_map(P, mask_args(doc_ids, q_row_ids, kv_col_ids, link_bits, R, W), state, kv_cnt, kv_idx, full_cnt,
                                   full_idx, q_cnt, q_idx, full_q_cnt, full_q_idx, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(-50, "block map launch failed: %s", cudaGetErrorString(e));
  return 0;
}

int ts2ts_segment_ids(const int32_t* bounds, const int32_t* ids, int n_seg, int T, int32_t* out, void* stream) {
  if (T <= 0 || T > kMaxT) return fail(-1, "T must be in 1..%d (got %d)", kMaxT, T);
  if (n_seg < 0 || n_seg > kMaxT) return fail(-1, "n_seg must be in 0..%d (got %d)", kMaxT, n_seg);
  if (out == nullptr || bounds == nullptr || (n_seg > 0 && ids == nullptr)) return fail(-3, "bounds / ids / out: null pointer");
  cudaError_t e = launch_segment_ids(bounds, ids, n_seg, T, out, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(-50, "segment id launch failed: %s", cudaGetErrorString(e));
  return 0;
}

int ts2ts_attn_fwd(const void* q, const void* k, const void* v, const int64_t* q_strides, const int64_t* k_strides,
                   const int64_t* v_strides, int B, int H, int T, int D, float scale, const int32_t* doc_ids,
                   const int32_t* q_row_ids, const int32_t* kv_col_ids, const int64_t* link_bits, int R, int W, const void* plan,
                   size_t plan_bytes, void* out, const int64_t* out_strides, float* lse, void* stream) {
  int r;
  if ((r = check_shape(B, H, T, D))) return r;
  if (!(scale > 0.f)) return fail(-8, "scale must be positive");
  if ((r = check_tensor("q", q, q_strides)) || (r = check_tensor("k", k, k_strides)) || (r = check_tensor("v", v, v_strides)) ||
      (r = check_tensor("out", out, out_strides)))
    return r;
  if (lse == nullptr) return fail(-3, "lse: null pointer");
  if ((r = check_mask(doc_ids, link_bits, R, W))) return r;
  if ((r = check_plan(plan, plan_bytes, B, T))) return r;
  PlanView P = plan_view(const_cast<void*>(plan), B, T);
  r = launch_fwd(q, k, v, out, lse, q_strides, k_strides, v_strides, out_strides, B, H, T, D, scale, P,
                 mask_args(doc_ids, q_row_ids, kv_col_ids, link_bits, R, W), static_cast<cudaStream_t>(stream));
  if (r) return fail(r, "forward launch failed (code %d, CUDA: %s)", r, cudaGetErrorString(cudaPeekAtLastError()));
  return 0;
}

size_t ts2ts_attn_decode_workspace_bytes(int B, int H, int Tk, int D) {
  if (B <= 0 || H <= 0 || Tk <= 0 || Tk > kMaxT || (D != 64 && D != 128)) return 0;
  return decode_workspace_bytes(B, H, Tk, D);
}

int ts2ts_attn_decode(const void* q, const void* k_cache, const void* v_cache, const int64_t* q_strides, const int64_t* k_strides,
                      const int64_t* v_strides, int B, int H, int Tk, int D, float scale, const int32_t* doc_ids,
                      const int32_t* q_row_ids, const int32_t* kv_col_ids, const int64_t* link_bits, int R, int W,
                      const int32_t* q_pos, void* out, const int64_t* out_strides, float* lse, void* workspace,
                      size_t workspace_bytes, void* stream) {
  int r;
  if ((r = check_shape(B, H, Tk, D))) return r;
  if (B > 65535 || H > 65535) return fail(-1, "B and H must not exceed 65535 for the decoding call");
  if (!(scale > 0.f)) return fail(-8, "scale must be positive");
  if ((r = check_tensor("q", q, q_strides)) || (r = check_tensor("k_cache", k_cache, k_strides)) ||
      (r = check_tensor("v_cache", v_cache, v_strides)) || (r = check_tensor("out", out, out_strides)))
    return r;
  if (lse == nullptr) return fail(-3, "lse: null pointer");
  if ((r = check_mask(doc_ids, link_bits, R, W))) return r;
  if (workspace == nullptr || !aligned(workspace, 256)) return fail(-9, "workspace must be a 256-byte aligned device buffer");
  if (workspace_bytes < decode_workspace_bytes(B, H, Tk, D))
    return fail(-9, "workspace too small: %zu < %zu", workspace_bytes, decode_workspace_bytes(B, H, Tk, D));
  r = launch_decode(q, k_cache, v_cache, q_strides, k_strides, v_strides, B, H, Tk, D, scale,
                    mask_args(doc_ids, q_row_ids, kv_col_ids, link_bits, R, W), q_pos, out, out_strides, lse, workspace,
                    static_cast<cudaStream_t>(stream));
  if (r) return fail(r, "decode launch failed (code %d, CUDA: %s)", r, cudaGetErrorString(cudaPeekAtLastError()));
  return 0;
}

size_t ts2ts_attn_bwd_workspace_bytes(int B, int H, int T, int D) {
  if (B <= 0 || H <= 0 || T <= 0 || T > kMaxT || (D != 64 && D != 128)) return 0;
  return bwd_workspace_bytes(B, H, T, D);
}

int ts2ts_attn_bwd(const void* q, const void* k, const void* v, const void* out, const void* dout, const float* lse,
                   const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides, const int64_t* out_strides,
                   const int64_t* dout_strides, int B, int H, int T, int D, float scale, const int32_t* doc_ids,
                   const int32_t* q_row_ids, const int32_t* kv_col_ids, const int64_t* link_bits, int R, int W, const void* plan,
                   size_t plan_bytes, void* dq, void* dk, void* dv, const int64_t* dq_strides, const int64_t* dk_strides,
                   const int64_t* dv_strides, void* workspace, size_t workspace_bytes, void* stream) {
  int r;
  if ((r = check_shape(B, H, T, D))) return r;
  if (!(scale > 0.f)) return fail(-8, "scale must be positive");
  if ((r = check_tensor("q", q, q_strides)) || (r = check_tensor("k", k, k_strides)) || (r = check_tensor("v", v, v_strides)) ||
      (r = check_tensor("out", out, out_strides)) || (r = check_tensor("dout", dout, dout_strides)) ||
      (r = check_tensor("dq", dq, dq_strides)) || (r = check_tensor("dk", dk, dk_strides)) || (r = check_tensor("dv", dv, dv_strides)))
    return r;
  if (lse == nullptr) return fail(-3, "lse: null pointer");
  if ((r = check_mask(doc_ids, link_bits, R, W))) return r;
  if ((r = check_plan(plan, plan_bytes, B, T))) return r;
  if (workspace == nullptr || !aligned(workspace, 256)) return fail(-9, "workspace must be a 256-byte aligned device buffer");
  if (workspace_bytes < bwd_workspace_bytes(B, H, T, D))
    return fail(-9, "workspace too small: %zu < %zu", workspace_bytes, bwd_workspace_bytes(B, H, T, D));
  PlanView P = plan_view(const_cast<void*>(plan), B, T);
  r = launch_bwd(q, k, v, out, dout, lse, q_strides, k_strides, v_strides, out_strides, dout_strides, B, H, T, D, scale, P,
                 mask_args(doc_ids, q_row_ids, kv_col_ids, link_bits, R, W), dq, dk, dv, dq_strides, dk_strides, dv_strides,
                 workspace, static_cast<cudaStream_t>(stream));
  if (r) return fail(r, "backward launch failed (code %d, CUDA: %s)", r, cudaGetErrorString(cudaPeekAtLastError()));
  return 0;
}

size_t ts2ts_attn_bwd_noalloc_max_bytes(void) {
  void* ptr = nullptr;
  size_t bytes = 0;
  return bwd_static_scratch(&ptr, &bytes) == 0 ? bytes : 0;
}

int ts2ts_attn_bwd_noalloc(const void* q, const void* k, const void* v, const void* out, const void* dout, const float* lse,
                           const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                           const int64_t* out_strides, const int64_t* dout_strides, int B, int H, int T, int D, float scale,
                           const int32_t* doc_ids, const int32_t* q_row_ids, const int32_t* kv_col_ids, const int64_t* link_bits,
                           int R, int W, const void* plan, size_t plan_bytes, void* dq, void* dk, void* dv,
                           const int64_t* dq_strides, const int64_t* dk_strides, const int64_t* dv_strides, void* stream) {
  int r;
  if ((r = check_shape(B, H, T, D))) return r;
  void* scratch = nullptr;
  size_t scratch_bytes = 0;
  if ((r = bwd_static_scratch(&scratch, &scratch_bytes)))
    return fail(r, "could not resolve the built-in scratch array on this device: %s", cudaGetErrorString(cudaPeekAtLastError()));
  const size_t need = bwd_workspace_bytes(B, H, T, D);
  if (need > scratch_bytes)
    return fail(-10, "this problem needs %zu bytes of scratch but the built-in array holds %zu; use ts2ts_attn_bwd with a "
                     "caller-owned workspace", need, scratch_bytes);
  return ts2ts_attn_bwd(q, k, v, out, dout, lse, q_strides, k_strides, v_strides, out_strides, dout_strides, B, H, T, D, scale,
                        doc_ids, q_row_ids, kv_col_ids, link_bits, R, W, plan, plan_bytes, dq, dk, dv, dq_strides, dk_strides,
                        dv_strides, scratch, scratch_bytes, stream);
}

size_t ts2ts_detect_links_scratch_bytes(int T) {
  if (T <= 0 || T > kMaxT) return 0;
  return (link_scan_scratch_ints(T) * sizeof(int32_t) + 255) & ~static_cast<size_t>(255);
}

int ts2ts_detect_links(const void* tokens, int token_bytes, int T, int64_t mid_id, const int64_t* start_ids, int n_start,
                       const uint8_t* close_flags, int vocab, int back_limit, int window, void* scratch, size_t scratch_bytes,
                       int32_t* links, int max_links, int32_t* count, void* stream) {
  if (T <= 0 || T > kMaxT) return fail(-1, "T must be in 1..%d (got %d)", kMaxT, T);
  if (token_bytes != 4 && token_bytes != 8) return fail(-2, "token_bytes must be 4 or 8 (got %d)", token_bytes);
  if (tokens == nullptr || !aligned(tokens, (size_t)token_bytes)) return fail(-3, "tokens: null or misaligned pointer");
  if (start_ids == nullptr || n_start <= 0 || n_start > kMaxStartIds)
    return fail(-6, "between 1 and %d start ids are needed (got %d)", kMaxStartIds, n_start);
  if (close_flags == nullptr || vocab <= 0) return fail(-6, "close_flags is null or vocab=%d is not positive", vocab);
  if (back_limit < 0 || window < 0) return fail(-6, "back_limit and window must not be negative");
  if (scratch == nullptr || !aligned(scratch, 16) || scratch_bytes < ts2ts_detect_links_scratch_bytes(T))
    return fail(-9, "scratch must be 16-byte aligned and hold %zu bytes", ts2ts_detect_links_scratch_bytes(T));
  if (links == nullptr || count == nullptr || max_links <= 0) return fail(-3, "links / count: null pointer or max_links <= 0");
  LinkScanArgs a;
  a.tokens = tokens; a.token_bytes = token_bytes; a.T = T; a.mid_id = mid_id; a.n_start = n_start;
  for (int i = 0; i < kMaxStartIds; ++i) a.start_ids[i] = i < n_start ? start_ids[i] : 0;
  a.close_flags = close_flags; a.vocab = vocab; a.back_limit = back_limit; a.window = window;
  cudaError_t e = launch_link_scan(a, static_cast<int32_t*>(scratch), links, max_links, count, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(-50, "link scan launch failed: %s", cudaGetErrorString(e));
  return 0;
}

int ts2ts_read_status(const void* plan, void* stream, int32_t* status_out) {
  if (plan == nullptr || status_out == nullptr) return fail(-3, "null pointer");
  cudaError_t e = cudaMemcpyAsync(status_out, plan, sizeof(int32_t), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream));
  if (e == cudaSuccess) e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(-60, "status read failed: %s", cudaGetErrorString(e));
  if (*status_out != 0)
    return fail(*status_out > 0 ? *status_out : -61, "a kernel recorded status %d (19xx / 29xx: the plan was not built for this call; "
                "otherwise 1000 / 2000 + the wait that ran out in the forward / backward kernel)", *status_out);
  return 0;
}

int ts2ts_profile_enable(int on) {
  ProfileSlot& s = profile_slot();
  if (on && s.start[0] == nullptr) {
    for (int i = 0; i < 2; ++i)
      if (cudaEventCreate(&s.start[i]) != cudaSuccess || cudaEventCreate(&s.stop[i]) != cudaSuccess)
        return fail(-70, "could not create timing events: %s", cudaGetErrorString(cudaGetLastError()));
  }
  s.enabled = on != 0;
  s.recorded[0] = s.recorded[1] = false;
  return 0;
}

int ts2ts_profile_last_ms(int which, float* ms) {
  ProfileSlot& s = profile_slot();
  if (ms == nullptr || which < 0 || which > 1) return fail(-3, "bad arguments");
  if (!s.enabled || !s.recorded[which]) return fail(-71, "no timed launch recorded");
  cudaError_t e = cudaEventSynchronize(s.stop[which]);
  if (e == cudaSuccess) e = cudaEventElapsedTime(ms, s.start[which], s.stop[which]);
  if (e != cudaSuccess) return fail(-72, "event timing failed: %s", cudaGetErrorString(e));
  return 0;
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------ decoder-layer pieces (ts2ts_lm.h)
namespace {
constexpr int64_t kMaxRows = int64_t(1) << 30;
int check_rows(int64_t N) { return (N <= 0 || N > kMaxRows) ? fail(-1, "N must be in 1..2^30 (got %lld)", (long long)N) : 0; }
int launched(cudaError_t e, const char* what) { return e == cudaSuccess ? 0 : fail(-50, "%s launch failed: %s", what, cudaGetErrorString(e)); }
}  // namespace

int ts2ts_add_rmsnorm_fwd(const float* x_in, const void* a, const float* w, float* x_out, void* h, float* rstd, int64_t N, int C,
                          float eps, void* stream) {
  int r;
  if ((r = check_rows(N))) return r;
  if (C < 4 || C > 16384 || C % 4) return fail(-2, "C must be a multiple of 4 in 4..16384 (got %d)", C);
  if (!(eps >= 0.f)) return fail(-8, "eps must not be negative");
  if (!x_in || !w || !x_out || !h || !rstd) return fail(-3, "add_rmsnorm_fwd: null pointer");
  if (!aligned(x_in, 16) || !aligned(x_out, 16) || !aligned(w, 16) || !aligned(h, 8) || (a && !aligned(a, 8)))
    return fail(-5, "add_rmsnorm_fwd: misaligned pointer");
  return launched(launch_add_rmsnorm_fwd(x_in, a, w, x_out, h, rstd, (int)N, C, eps, static_cast<cudaStream_t>(stream)), "add_rmsnorm_fwd");
}

size_t ts2ts_add_rmsnorm_bwd_workspace_bytes(int64_t N, int C) {
  if (N <= 0 || N > kMaxRows || C < 4 || C > 16384 || C % 4) return 0;
  return (size_t)add_rmsnorm_bwd_blocks(N, C) * C * sizeof(float);
}

int ts2ts_add_rmsnorm_bwd(const void* dh, const float* dx_up, const float* x, const float* w, const float* rstd, float* dx, void* da,
                          float* dw, void* workspace, size_t workspace_bytes, int64_t N, int C, void* stream) {
  int r;
  if ((r = check_rows(N))) return r;
  if (C < 4 || C > 16384 || C % 4) return fail(-2, "C must be a multiple of 4 in 4..16384 (got %d)", C);
  if (!dh || !x || !w || !rstd || !dx || !dw || !workspace) return fail(-3, "add_rmsnorm_bwd: null pointer");
  if (!aligned(dh, 8) || !aligned(x, 16) || !aligned(w, 16) || !aligned(dx, 16) || (dx_up && !aligned(dx_up, 16)) || (da && !aligned(da, 8)) ||
      !aligned(workspace, 16))
    return fail(-5, "add_rmsnorm_bwd: misaligned pointer");
  if (workspace_bytes < ts2ts_add_rmsnorm_bwd_workspace_bytes(N, C)) return fail(-4, "add_rmsnorm_bwd: workspace too small");
  return launched(launch_add_rmsnorm_bwd(dh, dx_up, x, w, rstd, dx, da, dw, static_cast<float*>(workspace), (int)N, C,
                                         static_cast<cudaStream_t>(stream)), "add_rmsnorm_bwd");
}

int ts2ts_rope_qk_inplace(void* qkv, const float* cos, const float* sin, int B, int T, int H, int D, float sign, void* stream) {
  if (B <= 0 || T <= 0 || H <= 0 || T > kMaxT) return fail(-1, "B, T, H must be positive (T <= %d)", kMaxT);
  if (D < 16 || D > 512 || D % 16) return fail(-2, "D must be a multiple of 16 in 16..512 (got %d)", D);
  if (!qkv || !cos || !sin) return fail(-3, "rope_qk_inplace: null pointer");
  if (!aligned(qkv, 16) || !aligned(cos, 16) || !aligned(sin, 16)) return fail(-5, "rope_qk_inplace: misaligned pointer");
  if (sign != 1.f && sign != -1.f) return fail(-8, "sign must be +1 or -1");
  return launched(launch_rope_qk(qkv, cos, sin, B, T, H, D, sign, static_cast<cudaStream_t>(stream)), "rope_qk");
}

int ts2ts_swiglu_fwd(const void* gu, void* act, int64_t N, int F, void* stream) {
  int r;
  if ((r = check_rows(N))) return r;
  if (F < 8 || F % 8) return fail(-2, "F must be a positive multiple of 8 (got %d)", F);
  if (!gu || !act) return fail(-3, "swiglu_fwd: null pointer");
  if (!aligned(gu, 16) || !aligned(act, 16)) return fail(-5, "swiglu_fwd: misaligned pointer");
  return launched(launch_swiglu_fwd(gu, act, N, F, static_cast<cudaStream_t>(stream)), "swiglu_fwd");
}

int ts2ts_swiglu_bwd(const void* gu, const void* dact, void* dgu, int64_t N, int F, void* stream) {
  int r;
  if ((r = check_rows(N))) return r;
  if (F < 8 || F % 8) return fail(-2, "F must be a positive multiple of 8 (got %d)", F);
  if (!gu || !dact || !dgu) return fail(-3, "swiglu_bwd: null pointer");
  if (!aligned(gu, 16) || !aligned(dact, 16) || !aligned(dgu, 16)) return fail(-5, "swiglu_bwd: misaligned pointer");
  return launched(launch_swiglu_bwd(gu, dact, dgu, N, F, static_cast<cudaStream_t>(stream)), "swiglu_bwd");
}

int ts2ts_ce_fwd(const void* logits, const int64_t* target, float* lse, float* loss, int64_t N, int V, void* stream) {
  int r;
  if ((r = check_rows(N))) return r;
  if (V < 8 || V % 8) return fail(-2, "V must be a positive multiple of 8 (got %d)", V);
  if (!logits || !target || !lse || !loss) return fail(-3, "ce_fwd: null pointer");
  if (!aligned(logits, 16)) return fail(-5, "ce_fwd: misaligned pointer");
  return launched(launch_ce_fwd(logits, target, lse, loss, (int)N, V, static_cast<cudaStream_t>(stream)), "ce_fwd");
}

int ts2ts_ce_bwd(void* logits, const int64_t* target, const float* lse, const float* gscale, float inv_n, int64_t N, int V,
                 void* stream) {
  int r;
  if ((r = check_rows(N))) return r;
  if (V < 8 || V % 8) return fail(-2, "V must be a positive multiple of 8 (got %d)", V);
  if (!logits || !target || !lse || !gscale) return fail(-3, "ce_bwd: null pointer");
  if (!aligned(logits, 16)) return fail(-5, "ce_bwd: misaligned pointer");
  return launched(launch_ce_bwd(logits, target, lse, gscale, inv_n, (int)N, V, static_cast<cudaStream_t>(stream)), "ce_bwd");
}
