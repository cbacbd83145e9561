/* libts2ts_attn -- C ABI of the sm_100a masked flash-attention path.
 *
 * The entry points replace, for TAGSeq2TAGSeq's attention hot path, what the
 * reference reaches through two Python seams (it has no FFI of its own):
 *   - the block_mask_creator callable injected into TS2TSTrainingModule
 *     (model/modules/training_module.py:36-65,199-200), which ends in torch's
 *     create_block_mask (model/graph_traversal/block_mask_creator.py:132-139,
 *     model/graph_traversal/cross_doc_mask.py:359-366);
 *   - the flex_attention symbol called by the attention module
 *     (model/modules/layer.py:33; patched at generate.py:167-178).
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless its comment says "host";
 *   - `stream` is a cudaStream_t passed as void*; all work is enqueued on it and
 *     the call returns without synchronising (ts2ts_read_status synchronises);
 *   - the caller owns every buffer; the library allocates no device memory;
 *   - return value 0 = OK, < 0 = rejected arguments or launch failure (nothing
 *     or only part of the work was enqueued; ts2ts_last_error_string() explains),
 *     > 0 only from ts2ts_read_status = code recorded by a kernel whose bounded
 *     wait ran out;
 *   - tensors q, k, v, out, dout, dq, dk, dv are bf16 [B,H,T,D] with D in
 *     {64, 128} contiguous and element strides {batch, head, token} given in
 *     a host int64_t[3]; base pointers and byte strides are multiples of 16;
 *   - the mask is
 *         allowed(q, kv) = q >= kv  and  ( doc_ids[q] == doc_ids[kv]
 *                          or  bit( link_bits[b, q_row_ids[q], :], kv_col_ids[kv] ) )
 *     with a negative or out-of-range class granting nothing.  link_bits == NULL
 *     is the reference's `doc_causal` mask; with link_bits it expresses
 *     `cross_doc_link` (cross_doc_mask.py:348-357).  q_row_ids / kv_col_ids may
 *     be NULL, meaning doc_ids are used as class numbers.
 */
#ifndef TS2TS_ATTN_H_
#define TS2TS_ATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TS2TS_TILE 128

/* Library version (major*1000 + minor). */
int ts2ts_version(void);

/* Host string describing the last non-zero return on the calling thread. */
const char* ts2ts_last_error_string(void);

/* Size in bytes of the block plan for B sequences of T tokens (0 if B or T is invalid). */
size_t ts2ts_plan_bytes(int B, int T);

/* Integer pre-pass.  Fills `plan` (ts2ts_plan_bytes(B,T) bytes, 256-byte aligned), which the
 * attention calls below read, from the per-token mask inputs:
 *   doc_ids    int32[B,T]
 *   q_row_ids  int32[B,T] or NULL     kv_col_ids int32[B,T] or NULL
 *   link_bits  int64[B,R,W] or NULL   (bit c%64 of word c/64 of row r)
 * Optional outputs (any may be NULL), NB = ceil(T/128), in the layout of torch's BlockMask
 * that create_block_mask returns to the reference (torch/nn/attention/flex_attention.py:1207-1289):
 *   state      uint8[B,NB,NB]   0 skip, 1 partial, 2 full, indexed [b, q tile, kv tile]
 *   kv_cnt     int32[B,NB]      kv_idx     int32[B,NB,NB]   partial kv tiles of a q tile, ascending, then -1
 *   full_cnt   int32[B,NB]      full_idx   int32[B,NB,NB]   full kv tiles
 *   q_cnt      int32[B,NB]      q_idx      int32[B,NB,NB]   partial q tiles of a kv tile
 *   full_q_cnt int32[B,NB]      full_q_idx int32[B,NB,NB]   full q tiles of a kv tile */
int ts2ts_block_map(const int32_t* doc_ids, const int32_t* q_row_ids, const int32_t* kv_col_ids,
                    const int64_t* link_bits, int B, int T, int R, int W, void* plan, size_t plan_bytes,
                    uint8_t* state, int32_t* kv_cnt, int32_t* kv_idx, int32_t* full_cnt, int32_t* full_idx,
                    int32_t* q_cnt, int32_t* q_idx, int32_t* full_q_cnt, int32_t* full_q_idx, void* stream);

/* Per-token class ids from a table of segments, filled on the device: out[t] = ids[j] for bounds[j] <= t < bounds[j+1]
 * (bounds: device int32[n_seg + 1], ascending; ids: device int32[n_seg]), -1 for tokens before bounds[0] or from
 * bounds[n_seg] on.  With the segments cut at the start and end of every grant this writes q_row_ids / kv_col_ids of
 * the cross_doc_link mask; it replaces the per-grant slice assignments into [T]-long int64 bit tensors of
 * _build_grant_bitmasks (model/graph_traversal/cross_doc_mask.py:258-294).  out: device int32[T]. */
int ts2ts_segment_ids(const int32_t* bounds, const int32_t* ids, int n_seg, int T, int32_t* out, void* stream);

/* Forward: out = softmax(scale * q k^T + mask) v, lse = natural-log row sums, fp32 [B,H,T].
 * A row with no allowed key gets out = 0 and lse = -inf.  Replaces the forward of
 * flex_attention(q, k, v, block_mask=...) (torch/nn/attention/flex_attention.py:1468). */
int ts2ts_attn_fwd(const void* q, const void* k, const void* v, const int64_t* q_strides, const int64_t* k_strides,
                   const int64_t* v_strides, int B, int H, int T, int D, float scale, const int32_t* doc_ids,
                   const int32_t* q_row_ids, const int32_t* kv_col_ids, const int64_t* link_bits, int R, int W,
                   const void* plan, size_t plan_bytes, void* out, const int64_t* out_strides, float* lse, void* stream);

/* Attention of ONE new token per sequence against cached keys and values (decoding with KV reuse).  The reference
 * recomputes the whole forward for every generated token (model/generation_loop.py:90-92, model/model.py:214-237)
 * and lists KV caching as not implemented (GENERATION_FEATURE_SPEC.md:163); this call computes the one row it needs.
 *   q            bf16 [B,H,1,D], strides {batch, head, (ignored)}
 *   k_cache, v_cache   bf16 [B,H,Tk,D] holding the keys / values of tokens 0 .. Tk-1, the new token's included
 *   doc_ids, q_row_ids, kv_col_ids   int32 [B,Tk] (classes of every cached token; the query's are those at q_pos)
 *   q_pos        device int32[B]: position of the query token, or NULL = Tk - 1
 *   out          bf16 [B,H,1,D]; lse fp32 [B,H] natural log; a token that may read no key gets out = 0, lse = -inf
 *   workspace    ts2ts_attn_decode_workspace_bytes(B,H,Tk,D) bytes, 256-byte aligned
 * Keys after q_pos are never read.  No block plan is needed: the mask row is evaluated per key. */
size_t ts2ts_attn_decode_workspace_bytes(int B, int H, int Tk, int D);
int ts2ts_attn_decode(const void* q, const void* k_cache, const void* v_cache, const int64_t* q_strides,
                      const int64_t* k_strides, const int64_t* v_strides, int B, int H, int Tk, int D, float scale,
                      const int32_t* doc_ids, const int32_t* q_row_ids, const int32_t* kv_col_ids,
                      const int64_t* link_bits, int R, int W, const int32_t* q_pos, void* out,
                      const int64_t* out_strides, float* lse, void* workspace, size_t workspace_bytes, void* stream);

/* Scratch size in bytes that ts2ts_attn_bwd needs. */
size_t ts2ts_attn_bwd_workspace_bytes(int B, int H, int T, int D);

/* Backward of the call above: given out, lse and dout computes dq, dk, dv (bf16, own strides).
 * `workspace` is caller-owned scratch of ts2ts_attn_bwd_workspace_bytes() bytes, 256-byte aligned;
 * its contents need not be preserved between calls.  Replaces the autograd backward of
 * flex_attention (torch/_higher_order_ops/flex_attention.py:947-1075). */
int ts2ts_attn_bwd(const void* q, const void* k, const void* v, const void* out, const void* dout, const float* lse,
                   const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                   const int64_t* out_strides, const int64_t* dout_strides, int B, int H, int T, int D, float scale,
                   const int32_t* doc_ids, const int32_t* q_row_ids, const int32_t* kv_col_ids,
                   const int64_t* link_bits, int R, int W, const void* plan, size_t plan_bytes, void* dq, void* dk,
                   void* dv, const int64_t* dq_strides, const int64_t* dk_strides, const int64_t* dv_strides,
                   void* workspace, size_t workspace_bytes, void* stream);

/* Backward without any caller-provided or freshly allocated scratch.  It has no counterpart in the reference.
 *
 * Who needs it: hosts that cannot obtain device memory at the moment of the call -- a process whose whole HBM
 * was handed to another allocator at start-up, a plug-in that may not call cudaMalloc because that call
 * synchronises the device and would stall unrelated streams, or a C caller with no allocator of its own.
 * For them the scratch of ts2ts_attn_bwd (fp32 dQ accumulator, delta, scaled LSE) lives in one array compiled
 * into the library; every GPU that loads the library keeps that array until the process ends.
 *
 * Same arguments and results as ts2ts_attn_bwd, minus the workspace.  Limits and rules:
 *   - the problem must satisfy ts2ts_attn_bwd_workspace_bytes(B,H,T,D) <= ts2ts_attn_bwd_noalloc_max_bytes()
 *     (64 MiB, e.g. H * ceil(T/128)*128 <= 129055 rows at D = 128); larger problems are rejected with -10;
 *   - set-up, once per device at start-up: call ts2ts_attn_bwd_noalloc_max_bytes() with that device current.  It
 *     looks up the array's device address (cudaGetSymbolAddress) and caches it; with CUDA's lazy module loading
 *     this is also the moment the module that holds the 64 MiB array is loaded and the array gets its memory, and
 *     the look-up may synchronise the device.  So make this call BEFORE the rest of the GPU's memory is handed to
 *     another allocator (afterwards the load can fail with -131) and before any stream capture.  The first
 *     ts2ts_attn_bwd_noalloc on a device does the same set-up if it was skipped.  The cache is indexed by device
 *     ordinal: after cudaDeviceReset, or in a second context on the same device, the cached address is stale and
 *     the process must not use this entry point again;
 *   - once set up, the call allocates nothing: no cudaMalloc / cudaFree and no allocating library routine, and
 *     the amount of free device memory is the same before and after it;
 *   - all calls on a device share the one array, which still holds the previous call's values: each call
 *     re-zeroes the accumulator part and rewrites the rest before use, and two calls whose kernels can
 *     overlap on the GPU (different streams without ordering) race -- serialise them. */
size_t ts2ts_attn_bwd_noalloc_max_bytes(void);
int ts2ts_attn_bwd_noalloc(const void* q, const void* k, const void* v, const void* out, const void* dout,
                           const float* lse, const int64_t* q_strides, const int64_t* k_strides,
                           const int64_t* v_strides, const int64_t* out_strides, const int64_t* dout_strides, int B,
                           int H, int T, int D, float scale, const int32_t* doc_ids, const int32_t* q_row_ids,
                           const int32_t* kv_col_ids, const int64_t* link_bits, int R, int W, const void* plan,
                           size_t plan_bytes, void* dq, void* dk, void* dv, const int64_t* dq_strides,
                           const int64_t* dk_strides, const int64_t* dv_strides, void* stream);

/* Candidate markdown links "[text](target)" of one token sequence, found on the device.  Replaces the scan of
 * MarkdownLinkDetector.detect_links (model/graph_traversal/markdown_link_detector.py:57-108), which reads tokens
 * one by one on the host:
 *   tokens       device, int32[T] (token_bytes = 4) or int64[T] (token_bytes = 8)
 *   mid_id       id of the "](" token (`:45`); start_ids / n_start (<= 8): ids that can be "[" (`:43-44`), host array
 *   close_flags  device uint8[vocab]: 1 when the token's bytes contain ')'
 *   back_limit   how far back "[" is looked for (100 in the reference, `:74`); window: `window_tokens` (`:88`)
 *   scratch      device, ts2ts_detect_links_scratch_bytes(T) bytes, 16-byte aligned
 *   links        device int32[max_links][3]: (position of "](", position of "[", position of the token that closes the
 *                link), ascending by position -- the order in which the reference appends its links
 *   count        device int32: candidates found (may exceed max_links; only max_links triples are stored)
 * A "](" without "[" in reach or without a closing token inside the window gives no triple, as in the reference.
 * Decoding the target tokens (positions mid+1 .. close) and the non-empty test (`:94-97`) stay with the caller. */
size_t ts2ts_detect_links_scratch_bytes(int T);
int ts2ts_detect_links(const void* tokens, int token_bytes, int T, int64_t mid_id, const int64_t* start_ids, int n_start,
                       const uint8_t* close_flags, int vocab, int back_limit, int window, void* scratch,
                       size_t scratch_bytes, int32_t* links, int max_links, int32_t* count, void* stream);

/* Waits for `stream`, then copies the plan's device status word to *status_out (host).
 * 0 = every kernel that used this plan since the last ts2ts_block_map ran to completion. */
int ts2ts_read_status(const void* plan, void* stream, int32_t* status_out);

/* Kernel timing for benchmarks.  ts2ts_profile_enable(1) makes the forward and backward calls on the
 * current device bracket their MAIN kernel (not the small preparation / conversion launches) with CUDA
 * events on the caller's stream; ts2ts_profile_last_ms waits for those events and returns the elapsed
 * milliseconds of the last forward (which = 0) or backward (which = 1) main kernel in *ms (host).
 * Has no counterpart in the reference (it times whole phases in profile_training.py:354-375). */
int ts2ts_profile_enable(int on);
int ts2ts_profile_last_ms(int which, float* ms);

#ifdef __cplusplus
}
#endif
#endif /* TS2TS_ATTN_H_ */
