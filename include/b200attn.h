/*
 * b200attn — causal grouped-query attention for NVIDIA B200 (sm_100a), C ABI.
 *
 * Drop-in boundary for the flash-attention entry points of AlsoTheZv3n/modern-llm-v1
 * (paths relative to that project's root).  Every function returns an int status
 * (0 = B200ATTN_OK), never throws and never aborts; kernels are enqueued on the
 * given CUDA stream and the call returns without synchronising.
 *
 * Data types: q, k, v, o, dout, dq, dk, dv are device pointers to BF16 stored as
 * 16-bit words (the reference's BF16 storage, llm/src/core/dtype.h:34-49); lse is
 * FP32.  All accumulation is FP32.
 *
 * Layouts (element strides, unit stride on the head dimension D):
 *   B200ATTN_LAYOUT_BHTD  [B, H, T, D] — the reference's "split" layout
 *                         [B*H, T, D] (llm/src/model/attention.h:39-46)
 *   B200ATTN_LAYOUT_BTHD  [B, T, H, D] — the projection output [B, T, H*D]
 *                         read in place, so split_heads / merge_heads
 *                         (llm/src/model/attention.cu:344-386) are not needed.
 * q, o, dout, dq have H = Hq heads; k, v, dk, dv have H = Hkv heads.  Query head h
 * reads KV head h / (Hq / Hkv) (llm/src/model/attention.cu:406); nothing is
 * replicated, which replaces repeat_kv_heads / accumulate_kv_grads
 * (llm/src/model/attention.cu:481-543).
 *
 * Constraints (checked, B200ATTN_ERR_* otherwise): D in {64, 128}; Hq % Hkv == 0;
 * all sizes > 0; base pointers 16-byte aligned.
 */
#ifndef B200ATTN_H_
#define B200ATTN_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    B200ATTN_OK = 0,
    B200ATTN_ERR_INVALID_ARG = 1,  /* null pointer, non-positive size, Hq % Hkv != 0, bad layout */
    B200ATTN_ERR_UNSUPPORTED = 2,  /* head dimension other than 64 / 128 */
    B200ATTN_ERR_ALIGNMENT = 3,    /* a base pointer is not 16-byte aligned */
    B200ATTN_ERR_WORKSPACE = 4,    /* workspace missing or too small */
    B200ATTN_ERR_CUDA = 5,         /* a CUDA runtime call or a launch failed */
    B200ATTN_ERR_TENSOR_MAP = 6,   /* the driver refused a TMA tensor map */
    B200ATTN_ERR_DEVICE_WAIT = 7,  /* a kernel gave up on a bounded wait (see b200attn_last_device_status) */
    B200ATTN_ERR_NO_DEVICE = 8,    /* no sm_100 device is current */
    B200ATTN_ERR_TOO_LARGE = 9     /* problem too large: beyond the fixed scratch of b200attn_bwd_static (524288 rows), or
                                      2^31 or more rows in a RoPE / QK-Norm / KV-append call */
};

enum { B200ATTN_LAYOUT_BHTD = 0, B200ATTN_LAYOUT_BTHD = 1 };

/*
 * Forward: o = softmax(softmax_scale * q k^T, causal) v and lse[b, h, t] = logsumexp of
 * the scaled scores of row t (natural log), lse laid out [B, Hq, T] contiguous.
 * Replaces flash_attn_forward (llm/src/model/flash_attn.h:25-28,
 * llm/src/model/flash_attn.cu:383-426); the reference fixes
 * softmax_scale = 1/sqrt(D) (llm/src/model/flash_attn.cu:418) — pass 0 to get that.
 */
int b200attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int T, int Hq, int Hkv, int D,
                 int layout, float softmax_scale, void* stream);

/*
 * Backward: dq, dk, dv (overwritten, not accumulated) from q, k, v, o, lse, dout.
 * Replaces flash_attn_backward (llm/src/model/flash_attn.h:47-52,
 * llm/src/model/flash_attn.cu:428-504): a dQ pass (which also computes D = rowsum(o * dout)) and
 * a dK/dV pass.  dk/dv are already summed over the query heads of each KV group (what
 * accumulate_kv_grads does in the reference, llm/src/model/attention.cu:510-543),
 * in a fixed order, so dk and dv are bit-reproducible; dq is too in the two-pass mode (see
 * b200attn_bwd_mode below for the modes and which one this call picks).  The reference allocates its
 * D vector per call (llm/src/model/flash_attn.cu:463); here the caller passes a
 * workspace of at least b200attn_bwd_workspace_bytes(...) bytes, 256-byte aligned.
 */
int b200attn_bwd(const void* q, const void* k, const void* v, const void* o, const float* lse, const void* dout,
                 void* dq, void* dk, void* dv, int B, int T, int Hq, int Hkv, int D, int layout, float softmax_scale,
                 void* workspace, size_t workspace_bytes, void* stream);
size_t b200attn_bwd_workspace_bytes(int B, int T, int Hq, int Hkv, int D);

/*
 * The same backward with the algorithm chosen by the caller (b200attn_bwd is mode B200ATTN_BWD_AUTO).
 *
 * B200ATTN_BWD_TWO_PASS: the structure of the reference (llm/src/model/flash_attn.cu:475-503): a dQ pass and a
 *   dK/dV pass that each recompute the scores.  No atomics anywhere: dq, dk and dv are bit-reproducible.
 *   Workspace: two FP32 row vectors, 2 * B * Hq * ceil(T/128)*128 * 4 bytes.
 * B200ATTN_BWD_ONE_PASS (D = 64 only, B200ATTN_ERR_UNSUPPORTED otherwise): one key-stationary kernel computes the
 *   scores once and produces dk, dv and the dq contributions together; the contributions of different key tiles
 *   to one query tile are summed in an FP32 accumulator in the workspace by reduce-adds whose order is not fixed,
 *   so dq is reproducible only to FP32 rounding (dk and dv stay bit-reproducible).  Five products and one
 *   exponential per score instead of seven and two, but measured slower than TWO_PASS below T = 4096 on B200
 *   (both are bound by shared-memory traffic, which is the same).  Workspace: the two row vectors plus
 *   B * Hq * ceil(T/128)*128 * D * 4 bytes.
 * B200ATTN_BWD_AUTO: TWO_PASS, unless the environment variable B200ATTN_BWD=two_pass|one_pass (read once) says
 *   otherwise.  If the workspace passed is too small for ONE_PASS but holds the two row vectors, AUTO runs TWO_PASS.
 * b200attn_bwd_workspace_bytes_mode gives the size for a mode (for AUTO: of the algorithm AUTO picks).
 */
enum { B200ATTN_BWD_AUTO = 0, B200ATTN_BWD_TWO_PASS = 1, B200ATTN_BWD_ONE_PASS = 2 };
int b200attn_bwd_mode(const void* q, const void* k, const void* v, const void* o, const float* lse, const void* dout,
                      void* dq, void* dk, void* dv, int B, int T, int Hq, int Hkv, int D, int layout,
                      float softmax_scale, int mode, void* workspace, size_t workspace_bytes, void* stream);
size_t b200attn_bwd_workspace_bytes_mode(int B, int T, int Hq, int Hkv, int D, int mode);

/*
 * Backward without a workspace argument and without any allocation (this entry point has no
 * counterpart in the reference, whose backward allocates its D vector with cudaMalloc on every
 * call, llm/src/model/flash_attn.cu:463).
 *
 * Same inputs, outputs and results as b200attn_bwd_mode with B200ATTN_BWD_TWO_PASS (it runs the same kernels), but the two
 * per-row FP32 vectors the backward needs live in a fixed array inside the library's device
 * image instead of a caller-provided workspace.  It is meant for callers that cannot obtain
 * device memory at the point of the call: code that runs between training steps under a
 * caching allocator that must not see a raw cudaMalloc (which synchronises the whole device),
 * latency-critical loops that forbid any allocation after start-up, and hosts that have no
 * allocator of their own to hand a workspace from.  The library calls no cudaMalloc, cudaFree
 * or other allocating routine here.
 *
 * Limit: B * Hq * ceil(T / 128) * 128 <= B200ATTN_BWD_STATIC_MAX_ROWS (524288, i.e. up to the
 * long-context shape B=4, Hq=16, T=8192); larger problems return B200ATTN_ERR_TOO_LARGE and
 * launch nothing.  The array costs 4 MiB of device memory on every GPU that loads the library,
 * until the process exits.
 *
 * The first call on each device resolves the array's device address (with that device
 * current); make that first call before any stream capture begins.  All calls on a device
 * share the one array: it still holds the previous call's vectors when the next call starts
 * (every call rewrites all the rows it uses, so nothing has to be cleared), and two calls
 * whose kernels can overlap on the GPU - different streams, or graphs replayed concurrently -
 * race on it.  Serialise them, or use b200attn_bwd with one workspace per stream.
 */
#define B200ATTN_BWD_STATIC_MAX_ROWS 524288
int b200attn_bwd_static(const void* q, const void* k, const void* v, const void* o, const float* lse,
                        const void* dout, void* dq, void* dk, void* dv, int B, int T, int Hq, int Hkv, int D,
                        int layout, float softmax_scale, void* stream);

/*
 * Decode: one query token per sequence against a KV cache of L tokens (the cache
 * already holds the current token), split over the cache length.  q, o: [B, Hq, D]
 * contiguous BF16; kcache, vcache: [B, Hkv, L, D] contiguous BF16; lse [B, Hq] FP32 or
 * NULL.  Equals row L-1 of b200attn_fwd with T = L.  The reference has no such
 * path: infer_modern_gpt re-runs the full forward per token
 * (llm/apps/infer_modern_gpt.cu:253-255); this is the kernel its KV cache would call.
 * n_splits <= 0 lets the library choose.  workspace: at least
 * b200attn_decode_workspace_bytes(...) bytes, 256-byte aligned.
 */
int b200attn_decode(const void* q, const void* kcache, const void* vcache, void* o, float* lse, int B, int L, int Hq,
                    int Hkv, int D, float softmax_scale, int n_splits, void* workspace, size_t workspace_bytes,
                    void* stream);
size_t b200attn_decode_workspace_bytes(int B, int L, int Hq, int Hkv, int D, int n_splits);
/* The split count b200attn_decode uses for n_splits <= 0. */
int b200attn_decode_default_splits(int B, int L, int Hq, int Hkv, int D);

/* Element type of a projection output handed to the RoPE / QK-Norm / KV-cache calls. */
enum { B200ATTN_DTYPE_BF16 = 0, B200ATTN_DTYPE_F32 = 1 };

/*
 * KV cache for inference.  The reference's sampler keeps no cache: it re-runs the whole
 * forward per generated token (llm/apps/infer_modern_gpt.cu:13,253-255; TODO.md "KV cache
 * for inference").  These three calls are what a cached ModernGPT block needs around
 * attention.  Caches are [B, Hkv, L_cap, D] contiguous BF16; the B sequences advance in
 * lock step (one length for all).
 *
 * b200attn_kv_append: for the n_new newest tokens at positions pos0 .. pos0 + n_new - 1, does
 * what the block does before attention (llm/src/model/modern_gpt.cu:351-370: split_heads,
 * rope_apply_inplace, rmsnorm_forward on q and k), with RoPE at the TRUE positions, in one
 * launch: xq [B, n_new, Hq, D] -> q_out [B, Hq, n_new, D] BF16; xk, xv [B, n_new, Hkv, D] ->
 * rows pos0 .. of kcache (rotated, normalised, times gamma_k) and vcache (converted).  x_dtype:
 * B200ATTN_DTYPE_BF16 or _F32.  cos_t, sin_t: [>= pos0 + n_new, D / 2] FP32 (b200attn_rope_table).
 * A row gets the same bits as from b200attn_rope_norm_fwd at the same position.
 * pos0 + n_new > L_cap is B200ATTN_ERR_INVALID_ARG.
 *
 * b200attn_fwd_kvcache: b200attn_fwd over the first T positions with K and V read from the
 * caches where they lie (prefill: append n_new = T at pos0 = 0, then this).  q, o: [.., T, ..]
 * in q_layout.
 *
 * b200attn_decode_cached: b200attn_decode against the first L rows of caches of capacity L_cap
 * (b200attn_decode is the case L_cap == L).  Workspace as for b200attn_decode.
 */
int b200attn_kv_append(const void* xq, const void* xk, const void* xv, int x_dtype, void* q_out, void* kcache,
                       void* vcache, const float* gamma_q, const float* gamma_k, const float* cos_t,
                       const float* sin_t, int B, int n_new, int pos0, int L_cap, int Hq, int Hkv, int D, float eps,
                       void* stream);
int b200attn_fwd_kvcache(const void* q, const void* kcache, const void* vcache, void* o, float* lse, int B, int T,
                         int L_cap, int Hq, int Hkv, int D, int q_layout, float softmax_scale, void* stream);
int b200attn_decode_cached(const void* q, const void* kcache, const void* vcache, void* o, float* lse, int B, int L,
                           int L_cap, int Hq, int Hkv, int D, float softmax_scale, int n_splits, void* workspace,
                           size_t workspace_bytes, void* stream);
/*
 * Chunked prefill: T new tokens at positions pos0 .. pos0 + T - 1 attend over the pos0 tokens already cached and,
 * causally, over themselves (append them with b200attn_kv_append at pos0 first).  q, o: [.., T, ..] in q_layout;
 * lse [B, Hq, T].  Row t equals row pos0 + t of b200attn_fwd over pos0 + T tokens.  pos0 == 0 is
 * b200attn_fwd_kvcache; pos0 + T > L_cap is B200ATTN_ERR_INVALID_ARG.  (The sampler it serves re-runs the whole
 * window per token, llm/apps/infer_modern_gpt.cu:253-255.)
 */
int b200attn_fwd_kvcache_at(const void* q, const void* kcache, const void* vcache, void* o, float* lse, int B, int T,
                            int pos0, int L_cap, int Hq, int Hkv, int D, int q_layout, float softmax_scale,
                            void* stream);

/*
 * The same two calls for sequences of different lengths (a batch that does not advance in lock step).
 * b200attn_kv_append_at: pos [B] (device, int32) is the first position of each sequence's n_new tokens.  A
 * sequence whose pos[b] + n_new exceeds L_cap is skipped and sets the device status word to 105 (unless the word
 * already holds an earlier code).  While the status word is non-zero every kernel of this library on that device
 * returns at once without writing anything, although its launching call still returns B200ATTN_OK: check
 * b200attn_last_device_status (which reports the code and clears the word) before trusting later results.
 * b200attn_decode_ragged: lens [B] (device, int32), 1 <= lens[b] <= L, is each sequence's cache length
 * (the newest token included); L is the host's upper bound on them: it sizes the grid, the splits and the
 * workspace (b200attn_decode_workspace_bytes with this L).  Rows lens[b] .. L-1 of a sequence's caches are
 * read but carry no weight; they must hold finite values (a cache that starts zeroed does).  lens == NULL is
 * b200attn_decode_cached.
 */
int b200attn_kv_append_at(const void* xq, const void* xk, const void* xv, int x_dtype, void* q_out, void* kcache,
                          void* vcache, const float* gamma_q, const float* gamma_k, const float* cos_t,
                          const float* sin_t, const int* pos, int B, int n_new, int L_cap, int Hq, int Hkv, int D,
                          float eps, void* stream);
int b200attn_decode_ragged(const void* q, const void* kcache, const void* vcache, void* o, float* lse, const int* lens,
                           int B, int L, int L_cap, int Hq, int Hkv, int D, float softmax_scale, int n_splits,
                           void* workspace, size_t workspace_bytes, void* stream);


/*
 * Fused RoPE + per-head RMSNorm ("QK-Norm") that prepares q or k for b200attn_fwd, and its backward.
 * Replaces, per tensor, split_heads -> rope_apply_inplace -> rmsnorm_forward of the reference
 * (llm/src/model/modern_gpt.cu:351-370; llm/src/model/attention.cu:344-364, llm/src/model/rope.cu:146-163,
 * llm/src/model/rmsnorm.cu:24-53) and rmsnorm_backward -> rope_apply_backward_inplace -> merge_heads
 * (llm/src/model/modern_gpt.cu:527-552; llm/src/model/rmsnorm.cu:55-101, llm/src/model/rope.cu:46-65).
 *
 *   r = RoPE(x, t)  (interleaved pairs: r[2i] = x[2i] cos - x[2i+1] sin, r[2i+1] = x[2i] sin + x[2i+1] cos)
 *   rstd = 1 / sqrt(mean_d r[d]^2 + eps);   y[d] = r[d] * rstd * gamma[d]
 *
 * x: B*T*H rows of D elements, BF16 or FP32 (x_dtype), in either layout (x_layout; BTHD is the projection
 * output read in place).  y: BF16 in y_layout (what b200attn_fwd takes).  rstd: FP32 [B, H, T], the row order of
 * the reference's rstd vector.  gamma: FP32 [D].  cos_t, sin_t: FP32 [T, D/2] device tables with the values of
 * make_rope_cache (llm/src/model/rope.cu:112-128); b200attn_rope_table fills host copies of them.
 * Backward: dy BF16 in y_layout; dx in x's type and layout (overwritten); d_gamma FP32 [D] is ACCUMULATED into,
 * as in the reference (llm/src/model/rmsnorm.h:17), but in a fixed order (no atomics: bit-reproducible).
 * workspace: at least b200attn_rope_norm_bwd_workspace_bytes(D) bytes, 256-byte aligned.
 */
int b200attn_rope_table(int T, int D, float base, float* cos_host, float* sin_host);
int b200attn_rope_norm_fwd(const void* x, int x_dtype, int x_layout, void* y, int y_layout, float* rstd,
                           const float* gamma, const float* cos_t, const float* sin_t, int B, int T, int H, int D,
                           float eps, void* stream);
int b200attn_rope_norm_bwd(const void* dy, int y_layout, const void* x, int x_dtype, int x_layout, const float* rstd,
                           const float* gamma, const float* cos_t, const float* sin_t, void* dx, float* d_gamma, int B,
                           int T, int H, int D, void* workspace, size_t workspace_bytes, void* stream);
size_t b200attn_rope_norm_bwd_workspace_bytes(int D);
/*
 * The same for q and k in one launch each way (what the model does back to back, llm/src/model/modern_gpt.cu:358-370
 * and :527-544): q has Hq heads and its own gamma, k has Hkv heads and its own; type, layouts, tables, B, T, D and
 * eps are shared.  Results are bit-identical to two single calls; the workspace size is the same.
 */
int b200attn_rope_norm_fwd_qk(const void* xq, const void* xk, int x_dtype, int x_layout, void* yq, void* yk, int y_layout,
                              float* rstd_q, float* rstd_k, const float* gamma_q, const float* gamma_k,
                              const float* cos_t, const float* sin_t, int B, int T, int Hq, int Hkv, int D, float eps,
                              void* stream);
int b200attn_rope_norm_bwd_qk(const void* dyq, const void* dyk, int y_layout, const void* xq, const void* xk, int x_dtype,
                              int x_layout, const float* rstd_q, const float* rstd_k, const float* gamma_q,
                              const float* gamma_k, const float* cos_t, const float* sin_t, void* dxq, void* dxk,
                              float* d_gamma_q, float* d_gamma_k, int B, int T, int Hq, int Hkv, int D, void* workspace,
                              size_t workspace_bytes, void* stream);

/*
 * Diagnostics for benchmarks (no counterpart in the reference): when three CUDA events are
 * set, every following b200attn_bwd records them on its stream before the dQ pass (which also
 * computes D = rowsum(o * dout)), after it, and after the dK/dV pass, so a caller can time each
 * kernel of the backward.  Pass three NULLs to switch it off (the default).  The events stay
 * owned by the caller.
 */
int b200attn_set_bwd_profile_events(void* ev_start, void* ev_after_dq, void* ev_after_dkdv);
/* With a fourth event for the one-pass backward, which has three kernels: events are recorded before the
 * row-vector kernel, after it, after the fused kernel and after the dq conversion.  The two-pass backward
 * records the first three as above and leaves the fourth alone. */
int b200attn_set_bwd_profile_events4(void* ev0, void* ev1, void* ev2, void* ev3);

/*
 * The static deal of work items the forward and the dQ pass use when a problem has fewer than four items per
 * CTA (host arithmetic only, no device needed; for inspection and tests).  Items are (128-query tile, head,
 * batch), numbered heaviest first: item id covers query tile n_qtiles - 1 - id / n_groups (n_groups = B * Hq).
 * Writes per_cta (0: this shape uses the closed formula or the device-wide counter instead) and, for block c,
 * its item ids ids[c * per_cta .. + per_cta), ended by 0xffff; ids must hold n_ctas * 8 entries, n_ctas <= 296.
 */
int b200attn_item_deal(int n_groups, int n_qtiles, int T, int n_ctas, int item_cost, unsigned short* ids, int* per_cta);

/*
 * Synchronises `stream` and returns the device status word of the current device:
 * 0, or the code of the first bounded wait that gave up since the last call (101 load,
 * 102 tensor core, 103 softmax hand-off, 104 buffer free), or 105 when b200attn_kv_append_at met a
 * position beyond the cache capacity (the word is then cleared).  The reference surfaces execution errors at a later
 * synchronisation too (llm/src/core/cuda_check.h:31-45).
 */
int b200attn_last_device_status(void* stream);

/* Human-readable text for a status returned by this library. */
const char* b200attn_strerror(int status);

/* Library version, major * 100 + minor. */
int b200attn_version(void);

#ifdef __cplusplus
}
#endif
#endif /* B200ATTN_H_ */
