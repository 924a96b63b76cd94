// Source-compatible replacement of the reference's flash-attention entry points
// (llm/src/model/flash_attn.h:25-28,47-52) on top of the b200attn C ABI.
//
// This header is meant to be compiled INSIDE the reference tree (it includes the
// reference's own core/tensor.h), with libb200attn.so on the link line.  Differences
// from the reference's declarations, all additive:
//   * tensors are DType::BF16 (the engine's I/O type), L stays FP32;
//   * `tile_kv` / `tile` are validated like the reference (<= 0 throws) and then ignored;
//   * `_gqa` overloads take (B, T, Hq, Hkv, D) plus a layout and index the shared KV head
//     directly, which replaces repeat_kv_heads / accumulate_kv_grads / split_heads /
//     merge_heads around the call (llm/src/model/modern_gpt.cu:351-378, 505-552).
//   * every function takes a trailing `stream` (a cudaStream_t as void*; default: the legacy default stream the
//     reference launches on, llm/src/model/flash_attn.cu:420-425).
// Error behaviour is the reference's: std::invalid_argument for bad arguments,
// std::runtime_error for CUDA failures (llm/src/model/flash_attn.cu:386-407,
// llm/src/core/cuda_check.h:12-27).
// Private temporaries: where the reference allocates per call (llm/src/model/flash_attn.cu:463,
// llm/src/model/attention.cu:197,225), the backward here uses the library's fixed scratch (b200attn_bwd_static)
// when the problem fits it, and otherwise - like decode and the RoPE/QK-Norm backward - a workspace kept per
// (device, stream, operator) that only ever grows: in steady state no call allocates, frees or synchronises.
#pragma once

#include "core/tensor.h"

namespace modernllm {
namespace b200 {

enum class Layout { BHTD = 0, BTHD = 1 };

void flash_attn_forward(const Tensor& q, const Tensor& k, const Tensor& v, Tensor& ctx, Tensor& L, int B, int T, int D,
                        int tile_kv = 32, void* stream = nullptr);

void flash_attn_backward(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& ctx, const Tensor& L,
                         const Tensor& d_ctx, Tensor& d_q, Tensor& d_k, Tensor& d_v, int B, int T, int D,
                         int tile = 16, void* stream = nullptr);

void flash_attn_forward_gqa(const Tensor& q, const Tensor& k, const Tensor& v, Tensor& ctx, Tensor& L, int B, int T,
                            int Hq, int Hkv, int D, Layout layout = Layout::BHTD, void* stream = nullptr);

void flash_attn_backward_gqa(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& ctx, const Tensor& L,
                             const Tensor& d_ctx, Tensor& d_q, Tensor& d_k, Tensor& d_v, int B, int T, int Hq,
                             int Hkv, int D, Layout layout = Layout::BHTD, void* stream = nullptr);

// One query token per sequence against a [B, Hkv, Lcache, D] KV cache; q, o: [B, Hq, D].
void flash_attn_decode(const Tensor& q, const Tensor& kcache, const Tensor& vcache, Tensor& o, int B, int Lcache,
                       int Hq, int Hkv, int D, void* stream = nullptr);

// Fused RoPE + QK-Norm in front of attention and its backward: one call instead of split_heads ->
// rope_apply_inplace -> rmsnorm_forward (llm/src/model/modern_gpt.cu:351-370) and of rmsnorm_backward ->
// rope_apply_backward_inplace -> merge_heads (llm/src/model/modern_gpt.cu:527-552).  x: FP32 or BF16 rows of d_h
// elements in x_layout (BTHD = the projection output [B, T, H*d_h] where it lies); y / d_y: BF16 in y_layout;
// cos, sin: the tables of make_rope_cache; rstd [B*H, T] FP32; d_gamma is accumulated into (rmsnorm.h:17).
void rope_qknorm_forward(const Tensor& x, const Tensor& cos, const Tensor& sin, const Tensor& gamma, float eps, Tensor& y,
                         Tensor& rstd, int B, int T, int H, int d_h, Layout x_layout = Layout::BTHD,
                         Layout y_layout = Layout::BHTD, void* stream = nullptr);

void rope_qknorm_backward(const Tensor& d_y, const Tensor& x, const Tensor& cos, const Tensor& sin, const Tensor& gamma,
                          const Tensor& rstd, Tensor& d_x, Tensor& d_gamma, int B, int T, int H, int d_h,
                          Layout x_layout = Layout::BTHD, Layout y_layout = Layout::BHTD, void* stream = nullptr);

// KV cache for the sampler (the reference re-runs the whole forward per token, llm/apps/infer_modern_gpt.cu:13,253-255).
// kv_cache_append: what a block does to the n_new newest tokens before attention (llm/src/model/modern_gpt.cu:351-370:
// split_heads, RoPE at positions pos0 .. pos0 + n_new - 1, QK-Norm) in one call: q_proj [B, n_new, Hq*d_h],
// k_proj / v_proj [B, n_new, Hkv*d_h] (FP32 or BF16) -> q_out [B*Hq, n_new, d_h] BF16 and rows pos0 .. of the caches
// [B*Hkv, L_cap, d_h] BF16.  cos, sin: make_rope_cache(L_cap, d_h, ...).
void kv_cache_append(const Tensor& q_proj, const Tensor& k_proj, const Tensor& v_proj, const Tensor& cos, const Tensor& sin,
                     const Tensor& gamma_q, const Tensor& gamma_k, float eps, Tensor& q_out, Tensor& kcache, Tensor& vcache,
                     int B, int n_new, int pos0, int L_cap, int Hq, int Hkv, int d_h, void* stream = nullptr);
// One query token per sequence against the first L rows of caches of capacity L_cap; q, o: [B, Hq, d_h].
void flash_attn_decode_cached(const Tensor& q, const Tensor& kcache, const Tensor& vcache, Tensor& o, int B, int L, int L_cap,
                              int Hq, int Hkv, int D, void* stream = nullptr);
// Causal attention over a prompt of T tokens with K and V read from the caches (rows 0 .. T-1); q, ctx: [B*Hq, T, D].
void flash_attn_forward_kvcache(const Tensor& q, const Tensor& kcache, const Tensor& vcache, Tensor& ctx, Tensor& L, int B,
                                int T, int L_cap, int Hq, int Hkv, int D, void* stream = nullptr);

}  // namespace b200
}  // namespace modernllm
