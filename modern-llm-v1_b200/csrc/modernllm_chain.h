// The attention chain of a ModernGPT block on the b200attn engine, for a build of the reference tree.
//
// Replaces, in ModernGPT::recompute_block_forward (llm/src/model/modern_gpt.cu:351-378),
//     split_heads x3 -> rope_apply_inplace x2 -> rmsnorm_forward x2 (QK-Norm) -> repeat_kv_heads x2
//     -> scaled_dot_attention_forward -> merge_heads
// by   rope_qknorm_forward (q) + rope_qknorm_forward (k) + a cast of v -> flash_attn_forward_gqa -> a cast of ctx
// and, in ModernGPT::backward (llm/src/model/modern_gpt.cu:505-552),
//     cudaMalloc'ed d_ctx_split + split_heads -> scaled_dot_attention_backward (two more cudaMallocs,
//     llm/src/model/attention.cu:197,225) -> zero x2 + accumulate_kv_grads x2 -> rmsnorm_backward x2
//     -> rope_apply_backward_inplace x2 -> merge_heads x3
// by   a cast of d_ctx -> flash_attn_backward_gqa -> rope_qknorm_backward (q) + (k) + a cast of d_v.
// Everything stays in the projection layout [B, T, H * d_h]: the engine reads and writes it in place
// (Layout::BTHD), so no head split or merge is left.  The buffers that disappear from the model are
// q_split, k_split, v_split, q_normed, k_normed, k_full, v_full, ctx_split, probs ([B*H, T, T]) and
// d_q_split_, d_k_full_, d_v_full_, d_k_split_, d_v_split_ (llm/src/model/modern_gpt.cu:74-78,94-105).
//
// Two variants, chosen by the projections' element type:
//   * FP32 projections (the stock linear layers): the engine's BF16 operands are made by the fused RoPE + QK-Norm
//     (which reads FP32) and by cast_fp32_to_bf16 / cast_bf16_to_fp32 (llm/src/core/cast.h:13-14) for v, ctx, d_ctx, d_v;
//   * BF16 projections (linear_forward_bf16inout / linear_backward_bf16inout, llm/src/model/linear.h:71-83): no cast at
//     all, the chain consumes and produces the projections' own buffers.
// Header-only; needs modernllm_shim.{h,cc} and libb200attn.so.
#pragma once

#include <mutex>
#include <unordered_map>

#include "core/cast.h"
#include "core/tensor.h"
#include "modernllm_shim.h"

namespace modernllm {
namespace b200 {

// BF16 operands of the engine that the model keeps between forward and backward of a block (shared by all blocks,
// like the reference's act_* buffers under gradient checkpointing), one set per model object.
struct ChainBuffers {
    Tensor q, k, v, ctx, L;         // [B, T, H, d_h] / [B, T, Hkv, d_h] BF16; L [B * H, T] FP32
    Tensor d_ctx, d_q, d_k, d_v;    // BF16, same shapes
    bool ready = false;
};

inline ChainBuffers& chain_buffers(const void* model, int B, int T, int H, int Hkv, int d_h) {
    static std::mutex mu;
    static std::unordered_map<const void*, ChainBuffers> all;
    std::lock_guard<std::mutex> lock(mu);
    ChainBuffers& c = all[model];
    if (!c.ready) {
        auto bf = [](std::int64_t rows, std::int64_t cols) { return Tensor({rows, cols}, DType::BF16, Device::Cuda); };
        const std::int64_t N = 1LL * B * T;
        c.q = bf(N, 1LL * H * d_h), c.k = bf(N, 1LL * Hkv * d_h), c.v = bf(N, 1LL * Hkv * d_h), c.ctx = bf(N, 1LL * H * d_h);
        c.d_ctx = bf(N, 1LL * H * d_h), c.d_q = bf(N, 1LL * H * d_h), c.d_k = bf(N, 1LL * Hkv * d_h), c.d_v = bf(N, 1LL * Hkv * d_h);
        c.L = Tensor({1LL * B * H, T}, DType::FP32, Device::Cuda);
        c.ready = true;
    }
    return c;
}

// BF16 activations around attention for the variant with BF16-in/BF16-out projections: the block's normalised input,
// the three projections, ctx and the output projection's result, and the matching gradients (shared by all blocks).
struct ChainIo {
    Tensor x, q_proj, k_proj, v_proj, ctx, attn_out;
    Tensor d_attn_out, d_ctx, d_q_proj, d_k_proj, d_v_proj, d_x;
    bool ready = false;
};

inline ChainIo& chain_io(const void* model, std::int64_t N, std::int64_t D, std::int64_t Dkv) {
    static std::mutex mu;
    static std::unordered_map<const void*, ChainIo> all;
    std::lock_guard<std::mutex> lock(mu);
    ChainIo& io = all[model];
    if (!io.ready) {
        auto bf = [](std::int64_t rows, std::int64_t cols) { return Tensor({rows, cols}, DType::BF16, Device::Cuda); };
        io.x = bf(N, D), io.q_proj = bf(N, D), io.k_proj = bf(N, Dkv), io.v_proj = bf(N, Dkv), io.ctx = bf(N, D), io.attn_out = bf(N, D);
        io.d_attn_out = bf(N, D), io.d_ctx = bf(N, D), io.d_q_proj = bf(N, D), io.d_k_proj = bf(N, Dkv), io.d_v_proj = bf(N, Dkv);
        io.d_x = bf(N, D);
        io.ready = true;
    }
    return io;
}

// q_proj [B*T, H*d_h], k_proj / v_proj [B*T, Hkv*d_h]: FP32 or BF16 (all three alike).  ctx [B, T, H*d_h] in the
// projections' type.  q_rstd [B*H*T], k_rstd [B*Hkv*T] FP32 are kept for the backward.
inline void chain_attention_forward(const void* model, const Tensor& q_proj, const Tensor& k_proj, const Tensor& v_proj,
                                    const Tensor& rope_cos, const Tensor& rope_sin, const Tensor& q_norm_g,
                                    const Tensor& k_norm_g, float eps, Tensor& q_rstd, Tensor& k_rstd, Tensor& ctx, int B, int T,
                                    int H, int Hkv, int d_h, void* stream = nullptr) {
    ChainBuffers& c = chain_buffers(model, B, T, H, Hkv, d_h);
    rope_qknorm_forward(q_proj, rope_cos, rope_sin, q_norm_g, eps, c.q, q_rstd, B, T, H, d_h, Layout::BTHD, Layout::BTHD, stream);
    rope_qknorm_forward(k_proj, rope_cos, rope_sin, k_norm_g, eps, c.k, k_rstd, B, T, Hkv, d_h, Layout::BTHD, Layout::BTHD, stream);
    const bool bf16_io = v_proj.dtype() == DType::BF16;
    if (!bf16_io) cast_fp32_to_bf16(v_proj, c.v);
    flash_attn_forward_gqa(c.q, c.k, bf16_io ? v_proj : c.v, bf16_io ? ctx : c.ctx, c.L, B, T, H, Hkv, d_h, Layout::BTHD, stream);
    if (!bf16_io) cast_bf16_to_fp32(c.ctx, ctx);
}

// d_ctx [B, T, H*d_h] (gradient of ctx) and ctx itself in the projections' type; writes d_q_proj, d_k_proj, d_v_proj
// (projection layout, projections' type) and ACCUMULATES into d_q_norm_g, d_k_norm_g like rmsnorm_backward
// (llm/src/model/rmsnorm.h:17).  v_proj and ctx are only read in the BF16 variant (the FP32 variant kept its own
// BF16 copies in the forward).
inline void chain_attention_backward(const void* model, const Tensor& d_ctx, const Tensor& q_proj, const Tensor& k_proj,
                                     const Tensor& v_proj, const Tensor& ctx, const Tensor& rope_cos, const Tensor& rope_sin,
                                     const Tensor& q_norm_g, const Tensor& k_norm_g, const Tensor& q_rstd, const Tensor& k_rstd,
                                     Tensor& d_q_proj, Tensor& d_k_proj, Tensor& d_v_proj, Tensor& d_q_norm_g, Tensor& d_k_norm_g,
                                     int B, int T, int H, int Hkv, int d_h, void* stream = nullptr) {
    ChainBuffers& c = chain_buffers(model, B, T, H, Hkv, d_h);
    const bool bf16_io = d_ctx.dtype() == DType::BF16;
    if (!bf16_io) cast_fp32_to_bf16(d_ctx, c.d_ctx);
    flash_attn_backward_gqa(c.q, c.k, bf16_io ? v_proj : c.v, bf16_io ? ctx : c.ctx, c.L, bf16_io ? d_ctx : c.d_ctx, c.d_q, c.d_k,
                            bf16_io ? d_v_proj : c.d_v, B, T, H, Hkv, d_h, Layout::BTHD, stream);
    rope_qknorm_backward(c.d_q, q_proj, rope_cos, rope_sin, q_norm_g, q_rstd, d_q_proj, d_q_norm_g, B, T, H, d_h, Layout::BTHD,
                         Layout::BTHD, stream);
    rope_qknorm_backward(c.d_k, k_proj, rope_cos, rope_sin, k_norm_g, k_rstd, d_k_proj, d_k_norm_g, B, T, Hkv, d_h, Layout::BTHD,
                         Layout::BTHD, stream);
    if (!bf16_io) cast_bf16_to_fp32(c.d_v, d_v_proj);
}

}  // namespace b200
}  // namespace modernllm
