// KV-cache append for single-token (and chunked-prefill) inference.
//
// The reference's sampler has no KV cache: infer_modern_gpt re-runs the whole T-token forward for every generated
// token (llm/apps/infer_modern_gpt.cu:13,253-255) and lists the cache as future work (TODO.md, "KV cache for
// inference").  A cached step needs, per layer, what ModernGPT's block does to the new tokens' q, k and v before
// attention (llm/src/model/modern_gpt.cu:351-370): split_heads, rope_apply_inplace at the tokens' TRUE positions
// (llm/src/model/rope.cu:25-44) and rmsnorm_forward over rows of length d_h on q and k (llm/src/model/rmsnorm.cu:24-53);
// v is only re-laid.  Then k and v must land in the cache rows of those positions.
//
// One kernel does all of it for the n_new newest tokens of B sequences that advance in lock step:
//   q rows  [B, n_new, Hq,  D] -> RoPE(pos0 + t) -> RMSNorm * gamma_q -> BF16 q_out [B, Hq, n_new, D]
//   k rows  [B, n_new, Hkv, D] -> RoPE(pos0 + t) -> RMSNorm * gamma_k -> BF16 kcache[b, h, pos0 + t, :]
//   v rows  [B, n_new, Hkv, D] -> BF16 vcache[b, h, pos0 + t, :]
// with the caches laid out [B, Hkv, L_cap, D], the layout the decode kernel streams.  The row arithmetic is the
// training kernel's (rn_rotate8 / rn_rstd / rn_scale8), so a cache filled here holds the same bits as the
// training path's k.  The work is a handful of rows per step (n_new = 1) or one read and one write of the tensors
// (prefill): bound by launch latency or by HBM bytes; a lane owns 8 consecutive elements of a row, as in
// rope_norm.cuh.
#pragma once

#include "rope_norm.cuh"

namespace b200attn {

struct KvAppendParams {
    const void* xq;      // [B, n_new, Hq, D]   projection output, FP32 or BF16
    const void* xk;      // [B, n_new, Hkv, D]
    const void* xv;      // [B, n_new, Hkv, D]
    uint16_t* q_out;     // [B, Hq, n_new, D] BF16
    uint16_t* kcache;    // [B, Hkv, L_cap, D] BF16
    uint16_t* vcache;
    const float* gamma_q;  // [D]
    const float* gamma_k;  // [D]
    const float* cos_t;    // [>= pos0 + n_new, D/2]
    const float* sin_t;
    const int* pos;        // [B] first position per sequence, or nullptr: pos0 for every sequence
    int* status;           // set to DEV_KV_CACHE_OVERFLOW when a row would land beyond the capacity (the row is skipped)
    int B, n_new, pos0, L_cap, Hq, Hkv;
    unsigned rows_q, rows_kv;  // B * n_new * Hq, B * n_new * Hkv
    FastDiv div_hq, div_hkv, div_n;
    float eps;
};

constexpr int kKvAppendThreads = 256;

// Rows are walked in the order they lie in the inputs (q rows, then k rows, then v rows), so loads are dense; a
// stored row is D * 2 bytes = one or two full 128-byte lines.
template <int D, bool F32>
__global__ void __launch_bounds__(kKvAppendThreads)
kv_append_kernel(const __grid_constant__ KvAppendParams p) {
    constexpr int LPR = D / 8;     // lanes per row
    constexpr int RPS = 32 / LPR;  // rows per warp and step
    const int lane = threadIdx.x & 31;
    const int sub = lane / LPR, li = lane % LPR;
    const unsigned warp0 = (blockIdx.x * kKvAppendThreads + threadIdx.x) >> 5;
    const unsigned n_warps = (gridDim.x * kKvAppendThreads) >> 5;
    const unsigned n_rows = p.rows_q + 2u * p.rows_kv;
    grid_dep_wait();  // launched with programmatic stream serialization: the inputs come from the kernel before

    for (unsigned long long r0 = static_cast<unsigned long long>(warp0) * RPS; r0 < n_rows;
         r0 += static_cast<unsigned long long>(n_warps) * RPS) {
        const unsigned long long rr = r0 + sub;
        const bool live = rr < n_rows;
        // which tensor, and the row inside it
        unsigned r = unsigned(rr);
        int which = 0;  // 0 q, 1 k, 2 v
        if (live && r >= p.rows_q) {
            r -= p.rows_q;
            which = 1;
            if (r >= p.rows_kv) {
                r -= p.rows_kv;
                which = 2;
            }
        }
        float v[8], rot[8], gm[8];
        float ss = 0.f;
        int b = 0, t = 0, h = 0, pos0 = 0;
        bool fits = true;
        if (live) {
            const int H = which == 0 ? p.Hq : p.Hkv;
            const unsigned bt = fastdiv(r, which == 0 ? p.div_hq : p.div_hkv);
            h = int(r - bt * unsigned(H));
            b = int(fastdiv(bt, p.div_n));
            t = int(bt - unsigned(b) * unsigned(p.n_new));
            pos0 = p.pos ? __ldg(p.pos + b) : p.pos0;
            fits = pos0 >= 0 && pos0 + p.n_new <= p.L_cap;  // the host checked pos0; an array of positions is checked here
            if (!fits) pos0 = 0;
            const void* x = which == 0 ? p.xq : (which == 1 ? p.xk : p.xv);
            rn_load8<F32>(x, static_cast<long long>(r) * D + li * 8, v);
            if (which != 2) {
                // every load of the row is issued before the first use (one round trip to memory, not two)
                const float* gamma = which == 0 ? p.gamma_q : p.gamma_k;
                const float4 g0 = *reinterpret_cast<const float4*>(gamma + li * 8);
                const float4 g1 = *reinterpret_cast<const float4*>(gamma + li * 8 + 4);
                gm[0] = g0.x, gm[1] = g0.y, gm[2] = g0.z, gm[3] = g0.w, gm[4] = g1.x, gm[5] = g1.y, gm[6] = g1.z, gm[7] = g1.w;
                const long long pos = pos0 + t;
                const float4 cs = *reinterpret_cast<const float4*>(p.cos_t + pos * (D / 2) + li * 4);
                const float4 sn = *reinterpret_cast<const float4*>(p.sin_t + pos * (D / 2) + li * 4);
                ss = rn_rotate8(v, cs, sn, rot);
            }
        }
        ss = rn_row_sum<LPR>(ss);  // every lane takes part in the shuffles
        if (!live) continue;
        if (!fits) {
            if (li == 0) atomicCAS(p.status, 0, int(DEV_KV_CACHE_OVERFLOW));  // the first error recorded stays
            continue;
        }
        if (which == 2) {
            rn_store8<false>(p.vcache, ((static_cast<long long>(b) * p.Hkv + h) * p.L_cap + pos0 + t) * D + li * 8, v);
            continue;
        }
        float out[8];
        rn_scale8(rot, rn_rstd<D>(ss, p.eps), gm, out);
        if (which == 0)
            rn_store8<false>(p.q_out, ((static_cast<long long>(b) * p.Hq + h) * p.n_new + t) * D + li * 8, out);
        else
            rn_store8<false>(p.kcache, ((static_cast<long long>(b) * p.Hkv + h) * p.L_cap + pos0 + t) * D + li * 8, out);
    }
}

}  // namespace b200attn
