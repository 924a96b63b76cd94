// Fused RoPE + per-head RMSNorm (QK-Norm) on the way into the attention kernels, and its backward.
//
// The reference prepares q and k for attention with five passes over each tensor
// (llm/src/model/modern_gpt.cu:351-370): split_heads ([B,T,H*d] -> [B*H,T,d], llm/src/model/attention.cu:344-364),
// rope_apply_inplace (llm/src/model/rope.cu:25-44,146-163) and rmsnorm_forward over rows of length d
// (llm/src/model/rmsnorm.cu:24-53), FP32 throughout; the backward mirrors it (modern_gpt.cu:527-552:
// rmsnorm_backward, llm/src/model/rmsnorm.cu:55-101, rope_apply_backward_inplace, llm/src/model/rope.cu:46-65,
// merge_heads).  Here one kernel reads a row of the projection output where it lies (either layout, FP32 or
// BF16), rotates it, normalises it, scales it by gamma and writes it as BF16 in the layout the attention
// kernels take; the backward does the inverse chain in one pass and reduces d_gamma without atomics.
//
//   r[2i]   = x[2i] cos(t, i) - x[2i+1] sin(t, i)          r[2i+1] = x[2i] sin(t, i) + x[2i+1] cos(t, i)
//   rstd    = rsqrt(mean_d r[d]^2 + eps)                    y[d]    = r[d] rstd gamma[d]
//   g[d]    = dy[d] gamma[d]       s = sum_d g[d] r[d]      dr[d]   = rstd g[d] - rstd^3 / D s r[d]
//   dx[2i]  = dr[2i] cos + dr[2i+1] sin                     dx[2i+1] = -dr[2i] sin + dr[2i+1] cos
//   d_gamma[d] += sum over rows of dy[d] r[d] rstd
//
// The work is bound by HBM bandwidth (one read and one write of the tensor), so the kernels are built for
// coalescing and for bytes in flight: a warp owns a row (D = 64: one rotation pair per lane, one 4- or 8-byte
// access; D = 128: two pairs per lane), takes kRowsPerIter rows per loop iteration with all their loads issued
// before the first use, and the grid is a multiple of the SM count.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace b200attn {

struct RopeNormParams {
    const void* x;       // input rows (forward) / the forward's input again (backward)
    void* y;             // forward: BF16 output;  backward: d_x output (same type and layout as x)
    const uint16_t* dy;  // backward: BF16 gradient of y, in y's layout
    float* rstd;         // [B, H, T]: written by the forward, read by the backward
    const float* gamma;  // [D]
    const float* cos_t;  // [T, D/2]
    const float* sin_t;  // [T, D/2]
    float* partial;      // backward: [gridDim.x, D] partial d_gamma sums
    int B, T, H;
    int x_bthd;          // x is [B, T, H, D] (else [B, H, T, D]): the order in which rows are walked
    long long x_st, x_sh, x_sb;  // element strides of x (and of d_x): token, head, batch
    long long y_st, y_sh, y_sb;  // element strides of y (and of dy)
    float eps;
};

constexpr int kRopeNormThreads = 256;  // 8 warps
constexpr int kRowsPerIter = 4;

__device__ __forceinline__ float rn_bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float rn_bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ uint32_t rn_pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ float rn_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Row r of the walk -> (batch, token, head)
__device__ __forceinline__ void rn_decode_row(const RopeNormParams& p, long long r, int& b, int& t, int& h) {
    if (p.x_bthd) {
        h = int(r % p.H);
        t = int((r / p.H) % p.T);
        b = int(r / (static_cast<long long>(p.H) * p.T));
    } else {
        t = int(r % p.T);
        h = int((r / p.T) % p.H);
        b = int(r / (static_cast<long long>(p.H) * p.T));
    }
}

// PPL = rotation pairs per lane (D / 64); the lane owns elements [lane * 2 PPL, lane * 2 PPL + 2 PPL)
template <int PPL, bool F32>
__device__ __forceinline__ void rn_load_row(const void* base, long long off, int lane, float (&v)[2 * PPL]) {
    if (F32) {
        const float* ptr = static_cast<const float*>(base) + off + lane * 2 * PPL;
        if (PPL == 1) {
            const float2 a = *reinterpret_cast<const float2*>(ptr);
            v[0] = a.x, v[1] = a.y;
        } else {
            const float4 a = *reinterpret_cast<const float4*>(ptr);
            v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w;
        }
    } else {
        const uint16_t* ptr = static_cast<const uint16_t*>(base) + off + lane * 2 * PPL;
        if (PPL == 1) {
            const uint32_t a = *reinterpret_cast<const uint32_t*>(ptr);
            v[0] = rn_bf16_lo(a), v[1] = rn_bf16_hi(a);
        } else {
            const uint2 a = *reinterpret_cast<const uint2*>(ptr);
            v[0] = rn_bf16_lo(a.x), v[1] = rn_bf16_hi(a.x), v[2] = rn_bf16_lo(a.y), v[3] = rn_bf16_hi(a.y);
        }
    }
}
template <int PPL, bool F32>
__device__ __forceinline__ void rn_store_row(void* base, long long off, int lane, const float (&v)[2 * PPL]) {
    if (F32) {
        float* ptr = static_cast<float*>(base) + off + lane * 2 * PPL;
        if (PPL == 1) *reinterpret_cast<float2*>(ptr) = make_float2(v[0], v[1]);
        else *reinterpret_cast<float4*>(ptr) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
        uint16_t* ptr = static_cast<uint16_t*>(base) + off + lane * 2 * PPL;
        if (PPL == 1) *reinterpret_cast<uint32_t*>(ptr) = rn_pack_bf16x2(v[0], v[1]);
        else *reinterpret_cast<uint2*>(ptr) = make_uint2(rn_pack_bf16x2(v[0], v[1]), rn_pack_bf16x2(v[2], v[3]));
    }
}

template <int D, bool F32>
__global__ void __launch_bounds__(kRopeNormThreads) rope_norm_fwd_kernel(const RopeNormParams p) {
    constexpr int PPL = D / 64;
    const int lane = threadIdx.x & 31;
    const long long n_rows = static_cast<long long>(p.B) * p.T * p.H;
    const long long warp0 = (static_cast<long long>(blockIdx.x) * kRopeNormThreads + threadIdx.x) >> 5;
    const long long n_warps = (static_cast<long long>(gridDim.x) * kRopeNormThreads) >> 5;
    float gm[2 * PPL];
#pragma unroll
    for (int e = 0; e < 2 * PPL; ++e) gm[e] = p.gamma[lane * 2 * PPL + e];

    for (long long r0 = warp0 * kRowsPerIter; r0 < n_rows; r0 += n_warps * kRowsPerIter) {
        float v[kRowsPerIter][2 * PPL], cs[kRowsPerIter][PPL], sn[kRowsPerIter][PPL];
        int bb[kRowsPerIter], tt[kRowsPerIter], hh[kRowsPerIter];
        // all loads of the iteration first
#pragma unroll
        for (int k = 0; k < kRowsPerIter; ++k) {
            const long long r = r0 + k;
            if (r < n_rows) {
                rn_decode_row(p, r, bb[k], tt[k], hh[k]);
                rn_load_row<PPL, F32>(p.x, bb[k] * p.x_sb + tt[k] * p.x_st + hh[k] * p.x_sh, lane, v[k]);
#pragma unroll
                for (int i = 0; i < PPL; ++i) {
                    cs[k][i] = p.cos_t[static_cast<long long>(tt[k]) * (D / 2) + lane * PPL + i];
                    sn[k][i] = p.sin_t[static_cast<long long>(tt[k]) * (D / 2) + lane * PPL + i];
                }
            }
        }
#pragma unroll
        for (int k = 0; k < kRowsPerIter; ++k) {
            const long long r = r0 + k;
            if (r >= n_rows) break;  // warp-uniform
            float rot[2 * PPL];
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < PPL; ++i) {
                const float x0 = v[k][2 * i], x1 = v[k][2 * i + 1];
                rot[2 * i] = x0 * cs[k][i] - x1 * sn[k][i];
                rot[2 * i + 1] = x0 * sn[k][i] + x1 * cs[k][i];
                ss += rot[2 * i] * rot[2 * i] + rot[2 * i + 1] * rot[2 * i + 1];
            }
            ss = rn_warp_sum(ss);
            const float rstd = rsqrtf(ss / float(D) + p.eps);
            float out[2 * PPL];
#pragma unroll
            for (int e = 0; e < 2 * PPL; ++e) out[e] = rot[e] * rstd * gm[e];
            rn_store_row<PPL, false>(p.y, bb[k] * p.y_sb + tt[k] * p.y_st + hh[k] * p.y_sh, lane, out);
            if (lane == 0) p.rstd[(static_cast<long long>(bb[k]) * p.H + hh[k]) * p.T + tt[k]] = rstd;
        }
    }
}

template <int D, bool F32>
__global__ void __launch_bounds__(kRopeNormThreads) rope_norm_bwd_kernel(const RopeNormParams p) {
    constexpr int PPL = D / 64;
    __shared__ float s_part[kRopeNormThreads / 32][D];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long n_rows = static_cast<long long>(p.B) * p.T * p.H;
    const long long warp0 = (static_cast<long long>(blockIdx.x) * kRopeNormThreads + threadIdx.x) >> 5;
    const long long n_warps = (static_cast<long long>(gridDim.x) * kRopeNormThreads) >> 5;
    float gm[2 * PPL], dg[2 * PPL];
#pragma unroll
    for (int e = 0; e < 2 * PPL; ++e) {
        gm[e] = p.gamma[lane * 2 * PPL + e];
        dg[e] = 0.f;
    }
    for (long long r0 = warp0 * kRowsPerIter; r0 < n_rows; r0 += n_warps * kRowsPerIter) {
        float v[kRowsPerIter][2 * PPL], dyv[kRowsPerIter][2 * PPL], cs[kRowsPerIter][PPL], sn[kRowsPerIter][PPL];
        float rs[kRowsPerIter];
        int bb[kRowsPerIter], tt[kRowsPerIter], hh[kRowsPerIter];
#pragma unroll
        for (int k = 0; k < kRowsPerIter; ++k) {
            const long long r = r0 + k;
            if (r < n_rows) {
                rn_decode_row(p, r, bb[k], tt[k], hh[k]);
                rn_load_row<PPL, F32>(p.x, bb[k] * p.x_sb + tt[k] * p.x_st + hh[k] * p.x_sh, lane, v[k]);
                rn_load_row<PPL, false>(p.dy, bb[k] * p.y_sb + tt[k] * p.y_st + hh[k] * p.y_sh, lane, dyv[k]);
                rs[k] = p.rstd[(static_cast<long long>(bb[k]) * p.H + hh[k]) * p.T + tt[k]];
#pragma unroll
                for (int i = 0; i < PPL; ++i) {
                    cs[k][i] = p.cos_t[static_cast<long long>(tt[k]) * (D / 2) + lane * PPL + i];
                    sn[k][i] = p.sin_t[static_cast<long long>(tt[k]) * (D / 2) + lane * PPL + i];
                }
            }
        }
#pragma unroll
        for (int k = 0; k < kRowsPerIter; ++k) {
            const long long r = r0 + k;
            if (r >= n_rows) break;  // warp-uniform
            float rot[2 * PPL], g[2 * PPL];
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < PPL; ++i) {
                const float x0 = v[k][2 * i], x1 = v[k][2 * i + 1];
                rot[2 * i] = x0 * cs[k][i] - x1 * sn[k][i];
                rot[2 * i + 1] = x0 * sn[k][i] + x1 * cs[k][i];
            }
#pragma unroll
            for (int e = 0; e < 2 * PPL; ++e) {
                g[e] = dyv[k][e] * gm[e];
                s += g[e] * rot[e];
                dg[e] += dyv[k][e] * rot[e] * rs[k];
            }
            s = rn_warp_sum(s);
            const float coeff = rs[k] * rs[k] * rs[k] * (1.f / float(D)) * s;
            float dx[2 * PPL];
#pragma unroll
            for (int i = 0; i < PPL; ++i) {
                const float d0 = rs[k] * g[2 * i] - coeff * rot[2 * i];
                const float d1 = rs[k] * g[2 * i + 1] - coeff * rot[2 * i + 1];
                dx[2 * i] = d0 * cs[k][i] + d1 * sn[k][i];
                dx[2 * i + 1] = -d0 * sn[k][i] + d1 * cs[k][i];
            }
            rn_store_row<PPL, F32>(p.y, bb[k] * p.x_sb + tt[k] * p.x_st + hh[k] * p.x_sh, lane, dx);
        }
    }
    // d_gamma: lanes hold per-column sums of their warp's rows; add the warps of the CTA in a fixed order
#pragma unroll
    for (int e = 0; e < 2 * PPL; ++e) s_part[warp][lane * 2 * PPL + e] = dg[e];
    __syncthreads();
    for (int d = threadIdx.x; d < D; d += kRopeNormThreads) {
        float acc = 0.f;
#pragma unroll
        for (int w = 0; w < kRopeNormThreads / 32; ++w) acc += s_part[w][d];
        p.partial[static_cast<long long>(blockIdx.x) * D + d] = acc;
    }
}

// d_gamma[d] += sum over the CTAs' partial sums, in CTA order (one thread per column: bit-reproducible)
template <int D>
__global__ void rope_norm_dgamma_kernel(const float* __restrict__ partial, int n_parts, float* __restrict__ d_gamma) {
    const int d = blockIdx.x * blockDim.x + threadIdx.x;
    if (d >= D) return;
    float acc = 0.f;
    for (int i = 0; i < n_parts; ++i) acc += partial[static_cast<long long>(i) * D + d];
    d_gamma[d] += acc;
}

}  // namespace b200attn
