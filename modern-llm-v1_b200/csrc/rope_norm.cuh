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
// coalescing and for bytes in flight: a lane owns 8 consecutive elements of a row (one 16-byte access for BF16,
// two for FP32), so a row takes D / 8 lanes and a warp covers 32 / (D / 8) rows per access; kStepsPerIter
// such accesses are issued before the first use, and the grid is a multiple of the SM count.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"

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
    float* d_gamma;      // backward: [D], accumulated into by rope_norm_dgamma_kernel
    int B, T, H;
    FastDiv div_h, div_t;  // division by H and by T as multiply + shift
    int walk_bthd;       // rows are walked in [B, T, H] order (else [B, H, T]): the order of the tensor that is WRITTEN
                         // (y in the forward, d_x in the backward), so that all stores are dense
    long long x_st, x_sh, x_sb;  // element strides of x (and of d_x): token, head, batch
    long long y_st, y_sh, y_sb;  // element strides of y (and of dy)
    float eps;
};

constexpr int kRopeNormThreads = 256;  // 8 warps
#ifndef RN_FWD_STEPS
#define RN_FWD_STEPS 1
#define RN_FWD_BLOCKS 4
#define RN_BWD_STEPS 1
#define RN_BWD_BLOCKS 3
#endif
constexpr int kFwdSteps = RN_FWD_STEPS;  // row groups per loop iteration (all their loads are issued first)
constexpr int kBwdSteps = RN_BWD_STEPS;

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
// sum over the LPR lanes that share a row (LPR a power of two, lanes of a row are adjacent)
template <int LPR>
__device__ __forceinline__ float rn_row_sum(float v) {
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Row r of the walk -> (batch, token, head)
__device__ __forceinline__ void rn_decode_row(const RopeNormParams& p, unsigned r, int& b, int& t, int& h) {
    if (p.walk_bthd) {
        const unsigned bt = fastdiv(r, p.div_h);
        h = int(r - bt * unsigned(p.H));
        b = int(fastdiv(bt, p.div_t));
        t = int(bt - unsigned(b) * unsigned(p.T));
    } else {
        const unsigned bh = fastdiv(r, p.div_t);
        t = int(r - bh * unsigned(p.T));
        b = int(fastdiv(bh, p.div_h));
        h = int(bh - unsigned(b) * unsigned(p.H));
    }
}

// 8 consecutive elements starting at element offset `off`
template <bool F32>
__device__ __forceinline__ void rn_load8(const void* base, long long off, float (&v)[8]) {
    if (F32) {
        const float4* ptr = reinterpret_cast<const float4*>(static_cast<const float*>(base) + off);
        const float4 a = ptr[0], c = ptr[1];
        v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = c.x, v[5] = c.y, v[6] = c.z, v[7] = c.w;
    } else {
        const uint4 a = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(base) + off);
        v[0] = rn_bf16_lo(a.x), v[1] = rn_bf16_hi(a.x), v[2] = rn_bf16_lo(a.y), v[3] = rn_bf16_hi(a.y);
        v[4] = rn_bf16_lo(a.z), v[5] = rn_bf16_hi(a.z), v[6] = rn_bf16_lo(a.w), v[7] = rn_bf16_hi(a.w);
    }
}
template <bool F32>
__device__ __forceinline__ void rn_store8(void* base, long long off, const float (&v)[8]) {
    if (F32) {
        float4* ptr = reinterpret_cast<float4*>(static_cast<float*>(base) + off);
        ptr[0] = make_float4(v[0], v[1], v[2], v[3]);
        ptr[1] = make_float4(v[4], v[5], v[6], v[7]);
    } else {
        *reinterpret_cast<uint4*>(static_cast<uint16_t*>(base) + off) =
            make_uint4(rn_pack_bf16x2(v[0], v[1]), rn_pack_bf16x2(v[2], v[3]), rn_pack_bf16x2(v[4], v[5]),
                       rn_pack_bf16x2(v[6], v[7]));
    }
}

// The forward arithmetic of one row, shared by every kernel that prepares q or k (so that a row gives the same
// bits whichever kernel computes it).  rn_rotate8: RoPE on a lane's 8 elements (4 pairs; cs, sn = the 4 cosines
// and sines of the lane's pairs at the row's position) and the lane's share of the row's sum of squares.
__device__ __forceinline__ float rn_rotate8(const float (&v)[8], const float4& cs, const float4& sn, float (&rot)[8]) {
    const float c[4] = {cs.x, cs.y, cs.z, cs.w}, s[4] = {sn.x, sn.y, sn.z, sn.w};
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float x0 = v[2 * i], x1 = v[2 * i + 1];
        rot[2 * i] = x0 * c[i] - x1 * s[i];
        rot[2 * i + 1] = x0 * s[i] + x1 * c[i];
        ss += rot[2 * i] * rot[2 * i] + rot[2 * i + 1] * rot[2 * i + 1];
    }
    return ss;
}
template <int D>
__device__ __forceinline__ float rn_rstd(float row_sum_sq, float eps) {
    return rsqrtf(row_sum_sq / float(D) + eps);
}
__device__ __forceinline__ void rn_scale8(const float (&rot)[8], float rstd, const float (&gm)[8], float (&out)[8]) {
#pragma unroll
    for (int e = 0; e < 8; ++e) out[e] = rot[e] * rstd * gm[e];
}

// 16-byte asynchronous copy global -> shared (LDGSTS): the data does not pass through registers, so a lane can keep
// several iterations' worth of loads in flight at no register cost.
__device__ __forceinline__ void rn_cp_async16(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void rn_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void rn_cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// iterations in flight per lane in the forward (their loads are staged in shared memory: 48 KB per CTA either way)
template <bool F32>
constexpr int kFwdDepth = F32 ? 3 : 4;

// Shared memory of one forward stage: per thread 16 bytes each of cos and sin and 16 (BF16 x) or 32 (FP32 x) bytes
// of x, laid out [piece][thread] so that a warp's accesses are contiguous.
template <bool F32>
struct RnFwdStage {
    uint4 cs[kRopeNormThreads], sn[kRopeNormThreads], x0[kRopeNormThreads], x1[kRopeNormThreads];
};
template <>
struct RnFwdStage<false> {
    uint4 cs[kRopeNormThreads], sn[kRopeNormThreads], x0[kRopeNormThreads];
};

// One tensor's forward.  (A function of its own, called once per tensor with the kernel parameter itself, so that
// every field stays a constant-bank operand; selecting the struct at run time would move it to local memory.)
// A lane works on one row piece per iteration; the loads of the next few iterations (x, cos, sin) are
// already on their way into this lane's own slots of the stage ring, so no barrier is needed: a lane only ever
// reads what it has copied itself, after cp.async.wait_group.
template <int D, bool F32>
__device__ __forceinline__ void rope_norm_fwd_tensor(const RopeNormParams& p, RnFwdStage<F32>* ring) {
    constexpr int LPR = D / 8;      // lanes per row
    constexpr int RPS = 32 / LPR;   // rows per warp and iteration
    const int lane = threadIdx.x & 31;
    const int sub = lane / LPR, li = lane % LPR;  // row within the iteration, position within the row
    const unsigned warp0 = (blockIdx.x * kRopeNormThreads + threadIdx.x) >> 5;
    const unsigned n_warps = (gridDim.x * kRopeNormThreads) >> 5;
    const unsigned n_rows = unsigned(p.B) * unsigned(p.T) * unsigned(p.H);
    float gm[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) gm[e] = p.gamma[li * 8 + e];
    const unsigned long long stride = static_cast<unsigned long long>(n_warps) * RPS;
    const unsigned long long first = static_cast<unsigned long long>(warp0) * RPS + sub;

    // requests the loads of this lane's iteration `it` (row first + it * stride) into ring slot it % depth
    auto request = [&](unsigned it) {
        const unsigned long long r = first + it * stride;
        if (r < n_rows) {
            int b, t, h;
            rn_decode_row(p, unsigned(r), b, t, h);
            RnFwdStage<F32>& st = ring[it % kFwdDepth<F32>];
            const long long off = b * p.x_sb + t * p.x_st + h * p.x_sh + li * 8;
            if constexpr (F32) {
                rn_cp_async16(&st.x0[threadIdx.x], static_cast<const float*>(p.x) + off);
                rn_cp_async16(&st.x1[threadIdx.x], static_cast<const float*>(p.x) + off + 4);
            } else {
                rn_cp_async16(&st.x0[threadIdx.x], static_cast<const uint16_t*>(p.x) + off);
            }
            rn_cp_async16(&st.cs[threadIdx.x], p.cos_t + static_cast<long long>(t) * (D / 2) + li * 4);
            rn_cp_async16(&st.sn[threadIdx.x], p.sin_t + static_cast<long long>(t) * (D / 2) + li * 4);
        }
        rn_cp_async_commit();  // one group per iteration, also when it is empty
    };
#pragma unroll
    for (int i = 0; i < kFwdDepth<F32> - 1; ++i) request(i);
    for (unsigned it = 0; first + it * stride - sub < n_rows; ++it) {  // (all lanes of a warp run the same iterations)
        request(it + kFwdDepth<F32> - 1);
        rn_cp_async_wait<kFwdDepth<F32> - 1>();  // everything but the newest kFwdDepth - 1 groups has landed: iteration `it`
        const unsigned long long r = first + it * stride;
        const bool live = r < n_rows;
        float rot[8];
        float ss = 0.f;
        int b = 0, t = 0, h = 0;
        if (live) {
            const RnFwdStage<F32>& st = ring[it % kFwdDepth<F32>];
            float v[8];
            if constexpr (F32) {
                const uint4 a = st.x0[threadIdx.x], c = st.x1[threadIdx.x];
                v[0] = __uint_as_float(a.x), v[1] = __uint_as_float(a.y), v[2] = __uint_as_float(a.z), v[3] = __uint_as_float(a.w);
                v[4] = __uint_as_float(c.x), v[5] = __uint_as_float(c.y), v[6] = __uint_as_float(c.z), v[7] = __uint_as_float(c.w);
            } else {
                const uint4 a = st.x0[threadIdx.x];
                v[0] = rn_bf16_lo(a.x), v[1] = rn_bf16_hi(a.x), v[2] = rn_bf16_lo(a.y), v[3] = rn_bf16_hi(a.y);
                v[4] = rn_bf16_lo(a.z), v[5] = rn_bf16_hi(a.z), v[6] = rn_bf16_lo(a.w), v[7] = rn_bf16_hi(a.w);
            }
            const uint4 cw = st.cs[threadIdx.x], sw = st.sn[threadIdx.x];
            const float4 cs = make_float4(__uint_as_float(cw.x), __uint_as_float(cw.y), __uint_as_float(cw.z), __uint_as_float(cw.w));
            const float4 sn = make_float4(__uint_as_float(sw.x), __uint_as_float(sw.y), __uint_as_float(sw.z), __uint_as_float(sw.w));
            ss = rn_rotate8(v, cs, sn, rot);
            rn_decode_row(p, unsigned(r), b, t, h);
        }
        ss = rn_row_sum<LPR>(ss);  // every lane takes part in the shuffles
        if (live) {
            const float rstd = rn_rstd<D>(ss, p.eps);
            float out[8];
            rn_scale8(rot, rstd, gm, out);
            rn_store8<false>(p.y, static_cast<long long>(r) * D + li * 8, out);  // y is dense in walk order
            if (li == 0) p.rstd[(static_cast<long long>(b) * p.H + h) * p.T + t] = rstd;
        }
    }
    rn_cp_async_wait<0>();
}

// one launch takes q and k (n_tensors = 2), one after the other
template <int D, bool F32>
__global__ void __launch_bounds__(kRopeNormThreads, RN_FWD_BLOCKS)
rope_norm_fwd_kernel(const __grid_constant__ RopeNormParams p0, const __grid_constant__ RopeNormParams p1,
                     const int n_tensors) {
    __shared__ RnFwdStage<F32> ring[kFwdDepth<F32>];
    grid_dep_wait();  // launched with programmatic stream serialization: the inputs come from the kernel before
    rope_norm_fwd_tensor<D, F32>(p0, ring);
    if (n_tensors > 1) rope_norm_fwd_tensor<D, F32>(p1, ring);
}

// Shared memory of one backward stage, per thread: cos, sin, x (16 or 32 bytes), dy (16 bytes) and the row's rstd.
template <bool F32>
struct RnBwdStage {
    uint4 cs[kRopeNormThreads], sn[kRopeNormThreads], x0[kRopeNormThreads], x1[kRopeNormThreads], dy[kRopeNormThreads];
    float rstd[kRopeNormThreads];
};
template <>
struct RnBwdStage<false> {
    uint4 cs[kRopeNormThreads], sn[kRopeNormThreads], x0[kRopeNormThreads], dy[kRopeNormThreads];
    float rstd[kRopeNormThreads];
};
constexpr int kBwdDepth = 3;  // iterations in flight per lane in the backward
template <bool F32>
constexpr int kRopeNormBwdSmemBytes = kBwdDepth * int(sizeof(RnBwdStage<F32>));

__device__ __forceinline__ void rn_cp_async4(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}

// One tensor's backward; the loads are staged like the forward's (see rope_norm_fwd_tensor).
template <int D, bool F32>
__device__ __forceinline__ void rope_norm_bwd_tensor(const RopeNormParams& p, float (*s_part)[D], RnBwdStage<F32>* ring) {
    constexpr int LPR = D / 8;
    constexpr int RPS = 32 / LPR;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = lane / LPR, li = lane % LPR;
    const unsigned warp0 = (blockIdx.x * kRopeNormThreads + threadIdx.x) >> 5;
    const unsigned n_warps = (gridDim.x * kRopeNormThreads) >> 5;
    const unsigned n_rows = unsigned(p.B) * unsigned(p.T) * unsigned(p.H);
    float gm[8], dg[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        gm[e] = p.gamma[li * 8 + e];
        dg[e] = 0.f;
    }
    const unsigned long long stride = static_cast<unsigned long long>(n_warps) * RPS;
    const unsigned long long first = static_cast<unsigned long long>(warp0) * RPS + sub;
    auto request = [&](unsigned it) {
        const unsigned long long r = first + it * stride;
        if (r < n_rows) {
            int b, t, h;
            rn_decode_row(p, unsigned(r), b, t, h);
            RnBwdStage<F32>& st = ring[it % kBwdDepth];
            const long long xoff = static_cast<long long>(r) * D + li * 8;  // x is dense in walk order
            if constexpr (F32) {
                rn_cp_async16(&st.x0[threadIdx.x], static_cast<const float*>(p.x) + xoff);
                rn_cp_async16(&st.x1[threadIdx.x], static_cast<const float*>(p.x) + xoff + 4);
            } else {
                rn_cp_async16(&st.x0[threadIdx.x], static_cast<const uint16_t*>(p.x) + xoff);
            }
            rn_cp_async16(&st.dy[threadIdx.x], p.dy + (b * p.y_sb + t * p.y_st + h * p.y_sh + li * 8));
            rn_cp_async4(&st.rstd[threadIdx.x], p.rstd + ((static_cast<long long>(b) * p.H + h) * p.T + t));
            rn_cp_async16(&st.cs[threadIdx.x], p.cos_t + static_cast<long long>(t) * (D / 2) + li * 4);
            rn_cp_async16(&st.sn[threadIdx.x], p.sin_t + static_cast<long long>(t) * (D / 2) + li * 4);
        }
        rn_cp_async_commit();
    };
#pragma unroll
    for (int i = 0; i < kBwdDepth - 1; ++i) request(i);
    for (unsigned it = 0; first + it * stride - sub < n_rows; ++it) {
        request(it + kBwdDepth - 1);
        rn_cp_async_wait<kBwdDepth - 1>();
        const unsigned long long r = first + it * stride;
        const bool live = r < n_rows;
        float rot[8], g[8];
        float s = 0.f, rs = 0.f;
        float c[4] = {0.f, 0.f, 0.f, 0.f}, sv[4] = {0.f, 0.f, 0.f, 0.f};
        if (live) {
            const RnBwdStage<F32>& st = ring[it % kBwdDepth];
            float v[8], dyv[8];
            if constexpr (F32) {
                const uint4 a = st.x0[threadIdx.x], q = st.x1[threadIdx.x];
                v[0] = __uint_as_float(a.x), v[1] = __uint_as_float(a.y), v[2] = __uint_as_float(a.z), v[3] = __uint_as_float(a.w);
                v[4] = __uint_as_float(q.x), v[5] = __uint_as_float(q.y), v[6] = __uint_as_float(q.z), v[7] = __uint_as_float(q.w);
            } else {
                const uint4 a = st.x0[threadIdx.x];
                v[0] = rn_bf16_lo(a.x), v[1] = rn_bf16_hi(a.x), v[2] = rn_bf16_lo(a.y), v[3] = rn_bf16_hi(a.y);
                v[4] = rn_bf16_lo(a.z), v[5] = rn_bf16_hi(a.z), v[6] = rn_bf16_lo(a.w), v[7] = rn_bf16_hi(a.w);
            }
            const uint4 d = st.dy[threadIdx.x];
            dyv[0] = rn_bf16_lo(d.x), dyv[1] = rn_bf16_hi(d.x), dyv[2] = rn_bf16_lo(d.y), dyv[3] = rn_bf16_hi(d.y);
            dyv[4] = rn_bf16_lo(d.z), dyv[5] = rn_bf16_hi(d.z), dyv[6] = rn_bf16_lo(d.w), dyv[7] = rn_bf16_hi(d.w);
            const uint4 cw = st.cs[threadIdx.x], sw = st.sn[threadIdx.x];
            c[0] = __uint_as_float(cw.x), c[1] = __uint_as_float(cw.y), c[2] = __uint_as_float(cw.z), c[3] = __uint_as_float(cw.w);
            sv[0] = __uint_as_float(sw.x), sv[1] = __uint_as_float(sw.y), sv[2] = __uint_as_float(sw.z), sv[3] = __uint_as_float(sw.w);
            rs = st.rstd[threadIdx.x];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float x0 = v[2 * i], x1 = v[2 * i + 1];
                rot[2 * i] = x0 * c[i] - x1 * sv[i];
                rot[2 * i + 1] = x0 * sv[i] + x1 * c[i];
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                g[e] = dyv[e] * gm[e];
                s += g[e] * rot[e];
                dg[e] += dyv[e] * rot[e] * rs;
            }
        }
        s = rn_row_sum<LPR>(s);
        if (live) {
            const float coeff = rs * rs * rs * (1.f / float(D)) * s;
            float dx[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float d0 = rs * g[2 * i] - coeff * rot[2 * i];
                const float d1 = rs * g[2 * i + 1] - coeff * rot[2 * i + 1];
                dx[2 * i] = d0 * c[i] + d1 * sv[i];
                dx[2 * i + 1] = -d0 * sv[i] + d1 * c[i];
            }
            rn_store8<F32>(p.y, static_cast<long long>(r) * D + li * 8, dx);
        }
    }
    rn_cp_async_wait<0>();
    // d_gamma: a lane holds sums for its 8 columns over its rows.  Add the lanes that own the same columns
    // (they differ in `sub`), then the warps of the CTA, both in a fixed order.
#pragma unroll
    for (int e = 0; e < 8; ++e) {
#pragma unroll
        for (int o = LPR; o < 32; o <<= 1) dg[e] += __shfl_xor_sync(0xffffffffu, dg[e], o);
    }
    if (sub == 0) {
#pragma unroll
        for (int e = 0; e < 8; ++e) s_part[warp][li * 8 + e] = dg[e];
    }
    __syncthreads();
    for (int d = threadIdx.x; d < D; d += kRopeNormThreads) {
        float acc = 0.f;
#pragma unroll
        for (int w = 0; w < kRopeNormThreads / 32; ++w) acc += s_part[w][d];
        p.partial[static_cast<long long>(blockIdx.x) * D + d] = acc;
    }
    __syncthreads();  // s_part is rewritten for the next tensor
}

template <int D, bool F32>
__global__ void __launch_bounds__(kRopeNormThreads, RN_BWD_BLOCKS)
rope_norm_bwd_kernel(const __grid_constant__ RopeNormParams p0, const __grid_constant__ RopeNormParams p1,
                     const int n_tensors) {
    __shared__ float s_part[kRopeNormThreads / 32][D];
    extern __shared__ uint4 rn_dyn_smem[];
    RnBwdStage<F32>* ring = reinterpret_cast<RnBwdStage<F32>*>(rn_dyn_smem);
    grid_dep_wait();
    rope_norm_bwd_tensor<D, F32>(p0, s_part, ring);
    if (n_tensors > 1) rope_norm_bwd_tensor<D, F32>(p1, s_part, ring);
}

// d_gamma[d] += sum of the CTAs' partial sums, for one or two tensors.  One warp per column (CTA c takes column
// c % D of tensor c / D): lane l adds parts l, l + 32, ... in order, then the 32 lane sums are added in a fixed
// tree, so the result is bit-reproducible; the loads of a lane are independent, which keeps this tail kernel at a
// microsecond or two.  (Done by the last CTA of the backward kernel instead, the same sums took 25 us: one CTA
// cannot keep enough loads in flight.)
template <int D>
__global__ void __launch_bounds__(32) rope_norm_dgamma_kernel(const float* __restrict__ partial0, float* __restrict__ d_gamma0,
                                                              const float* __restrict__ partial1, float* __restrict__ d_gamma1,
                                                              int n_parts) {
    const int ts = blockIdx.x / D, d = blockIdx.x % D, lane = threadIdx.x;
    const float* partial = ts ? partial1 : partial0;
    float* d_gamma = ts ? d_gamma1 : d_gamma0;
    float acc = 0.f;
    grid_dep_wait();  // the partial sums come from the kernel before this one
    for (int i = lane; i < n_parts; i += 32) acc += partial[static_cast<long long>(i) * D + d];
    acc = rn_warp_sum(acc);
    if (lane == 0) d_gamma[d] += acc;
}

}  // namespace b200attn
