// Split-KV decode for sm_100a: one query token per sequence against a KV cache.
// The reference has no such path (infer_modern_gpt re-runs the whole forward per token,
// llm/apps/infer_modern_gpt.cu:253-255); the math is row L-1 of its causal attention
// (llm/src/model/flash_attn.cu:28-131) with T = L.
//
// The kernel is bound by HBM: every K and V byte of the cache is read exactly once.
// A CTA owns one (batch, KV head, split of the cache length) and serves ALL query heads of
// the group from the same K/V tile, which is the whole bandwidth win of GQA.  K/V tiles
// (128 keys) stream through a 3-stage shared-memory ring filled by TMA (128-byte swizzle,
// which also makes the row-per-thread reads bank-conflict free).
//
// Roles (160 threads): warps 0-3 compute (thread t <-> key t of the tile for q.k; warp w,
// lane <-> head-dim pair for p.V over the warp's own 32 keys), warp 4 = TMA producer.
// Each split writes an un-normalised partial (m, l, O); a small combine kernel merges them.
#pragma once

#include "ptx.cuh"

namespace b200attn {

struct DecodeParams {
    int B, L, Hq, Hkv, group;
    int G;         // query heads served per CTA (a divisor of group, <= 8)
    int n_chunks;  // group / G
    int n_splits;
    int tiles_per_split;
    float scale, scale_log2;
    const uint16_t* q;  // [B, Hq, D]
    float* part_o;      // [B, Hq, n_splits, D]
    float* part_m;      // [B, Hq, n_splits]   row maximum, raw score units
    float* part_l;      // [B, Hq, n_splits]   sum of exp2((s - m) * scale_log2)
    int* status;
};

template <int D>
struct DecodeCfg {
    static constexpr int kStages = 3;
    static constexpr int kTileKeys = 128;
    static constexpr int kTileBytes = kTileKeys * D * 2;
    static constexpr int kBoxBytes = 128 * 64 * 2;
    static constexpr int kBoxes = D / 64;
    static constexpr int kMaxG = 8;
    // K and V rings, q (G x D floats), p (128 x G floats), cross-warp scratch
    static constexpr int kSmemBytes =
        2 * kStages * kTileBytes + kMaxG * D * 4 + 128 * kMaxG * 4 + 4 * kMaxG * D * 4 + 256 + 1024;
};

template <int D, int G>
__global__ void __launch_bounds__(160)
attn_decode_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                   const DecodeParams p) {
    using Cfg = DecodeCfg<D>;
    constexpr int NST = Cfg::kStages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sK = smem;
    uint8_t* sV = sK + NST * Cfg::kTileBytes;
    float* sQ = reinterpret_cast<float*>(sV + NST * Cfg::kTileBytes);  // [G][D]
    float* sP = sQ + Cfg::kMaxG * D;                                    // [128][G]
    float* sRed = sP + 128 * Cfg::kMaxG;                                // [4][G][D] / [4][G]
    uint64_t* bars = reinterpret_cast<uint64_t*>(sRed + 4 * Cfg::kMaxG * D);
    uint64_t* bar_full = bars;         // [NST]
    uint64_t* bar_free = bars + NST;   // [NST]
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * NST);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int split = blockIdx.x;
    const int hk = int(blockIdx.y) / p.n_chunks;
    const int chunk = int(blockIdx.y) % p.n_chunks;
    const int b = blockIdx.z;
    const int h0 = hk * p.group + chunk * G;  // first query head served here
    const int tile0 = split * p.tiles_per_split;
    const int n_all = (p.L + 127) / 128;
    const int n_tiles = max(0, min(p.tiles_per_split, n_all - tile0));

    if (tid == 0) *abort_flag = *reinterpret_cast<volatile int*>(p.status);
    __syncthreads();
    if (*abort_flag != 0) return;
    __syncthreads();

    if (tid == 0) {
        for (int s = 0; s < NST; ++s) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_free[s], 128);
        }
        fence_mbar_init();
    }
    // q rows of the G heads -> FP32 in shared memory
    for (int i = tid; i < G * D; i += blockDim.x) {
        const uint32_t raw = p.q[(size_t(b) * p.Hq + h0) * D + i];
        sQ[i] = __uint_as_float(raw << 16);
    }
    __syncthreads();

    if (warp == 4) {
        if (lane == 0) {
            tma_prefetch_desc(&tmK);
            tma_prefetch_desc(&tmV);
            for (int j = 0; j < n_tiles; ++j) {
                const int s = j % NST;
                if (j >= NST &&
                    !mbar_wait(&bar_free[s], ((j / NST) - 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_FREE))
                    break;
                mbar_arrive_expect_tx(&bar_full[s], 2 * Cfg::kTileBytes);
#pragma unroll
                for (int bx = 0; bx < Cfg::kBoxes; ++bx) {
                    tma_load_4d(sK + s * Cfg::kTileBytes + bx * Cfg::kBoxBytes, &tmK, &bar_full[s], bx * 64,
                                (tile0 + j) * 128, hk, b);
                    tma_load_4d(sV + s * Cfg::kTileBytes + bx * Cfg::kBoxBytes, &tmV, &bar_full[s], bx * 64,
                                (tile0 + j) * 128, hk, b);
                }
            }
        }
        return;
    }

    // ---------------------------------------------------------------------- compute warps
    constexpr int DPT = D / 32;  // head-dim elements per lane in the p.V phase (2 or 4)
    float m_run[G], l_part[G], acc[G][DPT];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m_run[g] = -INFINITY;
        l_part[g] = 0.f;
#pragma unroll
        for (int e = 0; e < DPT; ++e) acc[g][e] = 0.f;
    }
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
        const int s = j % NST;
        // A wait that gives up sets the CTA's abort word; the barrier makes every compute thread
        // see the same word, so the whole group leaves the loop together (no thread is left
        // behind at a later named barrier).
        mbar_wait(&bar_full[s], (j / NST) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_LOAD);
        named_bar_sync(1, 128);
        if (*abort_flag != 0) {
            ok = false;
            break;
        }
        const uint8_t* kt = sK + s * Cfg::kTileBytes;
        const uint8_t* vt = sV + s * Cfg::kTileBytes;
        // ---- scores of key `tid` against the G heads
        float sc[G];
#pragma unroll
        for (int g = 0; g < G; ++g) sc[g] = 0.f;
#pragma unroll
        for (int c = 0; c < D / 8; ++c) {
            const int bx = c >> 3, cc = c & 7;
            const uint4 kw = *reinterpret_cast<const uint4*>(kt + bx * Cfg::kBoxBytes + tid * 128 + ((cc ^ (tid & 7)) << 4));
            const uint32_t w[4] = {kw.x, kw.y, kw.z, kw.w};
            float kf[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                kf[2 * i] = __uint_as_float(w[i] << 16);
                kf[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
            }
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float4 qa = *reinterpret_cast<const float4*>(sQ + g * D + c * 8);
                const float4 qb = *reinterpret_cast<const float4*>(sQ + g * D + c * 8 + 4);
                sc[g] = fmaf(kf[0], qa.x, sc[g]);
                sc[g] = fmaf(kf[1], qa.y, sc[g]);
                sc[g] = fmaf(kf[2], qa.z, sc[g]);
                sc[g] = fmaf(kf[3], qa.w, sc[g]);
                sc[g] = fmaf(kf[4], qb.x, sc[g]);
                sc[g] = fmaf(kf[5], qb.y, sc[g]);
                sc[g] = fmaf(kf[6], qb.z, sc[g]);
                sc[g] = fmaf(kf[7], qb.w, sc[g]);
            }
        }
        const bool valid = (tile0 + j) * 128 + tid < p.L;
        // ---- tile maximum per head: warp shuffle, then across the 4 warps
        float mx[G];
#pragma unroll
        for (int g = 0; g < G; ++g) {
            if (!valid) sc[g] = -INFINITY;
            mx[g] = sc[g];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mx[g] = fmaxf(mx[g], __shfl_xor_sync(0xffffffffu, mx[g], o));
        }
        float* sMax = sRed;  // [4][G]
        if (lane == 0) {
#pragma unroll
            for (int g = 0; g < G; ++g) sMax[warp * G + g] = mx[g];
        }
        named_bar_sync(1, 128);
        float pv[G];
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const float m_new = fmaxf(fmaxf(fmaxf(sMax[g], sMax[G + g]), fmaxf(sMax[2 * G + g], sMax[3 * G + g])), m_run[g]);
            const float alpha = ex2_approx((m_run[g] - m_new) * p.scale_log2);  // 0 on the first tile
            m_run[g] = m_new;
            pv[g] = ex2_approx((sc[g] - m_new) * p.scale_log2);
            l_part[g] = l_part[g] * alpha + pv[g];
#pragma unroll
            for (int e = 0; e < DPT; ++e) acc[g][e] *= alpha;
            sP[tid * G + g] = pv[g];
        }
        named_bar_sync(1, 128);  // also orders the sMax reads before the next tile's writes
        // ---- O += p V over this warp's own 32 keys; lane owns DPT consecutive head-dim elements
#pragma unroll 4
        for (int kk = 0; kk < 32; ++kk) {
            const int key = warp * 32 + kk;
            const int col = lane * DPT;  // first head-dim element of this lane
            const int bx = col >> 6, cc = (col & 63) >> 3;
            const uint8_t* src = vt + bx * Cfg::kBoxBytes + key * 128 + ((cc ^ (key & 7)) << 4) + (col & 7) * 2;
            float vf[DPT];
            if (DPT == 2) {
                const uint32_t w = *reinterpret_cast<const uint32_t*>(src);
                vf[0] = __uint_as_float(w << 16);
                vf[1] = __uint_as_float(w & 0xffff0000u);
            } else {
                const uint2 w = *reinterpret_cast<const uint2*>(src);
                vf[0] = __uint_as_float(w.x << 16);
                vf[1] = __uint_as_float(w.x & 0xffff0000u);
                vf[2] = __uint_as_float(w.y << 16);
                vf[3] = __uint_as_float(w.y & 0xffff0000u);
            }
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float pg = sP[key * G + g];
#pragma unroll
                for (int e = 0; e < DPT; ++e) acc[g][e] = fmaf(pg, vf[e], acc[g][e]);
            }
        }
        mbar_arrive(&bar_free[s]);
    }
    if (!ok) return;
    // ---- reduce l over all threads and O over the 4 warps, write the partial
    float* sAcc = sRed;  // [4][G][D]
    named_bar_sync(1, 128);
#pragma unroll
    for (int g = 0; g < G; ++g) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) l_part[g] += __shfl_xor_sync(0xffffffffu, l_part[g], o);
#pragma unroll
        for (int e = 0; e < DPT; ++e) sAcc[(warp * G + g) * D + lane * DPT + e] = acc[g][e];
    }
    float* sL = sP;  // [4][G]
    if (lane == 0) {
#pragma unroll
        for (int g = 0; g < G; ++g) sL[warp * G + g] = l_part[g];
    }
    named_bar_sync(1, 128);
    for (int i = tid; i < G * D; i += 128) {
        const int g = i / D, d = i % D;
        const float o = sAcc[(0 * G + g) * D + d] + sAcc[(1 * G + g) * D + d] + sAcc[(2 * G + g) * D + d] +
                        sAcc[(3 * G + g) * D + d];
        p.part_o[((size_t(b) * p.Hq + h0 + g) * p.n_splits + split) * D + d] = o;
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
        if (tid == g) {
            const size_t idx = (size_t(b) * p.Hq + h0 + g) * p.n_splits + split;
            p.part_m[idx] = m_run[g];
            p.part_l[idx] = sL[g] + sL[G + g] + sL[2 * G + g] + sL[3 * G + g];
        }
    }
}

// Merges the per-split partials: one warp per (batch, query head).
template <int D>
__global__ void __launch_bounds__(128)
attn_decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_m,
                           const float* __restrict__ part_l, uint16_t* __restrict__ o, float* __restrict__ lse,
                           int n_rows, int n_splits, float scale, float scale_log2) {
    const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= n_rows) return;
    float m = -INFINITY;
    for (int s = 0; s < n_splits; ++s) m = fmaxf(m, part_m[(size_t)row * n_splits + s]);
    constexpr int DPT = D / 32;
    float acc[DPT];
#pragma unroll
    for (int e = 0; e < DPT; ++e) acc[e] = 0.f;
    float l = 0.f;
    for (int s = 0; s < n_splits; ++s) {
        const float ms = part_m[(size_t)row * n_splits + s];
        const float w = (ms == -INFINITY) ? 0.f : ex2_approx((ms - m) * scale_log2);  // empty split
        l += w * part_l[(size_t)row * n_splits + s];
#pragma unroll
        for (int e = 0; e < DPT; ++e) acc[e] += w * part_o[((size_t)row * n_splits + s) * D + lane * DPT + e];
    }
    const float inv = 1.f / l;
    if (DPT == 2) {
        reinterpret_cast<uint32_t*>(o)[(size_t)row * (D / 2) + lane] = pack_bf16x2(acc[0] * inv, acc[1] * inv);
    } else {
        uint2 w;
        w.x = pack_bf16x2(acc[0] * inv, acc[1] * inv);
        w.y = pack_bf16x2(acc[2] * inv, acc[3] * inv);
        reinterpret_cast<uint2*>(o)[(size_t)row * (D / 4) + lane] = w;
    }
    if (lse && lane == 0) lse[row] = m * scale + logf(l);
}

}  // namespace b200attn
