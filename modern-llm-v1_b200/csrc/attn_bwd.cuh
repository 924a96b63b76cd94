// Causal grouped-query attention backward for sm_100a, the three steps of the
// reference's flash_attn_backward (llm/src/model/flash_attn.cu:428-504, math :137-146):
//   1. preprocess  D[i] = sum_d O[i,d] dO[i,d]            (flash_attn_compute_D_kernel, :150-172)
//   2. dQ pass     query tile stationary, walks key tiles  (flash_attn_dq_kernel, :175-274)
//   3. dK/dV pass  key tile stationary, walks query tiles  (flash_attn_dkdv_kernel, :277-379)
// with  P = exp(s - L),  dP = dO V^T,  dS = P (dP - D),  dQ = scale dS K,
//       dK = scale dS^T Q,  dV = P^T dO.
// Both passes recompute P from the saved logsumexp on the tensor cores; neither uses
// atomics, so results are bit-reproducible.  GQA: the dK/dV CTA of a KV head loops over
// the query heads of its group and keeps one accumulator, which replaces
// accumulate_kv_grads (llm/src/model/attention.cu:412-429,510-543).
//
// Roles in both passes (320 threads):
//   warps 0-7  compute: thread owns TMEM lane (warp % 4) * 32 + lane and the 64 score
//              columns of its half (warp / 4)
//   warp  8    TMA producer (converged warp, one elected lane issues)
//   warp  9    TMEM allocation and tcgen05.mma issue (converged warp, one elected lane issues)
// TMEM (512 columns), D = 64:  S buffer 0 [0,128), S buffer 1 [128,256), dP [256,384),
//   accumulators [384,448) and [448,512).  With two S buffers the next tile's QK^T product
//   is issued while the compute warps still work on the current tile.
//   D = 128: one S buffer [0,128), dP [128,256), accumulators [256,384) and [384,512).
// The compute step has two phases so that it can start on S before dP has arrived:
//   A: P = exp2(S * scale*log2e - L*log2e)   (kept in registers; the dK/dV pass also stores it)
//   B: dS = P * (dP - D)                      (stored over dP as BF16)
// The BF16 operands of the second-stage MMAs overwrite the FP32 values they were computed
// from: half h of a 128-wide block keeps its 64 BF16 values in the first 32 columns of its
// own 64-column range.
#pragma once

#include "ptx.cuh"

namespace b200attn {

struct BwdParams {
    int B, T, Tpad, Hq, Hkv, group, n_tiles;
    float scale, scale_log2;
    const float* lse2;  // [B, Hq, Tpad]  logsumexp * log2(e); +inf in the padding rows
    const float* dvec;  // [B, Hq, Tpad]  rowsum(O * dO);       0 in the padding rows
    int* status;
};

struct PreParams {
    const uint16_t* o;
    const uint16_t* dout;
    const float* lse;  // [B, Hq, T]
    float* lse2;       // [B, Hq, Tpad]
    float* dvec;       // [B, Hq, Tpad]
    int B, T, Tpad, Hq;
    long long st, sh, sb;  // element strides of o / dout
};

// One thread per 8 head-dim elements; D/8 neighbouring lanes reduce one row.
template <int D>
__global__ void __launch_bounds__(256) attn_bwd_preprocess_kernel(const PreParams p) {
    constexpr int LPR = D / 8;  // lanes per row
    const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long row = gid / LPR;
    const int part = int(gid % LPR);
    const long long rows = (long long)p.B * p.Hq * p.Tpad;
    const bool in_range = row < rows;
    const int t = in_range ? int(row % p.Tpad) : 0;
    const long long bh = in_range ? row / p.Tpad : 0;
    float acc = 0.f;
    if (in_range && t < p.T) {
        const long long off = (bh / p.Hq) * p.sb + (bh % p.Hq) * p.sh + (long long)t * p.st + part * 8;
        const uint4 a = *reinterpret_cast<const uint4*>(p.o + off);
        const uint4 g = *reinterpret_cast<const uint4*>(p.dout + off);
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
        const uint32_t gw[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            acc = fmaf(__uint_as_float(aw[i] << 16), __uint_as_float(gw[i] << 16), acc);
            acc = fmaf(__uint_as_float(aw[i] & 0xffff0000u), __uint_as_float(gw[i] & 0xffff0000u), acc);
        }
    }
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (in_range && part == 0) {
        if (t < p.T) {
            p.dvec[row] = acc;
            p.lse2[row] = p.lse[bh * p.T + t] * 1.4426950408889634f;
        } else {
            p.dvec[row] = 0.f;
            p.lse2[row] = INFINITY;  // exp2(x - inf) = 0: padding query rows contribute nothing
        }
    }
}


template <int D>
struct BwdCfg {
    static constexpr bool kDoubleS = (D == 64);
    static constexpr int kStages = kDoubleS ? 3 : 2;  // streamed operand pairs in shared memory
    static constexpr int kTileBytes = 128 * D * 2;
    static constexpr int kBoxBytes = 128 * 64 * 2;
    static constexpr int kBoxes = D / 64;
    static constexpr int kVecBytes = kStages * 2 * 512;  // per stage (lse2, dvec) of 128 rows
    static constexpr int kBarBytes = 256;
    static constexpr int kSmemBytes = (2 + 2 * kStages) * kTileBytes + kVecBytes + kBarBytes + 1024;
    static constexpr int kTmemCols = 512;
    static constexpr int kColS0 = 0;
    static constexpr int kColS1 = kDoubleS ? 128 : 0;
    static constexpr int kColDP = kDoubleS ? 256 : 128;
    static constexpr int kColAcc0 = kDoubleS ? 384 : 256;
    static constexpr int kColAcc1 = kDoubleS ? 448 : 384;
    __host__ __device__ static constexpr int col_s(int buf) { return buf ? kColS1 : kColS0; }
};

// D[tmem] = A[smem, K-major] * B[smem, K-major]^T over the head dimension; a_desc / b_desc
// describe K step 0 of each operand.
template <int D>
__device__ __forceinline__ void issue_ss_over_headdim(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                                      uint32_t idesc) {
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks)
        umma_ss(d_tmem, a_desc + kmajor_step(ks, BwdCfg<D>::kBoxBytes), b_desc + kmajor_step(ks, BwdCfg<D>::kBoxBytes),
                idesc, ks > 0);
}

// D[tmem] (+)= A[tmem, BF16 pairs] * B[smem, MN-major] over 128 rows of B (b_desc describes
// rows 0..15).  The A operand lives in two 32-column pieces, `a_col` and `a_col + 64`.
template <int D>
__device__ __forceinline__ void issue_ts_over_rows(uint32_t d_tmem, uint32_t a_col, uint64_t b_desc, uint32_t idesc,
                                                   bool accumulate) {
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
        const uint32_t a = a_col + (ks < 4 ? ks * 8 : 64 + (ks - 4) * 8);
        umma_ts(d_tmem, a, b_desc + uint64_t(ks * 128), idesc, accumulate || ks > 0);
    }
}

template <int D>
__device__ __forceinline__ uint64_t kmajor_desc(const void* tile) {
    return make_sdesc_sw128(smem_u32(tile), 16, 1024);
}
template <int D>
__device__ __forceinline__ uint64_t mnmajor_desc(const void* tile) {
    return make_sdesc_sw128(smem_u32(tile), BwdCfg<D>::kBoxBytes, 1024);
}

// Converts 32 FP32 accumulator columns [col, col+32) of this thread's row to BF16 (times
// `mul`) and writes them into a 128-byte-swizzled [128 rows][64] box layout.
template <int D>
__device__ __forceinline__ void stage_row_chunk(uint8_t* tile, int row, int col, const uint32_t* v, float mul) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        uint4 w;
        w.x = pack_bf16x2(__uint_as_float(v[g * 8 + 0]) * mul, __uint_as_float(v[g * 8 + 1]) * mul);
        w.y = pack_bf16x2(__uint_as_float(v[g * 8 + 2]) * mul, __uint_as_float(v[g * 8 + 3]) * mul);
        w.z = pack_bf16x2(__uint_as_float(v[g * 8 + 4]) * mul, __uint_as_float(v[g * 8 + 5]) * mul);
        w.w = pack_bf16x2(__uint_as_float(v[g * 8 + 6]) * mul, __uint_as_float(v[g * 8 + 7]) * mul);
        const int c = col + g * 8;
        const int bx = c >> 6;
        const int cc = (c & 63) >> 3;
        *reinterpret_cast<uint4*>(tile + bx * BwdCfg<D>::kBoxBytes + row * 128 + ((cc ^ (row & 7)) << 4)) = w;
    }
}

// ---------------------------------------------------------------------------------------
// dQ pass: one CTA per (query tile, query head, batch).
// ---------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(320, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                   const __grid_constant__ CUtensorMap tmdQ, const BwdParams p) {
    using Cfg = BwdCfg<D>;
    constexpr int NST = Cfg::kStages;
    constexpr bool DBL = Cfg::kDoubleS;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;
    uint8_t* sdO = sQ + Cfg::kTileBytes;
    uint8_t* sK = sdO + Cfg::kTileBytes;        // [NST]
    uint8_t* sV = sK + NST * Cfg::kTileBytes;   // [NST]
    uint64_t* bars = reinterpret_cast<uint64_t*>(sV + NST * Cfg::kTileBytes + Cfg::kVecBytes);
    uint64_t* bar_q = bars + 0;
    uint64_t* bar_s_full = bars + 1;   // [2] one per S buffer
    uint64_t* bar_dp_full = bars + 3;
    uint64_t* bar_ds_full = bars + 4;
    uint64_t* bar_acc = bars + 5;
    uint64_t* bar_kv_full = bars + 6;          // [NST]
    uint64_t* bar_kv_free = bars + 6 + NST;    // [NST]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 17);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int qt = p.n_tiles - 1 - int(blockIdx.x);
    const int h = blockIdx.y, b = blockIdx.z;
    const int hk = h / p.group;
    const int q0 = qt * 128;
    const int n_kv = qt + 1;

    if (tid == 0) *abort_flag = *reinterpret_cast<volatile int*>(p.status);
    __syncthreads();
    if (*abort_flag != 0) return;
    __syncthreads();

    if (tid == 0) {
        mbar_init(bar_q, 1);
        mbar_init(&bar_s_full[0], 1);
        mbar_init(&bar_s_full[1], 1);
        mbar_init(bar_dp_full, 1);
        mbar_init(bar_ds_full, 256);
        mbar_init(bar_acc, 1);
        for (int s = 0; s < NST; ++s) {
            mbar_init(&bar_kv_full[s], 1);
            mbar_init(&bar_kv_free[s], 1);
        }
        fence_mbar_init();
    }
    if (warp == 9) {
        tmem_alloc(tmem_slot, Cfg::kTmemCols);
        tmem_relinquish();
    }
    if (warp == 8 && lane == 0) {
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
        tma_prefetch_desc(&tmdO);
        tma_prefetch_desc(&tmdQ);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (warp == 8) {
        // ------------------------------------------------------------------ producer (whole warp, one lane issues)
        if (elect_one()) {
            mbar_arrive_expect_tx(bar_q, 2 * Cfg::kTileBytes);
#pragma unroll
            for (int bx = 0; bx < Cfg::kBoxes; ++bx) {
                tma_load_4d(sQ + bx * Cfg::kBoxBytes, &tmQ, bar_q, bx * 64, q0, h, b);
                tma_load_4d(sdO + bx * Cfg::kBoxBytes, &tmdO, bar_q, bx * 64, q0, h, b);
            }
        }
        __syncwarp();
        for (int j = 0; j < n_kv; ++j) {
            const int s = j % NST;
            if (j >= NST &&
                !mbar_wait_warp(&bar_kv_free[s], ((j / NST) - 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_FREE))
                break;
            if (elect_one()) {
                mbar_arrive_expect_tx(&bar_kv_full[s], 2 * Cfg::kTileBytes);
#pragma unroll
                for (int bx = 0; bx < Cfg::kBoxes; ++bx) {
                    tma_load_4d(sK + s * Cfg::kTileBytes + bx * Cfg::kBoxBytes, &tmK, &bar_kv_full[s], bx * 64, j * 128,
                                hk, b);
                    tma_load_4d(sV + s * Cfg::kTileBytes + bx * Cfg::kBoxBytes, &tmV, &bar_kv_full[s], bx * 64, j * 128,
                                hk, b);
                }
            }
            __syncwarp();
        }
    } else if (warp == 9) {
        // ------------------------------------------------------------------ MMA issuer (whole warp, one lane issues)
        constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
        constexpr uint32_t idesc_acc = make_idesc_bf16(128, D, 0, 1);
        const uint64_t q_desc = kmajor_desc<D>(sQ), do_desc = kmajor_desc<D>(sdO);
        bool ok = mbar_wait_warp(bar_q, 0, abort_flag, p.status, DEV_WAIT_TIMEOUT_LOAD);
        // S(j) = Q K_j^T into S buffer (j & 1 when double-buffered); waits for the tile's loads first
        auto issue_s = [&](int j) -> bool {
            const int s = j % NST;
            if (!mbar_wait_warp(&bar_kv_full[s], (j / NST) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_LOAD))
                return false;
            tc_fence_after_sync();
            const int buf = DBL ? (j & 1) : 0;
            if (elect_one()) {
                issue_ss_over_headdim<D>(tmem + Cfg::col_s(buf), q_desc, kmajor_desc<D>(sK + s * Cfg::kTileBytes), idesc_s);
                umma_commit(&bar_s_full[buf]);
            }
            __syncwarp();
            return true;
        };
        auto issue_dp = [&](int j) {  // dP(j) = dO V_j^T; the loads of tile j are known to be complete
            const int s = j % NST;
            if (elect_one()) {
                issue_ss_over_headdim<D>(tmem + Cfg::kColDP, do_desc, kmajor_desc<D>(sV + s * Cfg::kTileBytes), idesc_s);
                umma_commit(bar_dp_full);
            }
            __syncwarp();
        };
        if (ok) ok = issue_s(0);
        if (ok) issue_dp(0);
        if (ok && DBL && n_kv > 1) ok = issue_s(1);
        for (int j = 0; j < n_kv && ok; ++j) {
            const int s = j % NST;
            ok = mbar_wait_warp(bar_ds_full, j & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_SOFTMAX);
            if (!ok) break;
            tc_fence_after_sync();
            if (elect_one()) {
                // dQ += dS K_j
                issue_ts_over_rows<D>(tmem + Cfg::kColAcc0, tmem + Cfg::kColDP, mnmajor_desc<D>(sK + s * Cfg::kTileBytes),
                                      idesc_acc, j > 0);
                umma_commit(&bar_kv_free[s]);
            }
            __syncwarp();
            if (j + 1 < n_kv) {
                if (!DBL) {
                    ok = issue_s(j + 1);
                    if (!ok) break;
                }
                issue_dp(j + 1);  // S(j+1) was issued earlier, so its loads have landed
            }
            if (DBL && j + 2 < n_kv) {
                ok = issue_s(j + 2);
                if (!ok) break;
            }
        }
        if (elect_one()) umma_commit(bar_acc);
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ compute
        const int w4 = warp & 3, half = warp >> 2;
        const int row = w4 * 32 + lane;  // query row in the tile == TMEM lane
        const uint32_t lane_base = uint32_t(w4 * 32) << 16;
        const int c0 = half * 64;  // first key column of this thread's half
        const size_t vrow = (size_t(b) * p.Hq + h) * p.Tpad + q0 + row;
        const float lse2 = p.lse2[vrow];
        const float dv = p.dvec[vrow];
        bool ok = true;
        for (int j = 0; j < n_kv; ++j) {
            const int buf = DBL ? (j & 1) : 0;
            const uint32_t s_par = DBL ? ((j >> 1) & 1) : (j & 1);
            ok = mbar_wait_warp(&bar_s_full[buf], s_par, abort_flag, p.status, DEV_WAIT_TIMEOUT_MMA);
            if (!ok) break;
            tc_fence_after_sync();
            // phase A: P from S
            float pr[64];
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t sv[32];
                tmem_ld_x32(tmem + lane_base + Cfg::col_s(buf) + c0 + c * 32, sv);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    pr[c * 32 + i] = ex2_approx(fmaf(__uint_as_float(sv[i]), p.scale_log2, -lse2));
            }
            if (j == qt) {
#pragma unroll
                for (int i = 0; i < 64; ++i)
                    if (c0 + i > row) pr[i] = 0.f;  // key above the diagonal
            }
            ok = mbar_wait_warp(bar_dp_full, j & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_MMA);
            if (!ok) break;
            tc_fence_after_sync();
            // phase B: dS = P (dP - D), written over dP as BF16
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t dp[32], pk[16];
                tmem_ld_x32(tmem + lane_base + Cfg::kColDP + c0 + c * 32, dp);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    pk[i] = pack_bf16x2(pr[c * 32 + 2 * i] * (__uint_as_float(dp[2 * i]) - dv),
                                        pr[c * 32 + 2 * i + 1] * (__uint_as_float(dp[2 * i + 1]) - dv));
                tmem_st_x16(tmem + lane_base + Cfg::kColDP + c0 + c * 16, pk);
            }
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(bar_ds_full);
        }
        if (ok) ok = mbar_wait(bar_acc, 0, abort_flag, p.status, DEV_WAIT_TIMEOUT_MMA);
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            tc_fence_after_sync();
#pragma unroll
            for (int c = 0; c < D / 64; ++c) {
                uint32_t v[32];
                const int col = half * (D / 2) + c * 32;
                tmem_ld_x32(tmem + lane_base + Cfg::kColAcc0 + col, v);
                tmem_wait_ld();
                stage_row_chunk<D>(sQ, row, col, v, p.scale);
            }
            fence_proxy_async_smem();
        }
        tc_fence_before_sync();
        named_bar_sync(1, 256);
        if (ok && tid == 0) {
#pragma unroll
            for (int bx = 0; bx < Cfg::kBoxes; ++bx) tma_store_4d(&tmdQ, sQ + bx * Cfg::kBoxBytes, bx * 64, q0, h, b);
            tma_store_commit();
            tma_store_wait_read0();
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 9) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, Cfg::kTmemCols);
    }
}

// ---------------------------------------------------------------------------------------
// dK/dV pass: one CTA per (key tile, KV head, batch); loops over the query heads of the
// group and, for each, over the query tiles at or below the diagonal.
// ---------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(320, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                     const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
                     const __grid_constant__ CUtensorMap tmdK, const __grid_constant__ CUtensorMap tmdV,
                     const BwdParams p) {
    using Cfg = BwdCfg<D>;
    constexpr int NST = Cfg::kStages;
    constexpr bool DBL = Cfg::kDoubleS;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sK = smem;
    uint8_t* sV = sK + Cfg::kTileBytes;
    uint8_t* sQ = sV + Cfg::kTileBytes;         // [NST]
    uint8_t* sdO = sQ + NST * Cfg::kTileBytes;  // [NST]
    float* sLse = reinterpret_cast<float*>(sdO + NST * Cfg::kTileBytes);  // [NST][128]
    float* sDv = sLse + NST * 128;                                         // [NST][128]
    uint64_t* bars = reinterpret_cast<uint64_t*>(sdO + NST * Cfg::kTileBytes + Cfg::kVecBytes);
    uint64_t* bar_kv = bars + 0;
    uint64_t* bar_s_full = bars + 1;  // [2]
    uint64_t* bar_dp_full = bars + 3;
    uint64_t* bar_pds_full = bars + 4;
    uint64_t* bar_acc = bars + 5;
    uint64_t* bar_full = bars + 6;        // [NST]
    uint64_t* bar_free = bars + 6 + NST;  // [NST]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 17);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kt = blockIdx.x;  // tile 0 has the most query tiles below it: heaviest first
    const int hk = blockIdx.y, b = blockIdx.z;
    const int k0 = kt * 128;
    const int n_i = p.n_tiles - kt;  // query tiles kt .. n_tiles-1
    const int n_it = p.group * n_i;  // times the query heads of the group

    if (tid == 0) *abort_flag = *reinterpret_cast<volatile int*>(p.status);
    __syncthreads();
    if (*abort_flag != 0) return;
    __syncthreads();

    if (tid == 0) {
        mbar_init(bar_kv, 1);
        mbar_init(&bar_s_full[0], 1);
        mbar_init(&bar_s_full[1], 1);
        mbar_init(bar_dp_full, 1);
        mbar_init(bar_pds_full, 256);
        mbar_init(bar_acc, 1);
        for (int s = 0; s < NST; ++s) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_free[s], 1);
        }
        fence_mbar_init();
    }
    if (warp == 9) {
        tmem_alloc(tmem_slot, Cfg::kTmemCols);
        tmem_relinquish();
    }
    if (warp == 8 && lane == 0) {
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmdO);
        tma_prefetch_desc(&tmdK);
        tma_prefetch_desc(&tmdV);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (warp == 8) {
        // ------------------------------------------------------------------ producer (whole warp, one lane issues)
        if (elect_one()) {
            mbar_arrive_expect_tx(bar_kv, 2 * Cfg::kTileBytes);
#pragma unroll
            for (int bx = 0; bx < Cfg::kBoxes; ++bx) {
                tma_load_4d(sK + bx * Cfg::kBoxBytes, &tmK, bar_kv, bx * 64, k0, hk, b);
                tma_load_4d(sV + bx * Cfg::kBoxBytes, &tmV, bar_kv, bx * 64, k0, hk, b);
            }
        }
        __syncwarp();
        for (int it = 0; it < n_it; ++it) {
            const int s = it % NST;
            const int h = hk * p.group + it / n_i;
            const int i = kt + it % n_i;
            if (it >= NST &&
                !mbar_wait_warp(&bar_free[s], ((it / NST) - 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_FREE))
                break;
            if (elect_one()) {
                mbar_arrive_expect_tx(&bar_full[s], 2 * Cfg::kTileBytes + 1024);
#pragma unroll
                for (int bx = 0; bx < Cfg::kBoxes; ++bx) {
                    tma_load_4d(sQ + s * Cfg::kTileBytes + bx * Cfg::kBoxBytes, &tmQ, &bar_full[s], bx * 64, i * 128, h,
                                b);
                    tma_load_4d(sdO + s * Cfg::kTileBytes + bx * Cfg::kBoxBytes, &tmdO, &bar_full[s], bx * 64, i * 128,
                                h, b);
                }
                const size_t voff = (size_t(b) * p.Hq + h) * p.Tpad + size_t(i) * 128;
                bulk_load_1d(sLse + s * 128, p.lse2 + voff, 512, &bar_full[s]);
                bulk_load_1d(sDv + s * 128, p.dvec + voff, 512, &bar_full[s]);
            }
            __syncwarp();
        }
    } else if (warp == 9) {
        // ------------------------------------------------------------------ MMA issuer (whole warp, one lane issues)
        constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
        constexpr uint32_t idesc_acc = make_idesc_bf16(128, D, 0, 1);
        const uint64_t k_desc = kmajor_desc<D>(sK), v_desc = kmajor_desc<D>(sV);
        bool ok = mbar_wait_warp(bar_kv, 0, abort_flag, p.status, DEV_WAIT_TIMEOUT_LOAD);
        auto issue_s = [&](int it) -> bool {  // S^T(it) = K Q^T
            const int s = it % NST;
            if (!mbar_wait_warp(&bar_full[s], (it / NST) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_LOAD)) return false;
            tc_fence_after_sync();
            const int buf = DBL ? (it & 1) : 0;
            if (elect_one()) {
                issue_ss_over_headdim<D>(tmem + Cfg::col_s(buf), k_desc, kmajor_desc<D>(sQ + s * Cfg::kTileBytes), idesc_s);
                umma_commit(&bar_s_full[buf]);
            }
            __syncwarp();
            return true;
        };
        auto issue_dp = [&](int it) {  // dP^T(it) = V dO^T; the loads of `it` are known to be complete
            const int s = it % NST;
            if (elect_one()) {
                issue_ss_over_headdim<D>(tmem + Cfg::kColDP, v_desc, kmajor_desc<D>(sdO + s * Cfg::kTileBytes), idesc_s);
                umma_commit(bar_dp_full);
            }
            __syncwarp();
        };
        if (ok) ok = issue_s(0);
        if (ok) issue_dp(0);
        if (ok && DBL && n_it > 1) ok = issue_s(1);
        for (int it = 0; it < n_it && ok; ++it) {
            const int s = it % NST;
            const int buf = DBL ? (it & 1) : 0;
            ok = mbar_wait_warp(bar_pds_full, it & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_SOFTMAX);
            if (!ok) break;
            B200ATTN_STAMP(lane == 0, 200 + 4 * it);
            tc_fence_after_sync();
            if (elect_one()) {
                // dV += P^T dO ; dK += dS^T Q
                issue_ts_over_rows<D>(tmem + Cfg::kColAcc0, tmem + Cfg::col_s(buf),
                                      mnmajor_desc<D>(sdO + s * Cfg::kTileBytes), idesc_acc, it > 0);
                issue_ts_over_rows<D>(tmem + Cfg::kColAcc1, tmem + Cfg::kColDP, mnmajor_desc<D>(sQ + s * Cfg::kTileBytes),
                                      idesc_acc, it > 0);
                umma_commit(&bar_free[s]);
            }
            __syncwarp();
            B200ATTN_STAMP(lane == 0, 201 + 4 * it);
            if (it + 1 < n_it) {
                if (!DBL) {
                    ok = issue_s(it + 1);
                    if (!ok) break;
                }
                issue_dp(it + 1);
            }
            if (DBL && it + 2 < n_it) {
                ok = issue_s(it + 2);
                if (!ok) break;
            }
            B200ATTN_STAMP(lane == 0, 202 + 4 * it);
        }
        if (elect_one()) umma_commit(bar_acc);
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ compute
        const int w4 = warp & 3, half = warp >> 2;
        const int row = w4 * 32 + lane;  // key row in the tile == TMEM lane
        const uint32_t lane_base = uint32_t(w4 * 32) << 16;
        const int c0 = half * 64;  // first query column of this thread's half
        bool ok = true;
        for (int it = 0; it < n_it; ++it) {
            const int s = it % NST;
            const int buf = DBL ? (it & 1) : 0;
            const uint32_t s_par = DBL ? ((it >> 1) & 1) : (it & 1);
            const bool diag = (it % n_i) == 0;
            ok = mbar_wait_warp(&bar_s_full[buf], s_par, abort_flag, p.status, DEV_WAIT_TIMEOUT_MMA);
            if (!ok) break;
            B200ATTN_STAMP(tid == 0, 8 + 4 * it);
            tc_fence_after_sync();
            const float4* lse4 = reinterpret_cast<const float4*>(sLse + s * 128 + c0);
            const float4* dv4 = reinterpret_cast<const float4*>(sDv + s * 128 + c0);
            // phase A: P^T from S^T (kept in registers and stored over S^T as BF16)
            float pr[64];
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t sv[32], pk[16];
                tmem_ld_x32(tmem + lane_base + Cfg::col_s(buf) + c0 + c * 32, sv);
                tmem_wait_ld();
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                    const float4 l4 = lse4[c * 8 + g];
                    pr[c * 32 + g * 4 + 0] = ex2_approx(fmaf(__uint_as_float(sv[g * 4 + 0]), p.scale_log2, -l4.x));
                    pr[c * 32 + g * 4 + 1] = ex2_approx(fmaf(__uint_as_float(sv[g * 4 + 1]), p.scale_log2, -l4.y));
                    pr[c * 32 + g * 4 + 2] = ex2_approx(fmaf(__uint_as_float(sv[g * 4 + 2]), p.scale_log2, -l4.z));
                    pr[c * 32 + g * 4 + 3] = ex2_approx(fmaf(__uint_as_float(sv[g * 4 + 3]), p.scale_log2, -l4.w));
                }
                if (diag) {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (c0 + c * 32 + i < row) pr[c * 32 + i] = 0.f;  // query above the key: masked
                }
#pragma unroll
                for (int i = 0; i < 16; ++i) pk[i] = pack_bf16x2(pr[c * 32 + 2 * i], pr[c * 32 + 2 * i + 1]);
                tmem_st_x16(tmem + lane_base + Cfg::col_s(buf) + c0 + c * 16, pk);
            }
            ok = mbar_wait_warp(bar_dp_full, it & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_MMA);
            if (!ok) break;
            B200ATTN_STAMP(tid == 0, 10 + 4 * it);
            tc_fence_after_sync();
            // phase B: dS^T = P^T (dP^T - D), stored over dP^T as BF16
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t dp[32], pk[16];
                tmem_ld_x32(tmem + lane_base + Cfg::kColDP + c0 + c * 32, dp);
                tmem_wait_ld();
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                    const float4 d4 = dv4[c * 8 + g];
                    const int i = c * 32 + g * 4;
                    pk[g * 2 + 0] = pack_bf16x2(pr[i + 0] * (__uint_as_float(dp[g * 4 + 0]) - d4.x),
                                                pr[i + 1] * (__uint_as_float(dp[g * 4 + 1]) - d4.y));
                    pk[g * 2 + 1] = pack_bf16x2(pr[i + 2] * (__uint_as_float(dp[g * 4 + 2]) - d4.z),
                                                pr[i + 3] * (__uint_as_float(dp[g * 4 + 3]) - d4.w));
                }
                tmem_st_x16(tmem + lane_base + Cfg::kColDP + c0 + c * 16, pk);
            }
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(bar_pds_full);
            B200ATTN_STAMP(tid == 0, 9 + 4 * it);
        }
        if (ok) ok = mbar_wait(bar_acc, 0, abort_flag, p.status, DEV_WAIT_TIMEOUT_MMA);
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            tc_fence_after_sync();
            // half 0 drains dV into the first Q stage, half 1 drains dK (times scale) into the first dO stage
            uint8_t* tile = half == 0 ? sQ : sdO;
            const uint32_t acc = half == 0 ? Cfg::kColAcc0 : Cfg::kColAcc1;
            const float mul = half == 0 ? 1.f : p.scale;
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
                uint32_t v[32];
                tmem_ld_x32(tmem + lane_base + acc + c * 32, v);
                tmem_wait_ld();
                stage_row_chunk<D>(tile, row, c * 32, v, mul);
            }
            fence_proxy_async_smem();
        }
        tc_fence_before_sync();
        named_bar_sync(1, 256);
        if (ok && tid == 0) {
#pragma unroll
            for (int bx = 0; bx < Cfg::kBoxes; ++bx) {
                tma_store_4d(&tmdV, sQ + bx * Cfg::kBoxBytes, bx * 64, k0, hk, b);
                tma_store_4d(&tmdK, sdO + bx * Cfg::kBoxBytes, bx * 64, k0, hk, b);
            }
            tma_store_commit();
            tma_store_wait_read0();
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 9) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, Cfg::kTmemCols);
    }
}

}  // namespace b200attn
