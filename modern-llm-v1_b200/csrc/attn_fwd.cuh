// Causal grouped-query attention forward for sm_100a: O = softmax(scale * Q K^T) V and
// L = logsumexp of the scaled scores (natural log), the pair of outputs of the
// reference's flash_attn_forward (llm/src/model/flash_attn.h:25-28,
// llm/src/model/flash_attn.cu:28-131), computed tile-wise on the tensor cores.
//
// One CTA owns one 128-row query tile of one (batch, query head) and walks the
// key/value tiles at or below the diagonal (tiles above it are never loaded).
// GQA is an index: the K/V tensor maps are addressed with h_kv = h_q / group
// (llm/src/model/attention.cu:406), nothing is replicated.
//
// Roles (256 threads = two warpgroups, so that setmaxnreg can move registers
// from the second group to the first):
//   warps 0-3  softmax + epilogue, thread r owns query row r == TMEM lane r
//   warp  4    TMA producer (one elected lane)
//   warp  5    TMEM allocation and tcgen05.mma issue (one elected lane)
//   warps 6-7  idle (they only donate registers)
// TMEM (256 columns): [0,128) S as FP32, re-used as P (BF16 pairs) in [0,64);
//                     [128,128+D) O accumulator FP32.
// Two CTAs are resident per SM, so one CTA's softmax overlaps the other's MMAs.
#pragma once

#include "ptx.cuh"

namespace b200attn {

struct FwdParams {
    int B, T, Hq, Hkv, group;
    int n_qtiles;
    float scale;       // softmax scale
    float scale_log2;  // scale * log2(e)
    float* lse;        // [B, Hq, T]
    int* status;       // device status word
};

template <int D>
struct FwdCfg {
    static constexpr int kStages = (D == 64) ? 2 : 1;
    static constexpr int kTileBytes = 128 * D * 2;  // one Q, K or V tile
    static constexpr int kBoxBytes = 128 * 64 * 2;  // one TMA box: 128 rows x 64 bf16
    static constexpr int kBoxes = D / 64;
    static constexpr int kBarBytes = 256;
    static constexpr int kSmemBytes = kTileBytes * (1 + 2 * kStages) + kBarBytes + 1024;
    static constexpr int kTmemCols = 256;
    static constexpr int kColS = 0;
    static constexpr int kColP = 0;
    static constexpr int kColO = 128;
};

// log2 of the growth of the row maximum that is tolerated before O and the row
// sum are rescaled; below it the stale maximum stays the exponent reference.
constexpr float kRescaleThresholdLog2 = 8.0f;

template <int D>
__global__ void __launch_bounds__(256, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                const FwdParams p) {
    using Cfg = FwdCfg<D>;
    constexpr int NST = Cfg::kStages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;
    uint8_t* sK = sQ + Cfg::kTileBytes;
    uint8_t* sV = sK + NST * Cfg::kTileBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sV + NST * Cfg::kTileBytes);
    uint64_t* bar_q = bars + 0;
    uint64_t* bar_s_full = bars + 1;
    uint64_t* bar_p_full = bars + 2;
    uint64_t* bar_o_full = bars + 3;
    uint64_t* bar_drain = bars + 4;
    uint64_t* bar_k_full = bars + 5;           // [NST]
    uint64_t* bar_k_free = bars + 5 + NST;     // [NST]
    uint64_t* bar_v_full = bars + 5 + 2 * NST; // [NST]
    uint64_t* bar_v_free = bars + 5 + 3 * NST; // [NST]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 17);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;

    // Heaviest query tiles (most key tiles) are scheduled first.
    const int qt = p.n_qtiles - 1 - int(blockIdx.x);
    const int h = blockIdx.y;
    const int b = blockIdx.z;
    const int hk = h / p.group;
    const int q0 = qt * 128;
    const int n_kv = qt + 1;  // key tiles 0..qt

    B200ATTN_STAMP(tid == 0, 0);
    // An earlier CTA already failed: leave at once.  The decision is taken by one thread
    // and shared, so that the whole CTA agrees on it.
    if (tid == 0) *abort_flag = *reinterpret_cast<volatile int*>(p.status);
    __syncthreads();
    if (*abort_flag != 0) return;
    __syncthreads();

    if (tid == 0) {
        mbar_init(bar_q, 1);
        mbar_init(bar_s_full, 1);
        mbar_init(bar_p_full, 128);
        mbar_init(bar_o_full, 1);
        mbar_init(bar_drain, 1);
        for (int s = 0; s < NST; ++s) {
            mbar_init(&bar_k_full[s], 1);
            mbar_init(&bar_k_free[s], 1);
            mbar_init(&bar_v_full[s], 1);
            mbar_init(&bar_v_free[s], 1);
        }
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 5) {
        tmem_alloc(tmem_slot, Cfg::kTmemCols);
        tmem_relinquish();
    }
    if (warp == 4 && lane == 0) {
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
        tma_prefetch_desc(&tmO);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    B200ATTN_STAMP(tid == 0, 1);

    if (warp >= 6) {
        reg_dealloc<56>();  // idle warps
    } else if (warp == 4) {
        // ------------------------------------------------------------------ producer
        // All 32 lanes run the loop; one elected lane issues the copies.
        reg_dealloc<56>();
        if (elect_one()) {
            mbar_arrive_expect_tx(bar_q, Cfg::kTileBytes);
#pragma unroll
            for (int bx = 0; bx < Cfg::kBoxes; ++bx)
                tma_load_4d(sQ + bx * Cfg::kBoxBytes, &tmQ, bar_q, bx * 64, q0, h, b);
        }
        __syncwarp();
        for (int j = 0; j < n_kv; ++j) {
            const int s = j % NST;
            const uint32_t use = uint32_t(j / NST);
            if (j >= NST &&
                !mbar_wait_warp(&bar_k_free[s], (use - 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_FREE))
                break;
            if (elect_one()) {
                mbar_arrive_expect_tx(&bar_k_full[s], Cfg::kTileBytes);
#pragma unroll
                for (int bx = 0; bx < Cfg::kBoxes; ++bx)
                    tma_load_4d(sK + s * Cfg::kTileBytes + bx * Cfg::kBoxBytes, &tmK, &bar_k_full[s], bx * 64, j * 128,
                                hk, b);
            }
            __syncwarp();
            if (j >= NST &&
                !mbar_wait_warp(&bar_v_free[s], (use - 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_FREE))
                break;
            if (elect_one()) {
                mbar_arrive_expect_tx(&bar_v_full[s], Cfg::kTileBytes);
#pragma unroll
                for (int bx = 0; bx < Cfg::kBoxes; ++bx)
                    tma_load_4d(sV + s * Cfg::kTileBytes + bx * Cfg::kBoxBytes, &tmV, &bar_v_full[s], bx * 64, j * 128,
                                hk, b);
            }
            __syncwarp();
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------------ MMA issuer
        // All 32 lanes run the loop; one elected lane issues.
        reg_dealloc<56>();
        constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
        constexpr uint32_t idesc_o = make_idesc_bf16(128, D, 0, 1);
        const uint64_t q_desc = make_sdesc_sw128(smem_u32(sQ), 16, 1024);
        bool ok = mbar_wait_warp(bar_q, 0, abort_flag, p.status, DEV_WAIT_TIMEOUT_LOAD);
        for (int j = 0; j < n_kv && ok; ++j) {
            const int s = j % NST;
            const uint32_t ph = uint32_t(j / NST) & 1;
            ok = mbar_wait_warp(&bar_k_full[s], ph, abort_flag, p.status, DEV_WAIT_TIMEOUT_LOAD);
            if (!ok) break;
            B200ATTN_STAMP(lane == 0, 128 + 8 * j);
            tc_fence_after_sync();
            const uint64_t k_desc = make_sdesc_sw128(smem_u32(sK + s * Cfg::kTileBytes), 16, 1024);
            if (elect_one()) {
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks)
                    umma_ss(tmem + Cfg::kColS, q_desc + kmajor_step(ks, Cfg::kBoxBytes),
                            k_desc + kmajor_step(ks, Cfg::kBoxBytes), idesc_s, ks > 0);
                umma_commit(bar_s_full);
                umma_commit(&bar_k_free[s]);
            }
            __syncwarp();
            B200ATTN_STAMP(lane == 0, 129 + 8 * j);
            ok = mbar_wait_warp(bar_p_full, j & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_SOFTMAX);
            if (!ok) break;
            B200ATTN_STAMP(lane == 0, 130 + 8 * j);
            ok = mbar_wait_warp(&bar_v_full[s], ph, abort_flag, p.status, DEV_WAIT_TIMEOUT_LOAD);
            if (!ok) break;
            B200ATTN_STAMP(lane == 0, 131 + 8 * j);
            tc_fence_after_sync();
            const uint64_t v_desc = make_sdesc_sw128(smem_u32(sV + s * Cfg::kTileBytes), Cfg::kBoxBytes, 1024);
            if (elect_one()) {
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)
                    umma_ts(tmem + Cfg::kColO, tmem + Cfg::kColP + ks * 8, v_desc + uint64_t(ks * 128), idesc_o,
                            (j > 0) || (ks > 0));
                umma_commit(bar_o_full);
                umma_commit(&bar_v_free[s]);
            }
            __syncwarp();
            B200ATTN_STAMP(lane == 0, 132 + 8 * j);
        }
        // Every MMA issued above has completed once this barrier fires; TMEM may then be freed.
        if (elect_one()) umma_commit(bar_drain);
        __syncwarp();
        mbar_wait_warp(bar_drain, 0, abort_flag, p.status, DEV_WAIT_TIMEOUT_MMA);
    } else {
        // ------------------------------------------------------------------ softmax + epilogue
        reg_alloc<200>();
        const int row = tid;                                   // query row inside the tile == TMEM lane
        const uint32_t lane_base = uint32_t(warp * 32) << 16;  // this warp's TMEM lane quadrant
        const uint32_t t_s = tmem + lane_base + Cfg::kColS;
        const uint32_t t_p = tmem + lane_base + Cfg::kColP;
        const uint32_t t_o = tmem + lane_base + Cfg::kColO;
        float m_ref = -INFINITY;  // exponent reference (a past row maximum), raw score units
        float l = 0.f;            // running sum of exp2((s - m_ref) * scale_log2)
        bool ok = true;
        for (int j = 0; j < n_kv; ++j) {
            ok = __all_sync(0xffffffffu, mbar_wait(bar_s_full, j & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_MMA));
            if (!ok) break;
            B200ATTN_STAMP(tid == 0, 8 + 8 * j);
            tc_fence_after_sync();
            uint32_t sr[128];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_ld_x32(t_s + c * 32, &sr[c * 32]);
            tmem_wait_ld();
            B200ATTN_STAMP(tid == 0, 9 + 8 * j);
            if (j == qt) {
                // diagonal tile: key column c is visible to query row r iff c <= r
#pragma unroll
                for (int c = 0; c < 128; ++c)
                    if (c > row) sr[c] = 0xff800000u;  // -inf
            }
            float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
            for (int c = 0; c < 128; c += 4) {
                mx0 = fmaxf(mx0, __uint_as_float(sr[c + 0]));
                mx1 = fmaxf(mx1, __uint_as_float(sr[c + 1]));
                mx2 = fmaxf(mx2, __uint_as_float(sr[c + 2]));
                mx3 = fmaxf(mx3, __uint_as_float(sr[c + 3]));
            }
            const float m_new = fmaxf(fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)), m_ref);
            float alpha = 1.f;
            if ((m_new - m_ref) * p.scale_log2 > kRescaleThresholdLog2) {  // also true for m_ref == -inf
                alpha = ex2_approx((m_ref - m_new) * p.scale_log2);
                m_ref = m_new;
            }
            const float neg_m = -m_ref * p.scale_log2;
            float sum0 = 0.f, sum1 = 0.f, sum2 = 0.f, sum3 = 0.f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 16; i += 2) {
                    const float p0 = ex2_approx(fmaf(__uint_as_float(sr[c * 32 + 2 * i + 0]), p.scale_log2, neg_m));
                    const float p1 = ex2_approx(fmaf(__uint_as_float(sr[c * 32 + 2 * i + 1]), p.scale_log2, neg_m));
                    const float p2 = ex2_approx(fmaf(__uint_as_float(sr[c * 32 + 2 * i + 2]), p.scale_log2, neg_m));
                    const float p3 = ex2_approx(fmaf(__uint_as_float(sr[c * 32 + 2 * i + 3]), p.scale_log2, neg_m));
                    sum0 += p0;
                    sum1 += p1;
                    sum2 += p2;
                    sum3 += p3;
                    pk[i + 0] = pack_bf16x2(p0, p1);
                    pk[i + 1] = pack_bf16x2(p2, p3);
                }
                tmem_st_x16(t_p + c * 16, pk);
            }
            l = l * alpha + ((sum0 + sum1) + (sum2 + sum3));
            B200ATTN_STAMP(tid == 0, 10 + 8 * j);
            if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
                // O must hold PV(j-1) before it is rescaled
                ok = mbar_wait(bar_o_full, (j - 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_MMA);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after_sync();
#pragma unroll
                for (int c = 0; c < D / 32; ++c) {
                    uint32_t orr[32];
                    tmem_ld_x32(t_o + c * 32, orr);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) orr[i] = __float_as_uint(__uint_as_float(orr[i]) * alpha);
                    tmem_st_x32(t_o + c * 32, orr);
                }
            }
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(bar_p_full);
            B200ATTN_STAMP(tid == 0, 11 + 8 * j);
        }
        if (ok) ok = mbar_wait(bar_o_full, (n_kv - 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_MMA);
        ok = __all_sync(0xffffffffu, ok);
        B200ATTN_STAMP(tid == 0, 2);
        if (ok) {
            tc_fence_after_sync();
            const float inv_l = 1.f / l;
            // O tile -> BF16 -> shared memory in the 128-byte-swizzled box layout (the Q tile is dead by now)
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
                uint32_t orr[32];
                tmem_ld_x32(t_o + c * 32, orr);
                tmem_wait_ld();
#pragma unroll
                for (int g = 0; g < 4; ++g) {  // 4 chunks of 8 columns (16 bytes)
                    uint4 w;
                    w.x = pack_bf16x2(__uint_as_float(orr[g * 8 + 0]) * inv_l, __uint_as_float(orr[g * 8 + 1]) * inv_l);
                    w.y = pack_bf16x2(__uint_as_float(orr[g * 8 + 2]) * inv_l, __uint_as_float(orr[g * 8 + 3]) * inv_l);
                    w.z = pack_bf16x2(__uint_as_float(orr[g * 8 + 4]) * inv_l, __uint_as_float(orr[g * 8 + 5]) * inv_l);
                    w.w = pack_bf16x2(__uint_as_float(orr[g * 8 + 6]) * inv_l, __uint_as_float(orr[g * 8 + 7]) * inv_l);
                    const int col = c * 32 + g * 8;  // first column of this chunk
                    const int bx = col >> 6;         // 64-column box
                    const int cc = (col & 63) >> 3;  // 16-byte chunk inside the 128-byte row
                    uint8_t* dst = sQ + bx * Cfg::kBoxBytes + row * 128 + ((cc ^ (row & 7)) << 4);
                    *reinterpret_cast<uint4*>(dst) = w;
                }
            }
            if (q0 + row < p.T)
                p.lse[(size_t(b) * p.Hq + h) * p.T + q0 + row] = m_ref * p.scale + logf(l);
            fence_proxy_async_smem();
        }
        tc_fence_before_sync();
        named_bar_sync(1, 128);
        B200ATTN_STAMP(tid == 0, 3);
        if (ok && tid == 0) {
#pragma unroll
            for (int bx = 0; bx < Cfg::kBoxes; ++bx) tma_store_4d(&tmO, sQ + bx * Cfg::kBoxBytes, bx * 64, q0, h, b);
            tma_store_commit();
            tma_store_wait_read0();
        }
        B200ATTN_STAMP(tid == 0, 4);
    }

    // teardown: every role falls through to here, also after a wait that gave up
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 5) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, Cfg::kTmemCols);
    }
}

}  // namespace b200attn
