// Causal grouped-query attention forward for sm_100a: O = softmax(scale * Q K^T) V and
// L = logsumexp of the scaled scores (natural log), the pair of outputs of the
// reference's flash_attn_forward (llm/src/model/flash_attn.h:25-28,
// llm/src/model/flash_attn.cu:28-131), computed tile-wise on the tensor cores.
//
// One CTA owns one 128-row query tile of one (batch, query head) and walks 64-key tiles of
// K/V up to the diagonal (tiles above it are never loaded).  GQA is an index: the K/V tensor
// maps are addressed with h_kv = h_q / group (llm/src/model/attention.cu:406), nothing is
// replicated.
//
// Roles (256 threads = two warpgroups, so that setmaxnreg can move registers from the
// second group to the first):
//   warps 0-3  softmax + epilogue, thread r owns query row r == TMEM lane r
//   warp  4    TMA producer (converged warp, one elected lane issues)
//   warp  5    TMEM allocation and tcgen05.mma issue (converged warp, one elected lane issues)
//   warps 6-7  idle (they only donate registers)
// TMEM (256 columns): S buffer 0 [0,64), S buffer 1 [64,128) as FP32, each re-used as P
//   (BF16 pairs, 32 columns); O accumulator FP32 [128,128+D).
// With two S buffers the product Q K^T of tile j+1 is issued before the softmax of tile j
// ends, and P V of tile j runs under the softmax of tile j+1.  Two CTAs are resident per
// SM, so prologue and epilogue of one CTA hide under the main loop of the other.
#pragma once

#include "ptx.cuh"

namespace b200attn {

struct FwdParams {
    int B, T, Hq, Hkv, group;
    int n_qtiles;
    float scale;       // softmax scale
    float scale_log2;  // scale * log2(e)
    float* lse;        // [B, Hq, T]
    uint16_t* o;       // output, BF16
    long long o_st, o_sh, o_sb;  // element strides of o: token, head, batch
    int* status;       // device status word
};

template <int D>
struct FwdCfg {
    static constexpr int kKeys = 64;                  // keys per K/V tile
    static constexpr int kStages = (D == 64) ? 4 : 2;
    static constexpr int kQTileBytes = 128 * D * 2;
    static constexpr int kQBoxBytes = 128 * 64 * 2;   // Q/O TMA box: 128 rows x 64 bf16
    static constexpr int kKVTileBytes = kKeys * D * 2;
    static constexpr int kKVBoxBytes = kKeys * 64 * 2;  // K/V TMA box: 64 rows x 64 bf16
    static constexpr int kBoxes = D / 64;
    static constexpr int kBarBytes = 256;
    static constexpr int kSmemBytes = kQTileBytes + 2 * kStages * kKVTileBytes + kBarBytes + 1024;
    static constexpr int kTmemCols = 256;
    static constexpr int kColS0 = 0;
    static constexpr int kColS1 = 64;
    static constexpr int kColO = 128;
};

// log2 of the growth of the row maximum that is tolerated before O and the row
// sum are rescaled; below it the stale maximum stays the exponent reference.
constexpr float kRescaleThresholdLog2 = 8.0f;

template <int D>
__global__ void __launch_bounds__(256, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const FwdParams p) {
    using Cfg = FwdCfg<D>;
    constexpr int NST = Cfg::kStages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;
    uint8_t* sK = sQ + Cfg::kQTileBytes;
    uint8_t* sV = sK + NST * Cfg::kKVTileBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sV + NST * Cfg::kKVTileBytes);
    uint64_t* bar_q = bars + 0;
    uint64_t* bar_s_full = bars + 1;   // [2]
    uint64_t* bar_p_full = bars + 3;   // [2]
    uint64_t* bar_pv_done = bars + 5;
    uint64_t* bar_drain = bars + 6;
    uint64_t* bar_k_full = bars + 7;            // [NST]
    uint64_t* bar_k_free = bars + 7 + NST;      // [NST]
    uint64_t* bar_v_full = bars + 7 + 2 * NST;  // [NST]
    uint64_t* bar_v_free = bars + 7 + 3 * NST;  // [NST]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 24);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 25);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;

    // 1-D grid ordered by work: all CTAs of the heaviest query tile (most key tiles) come first.
    const int n_bh = p.B * p.Hq;
    const int qt = p.n_qtiles - 1 - int(blockIdx.x) / n_bh;
    const int bh = int(blockIdx.x) % n_bh;
    const int h = bh % p.Hq;
    const int b = bh / p.Hq;
    const int hk = h / p.group;
    const int q0 = qt * 128;
    const int k_end = min(p.T, q0 + 128);                  // keys [0, k_end) are visible to this tile
    const int n_kv = (k_end + Cfg::kKeys - 1) / Cfg::kKeys; // 64-key tiles to walk

    B200ATTN_STAMP(tid == 0, 0);
    B200ATTN_TRACE_BEGIN();
    // Set-up with one CTA-wide barrier: one lane of the producer warp reads the device status word
    // (an earlier CTA may already have failed), initialises every mbarrier and immediately starts
    // the first loads, while the MMA warp allocates TMEM.
    grid_dep_launch();
    if (warp == 4 && lane == 0) {
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
        mbar_init(bar_q, 1);
        mbar_init(&bar_s_full[0], 1);
        mbar_init(&bar_s_full[1], 1);
        mbar_init(&bar_p_full[0], 128);
        mbar_init(&bar_p_full[1], 128);
        mbar_init(bar_pv_done, 1);
        mbar_init(bar_drain, 1);
        for (int s = 0; s < NST; ++s) {
            mbar_init(&bar_k_full[s], 1);
            mbar_init(&bar_k_free[s], 1);
            mbar_init(&bar_v_full[s], 1);
            mbar_init(&bar_v_free[s], 1);
        }
        fence_mbar_init();
        grid_dep_wait();  // first global access of this CTA comes next
        const int failed = *reinterpret_cast<volatile int*>(p.status);
        *abort_flag = failed;
        if (!failed) {
            mbar_arrive_expect_tx(bar_q, Cfg::kQTileBytes);
#pragma unroll
            for (int bx = 0; bx < Cfg::kBoxes; ++bx)
                tma_load_4d(sQ + bx * Cfg::kQBoxBytes, &tmQ, bar_q, bx * 64, q0, h, b);
            const int n_pre = n_kv < NST ? n_kv : NST;
            for (int j = 0; j < n_pre; ++j) {
                mbar_arrive_expect_tx(&bar_k_full[j], Cfg::kKVTileBytes);
#pragma unroll
                for (int bx = 0; bx < Cfg::kBoxes; ++bx)
                    tma_load_4d(sK + j * Cfg::kKVTileBytes + bx * Cfg::kKVBoxBytes, &tmK, &bar_k_full[j], bx * 64,
                                j * Cfg::kKeys, hk, b);
                mbar_arrive_expect_tx(&bar_v_full[j], Cfg::kKVTileBytes);
#pragma unroll
                for (int bx = 0; bx < Cfg::kBoxes; ++bx)
                    tma_load_4d(sV + j * Cfg::kKVTileBytes + bx * Cfg::kKVBoxBytes, &tmV, &bar_v_full[j], bx * 64,
                                j * Cfg::kKeys, hk, b);
            }
        }
    }
    if (warp == 5) {
        tmem_alloc(tmem_slot, Cfg::kTmemCols);
        tmem_relinquish();
    }
    grid_dep_wait();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    const bool failed_early = (*abort_flag != 0);
    B200ATTN_STAMP(tid == 0, 1);

    if (failed_early) {
        // nothing was started; fall through to the teardown
    } else
    if (warp >= 6) {
        reg_dealloc<88>();  // idle warps
    } else if (warp == 4) {
        // ------------------------------------------------------------------ producer
        // All 32 lanes run the loop; one elected lane issues the copies.
        reg_dealloc<88>();
        for (int j = NST; j < n_kv; ++j) {  // tiles 0..NST-1 were issued during set-up
            const int s = j % NST;
            const uint32_t use = uint32_t(j / NST);
            if (!mbar_wait_warp(&bar_k_free[s], (use - 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_FREE)) break;
            if (elect_one()) {
                mbar_arrive_expect_tx(&bar_k_full[s], Cfg::kKVTileBytes);
#pragma unroll
                for (int bx = 0; bx < Cfg::kBoxes; ++bx)
                    tma_load_4d(sK + s * Cfg::kKVTileBytes + bx * Cfg::kKVBoxBytes, &tmK, &bar_k_full[s], bx * 64,
                                j * Cfg::kKeys, hk, b);
            }
            __syncwarp();
            if (!mbar_wait_warp(&bar_v_free[s], (use - 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_FREE)) break;
            if (elect_one()) {
                mbar_arrive_expect_tx(&bar_v_full[s], Cfg::kKVTileBytes);
#pragma unroll
                for (int bx = 0; bx < Cfg::kBoxes; ++bx)
                    tma_load_4d(sV + s * Cfg::kKVTileBytes + bx * Cfg::kKVBoxBytes, &tmV, &bar_v_full[s], bx * 64,
                                j * Cfg::kKeys, hk, b);
            }
            __syncwarp();
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------------ MMA issuer
        // All 32 lanes run the loop; one elected lane issues.
        reg_dealloc<88>();
        constexpr uint32_t idesc_s = make_idesc_bf16(128, Cfg::kKeys, 0, 0);
        constexpr uint32_t idesc_o = make_idesc_bf16(128, D, 0, 1);
        const uint64_t q_desc = make_sdesc_sw128(smem_u32(sQ), 16, 1024);
        bool ok = mbar_wait_warp(bar_q, 0, abort_flag, p.status, DEV_WAIT_TIMEOUT_LOAD);
        // S(j) = Q K_j^T into S buffer j & 1
        auto issue_s = [&](int j) -> bool {
            const int s = j % NST;
            if (!mbar_wait_warp(&bar_k_full[s], uint32_t(j / NST) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_LOAD))
                return false;
            tc_fence_after_sync();
            const uint64_t k_desc = make_sdesc_sw128(smem_u32(sK + s * Cfg::kKVTileBytes), 16, 1024);
            if (elect_one()) {
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks)
                    umma_ss(tmem + ((j & 1) ? Cfg::kColS1 : Cfg::kColS0), q_desc + kmajor_step(ks, Cfg::kQBoxBytes),
                            k_desc + kmajor_step(ks, Cfg::kKVBoxBytes), idesc_s, ks > 0);
                umma_commit(&bar_s_full[j & 1]);
                umma_commit(&bar_k_free[s]);
            }
            __syncwarp();
            return true;
        };
        if (ok) ok = issue_s(0);
        if (ok && n_kv > 1) ok = issue_s(1);
        for (int j = 0; j < n_kv && ok; ++j) {
            const int s = j % NST;
            ok = mbar_wait_warp(&bar_p_full[j & 1], uint32_t(j >> 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_SOFTMAX);
            if (!ok) break;
            ok = mbar_wait_warp(&bar_v_full[s], uint32_t(j / NST) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_LOAD);
            if (!ok) break;
            tc_fence_after_sync();
            const uint64_t v_desc = make_sdesc_sw128(smem_u32(sV + s * Cfg::kKVTileBytes), Cfg::kKVBoxBytes, 1024);
            if (elect_one()) {
                // O += P_j V_j : 64 keys = 4 K steps; P lives in the first 32 columns of its S buffer
#pragma unroll
                for (int ks = 0; ks < Cfg::kKeys / 16; ++ks)
                    umma_ts(tmem + Cfg::kColO, tmem + ((j & 1) ? Cfg::kColS1 : Cfg::kColS0) + ks * 8,
                            v_desc + uint64_t(ks * 128), idesc_o, (j > 0) || (ks > 0));
                umma_commit(bar_pv_done);
                umma_commit(&bar_v_free[s]);
            }
            __syncwarp();
            if (j + 2 < n_kv) ok = issue_s(j + 2);
        }
        // Every MMA issued above has completed once this barrier fires; TMEM may then be freed.
        if (elect_one()) umma_commit(bar_drain);
        __syncwarp();
        mbar_wait_warp(bar_drain, 0, abort_flag, p.status, DEV_WAIT_TIMEOUT_MMA);
    } else {
        // ------------------------------------------------------------------ softmax + epilogue
        reg_alloc<168>();
        const int row = tid;                                   // query row inside the tile == TMEM lane
        const uint32_t lane_base = uint32_t(warp * 32) << 16;  // this warp's TMEM lane quadrant
        const uint32_t t_o = tmem + lane_base + Cfg::kColO;
        float m_ref = -INFINITY;  // exponent reference (a past row maximum), raw score units
        float l = 0.f;            // running sum of exp2((s - m_ref) * scale_log2)
        bool ok = true;
        for (int j = 0; j < n_kv; ++j) {
            const uint32_t t_s = tmem + lane_base + ((j & 1) ? Cfg::kColS1 : Cfg::kColS0);
            ok = mbar_wait_warp(&bar_s_full[j & 1], uint32_t(j >> 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_MMA);
            if (!ok) break;
            B200ATTN_STAMP(tid == 0, 8 + 4 * j);
            tc_fence_after_sync();
            uint32_t sr[64];
            tmem_ld_x32(t_s, &sr[0]);
            tmem_ld_x32(t_s + 32, &sr[32]);
            tmem_wait_ld();
            const int kbase = j * Cfg::kKeys;  // first key of this tile
            if (kbase + Cfg::kKeys - 1 > q0) {
                // tile touches the diagonal: key kbase + c is visible to query q0 + row iff it is <= the query
                const int lim = q0 + row - kbase;  // columns c <= lim are visible
#pragma unroll
                for (int c = 0; c < 64; ++c)
                    if (c > lim) sr[c] = 0xff800000u;  // -inf
            }
            float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
            for (int c = 0; c < 64; c += 4) {
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
            for (int c = 0; c < 2; ++c) {
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
                tmem_st_x16(t_s + c * 16, pk);
            }
            l = l * alpha + ((sum0 + sum1) + (sum2 + sum3));
            B200ATTN_STAMP(tid == 0, 9 + 4 * j);
            if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
                // O must hold P V of tile j-1 before it is rescaled
                ok = mbar_wait_warp(bar_pv_done, uint32_t(j - 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_MMA);
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
            mbar_arrive(&bar_p_full[j & 1]);
            B200ATTN_STAMP(tid == 0, 10 + 4 * j);
        }
        // All MMAs of this CTA are complete when the drain barrier fires.  (bar_pv_done cannot be used
        // here: P V of the last TWO tiles may still be in flight, and a parity wait is only
        // unambiguous when the waiter is at most one phase behind.)
        if (ok) ok = mbar_wait(bar_drain, 0, abort_flag, p.status, DEV_WAIT_TIMEOUT_MMA);
        ok = __all_sync(0xffffffffu, ok);
        B200ATTN_STAMP(tid == 0, 2);
        if (ok) {
            tc_fence_after_sync();
            const float inv_l = 1.f / l;
            // O row -> BF16 -> global memory: every thread owns one contiguous row of D elements
            const bool in_range = q0 + row < p.T;
            uint16_t* orow = p.o + size_t(b) * p.o_sb + size_t(h) * p.o_sh + size_t(q0 + row) * p.o_st;
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
                    if (in_range) *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = w;
                }
            }
            if (in_range) p.lse[(size_t(b) * p.Hq + h) * p.T + q0 + row] = m_ref * p.scale + logf(l);
        }
        tc_fence_before_sync();
        B200ATTN_STAMP(tid == 0, 4);
    }

    // teardown: every role falls through to here, also after a wait that gave up
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 5) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, Cfg::kTmemCols);
    }
    B200ATTN_TRACE_END();
}

}  // namespace b200attn
