// Causal grouped-query attention backward for sm_100a in ONE pass over the scores (D = 64).
//
// The reference's flash_attn_backward (llm/src/model/flash_attn.cu:428-504) runs a dQ kernel and a
// dK/dV kernel that each recompute S, P and dP (:175-274 and :277-379): seven products and two
// exponentials per score for five products' worth of results.  Here one kernel, key-tile stationary like
// the dK/dV pass, computes S, P, dP and dS once per 128 x 128 block of scores and uses dS three times:
//      dV += P^T dO        dK += dS^T Q        dQ(query tile) += dS K
// dV and dK stay in tensor memory for the whole item (no atomics, fixed order: bit-reproducible, the group's
// query heads summed in the CTA as in attn_bwd.cuh).  The dQ contribution of a block belongs to a query tile
// that other CTAs contribute to as well, so it is added into an FP32 accumulator in global memory with vector
// reduce-adds (red.global.add.v4.f32, performed in L2) straight from the registers that tcgen05.ld filled; a
// small kernel converts the accumulator to BF16 afterwards.  The order of those additions is not fixed: dQ is NOT bit-reproducible in
// this mode (dK and dV are).  A kernel in front computes D = rowsum(O * dO) and L * log2(e) per row
// (flash_attn_compute_D_kernel, llm/src/model/flash_attn.cu:150-172) and clears the accumulator.
//
// Roles (768 threads = six warpgroups, so that setmaxnreg can move registers to the compute warps):
//   warps 0-15  compute: thread owns TMEM lane (key row) (warp % 4) * 32 + lane and, of the 128 query columns,
//               the two runs 16 p + [0,16) and 64 + 16 p + [0,16) of its part p = warp / 4
//   warps 16-19 drain: thread = TMEM lane; dQ blocks TMEM -> registers -> reduce-add, and the item
//               epilogues (dV, dK -> BF16 -> global memory)
//   warp  20    TMA producer          warp 21  TMEM allocation + tcgen05.mma issue          warps 22-23 idle
// TMEM (512 columns): S buffer 0 [0,128), S buffer 1 [128,256), dP [256,384), dV [384,448), dK [448,512).
//   Unit u (one block of scores) uses S buffer u & 1.  Phase A reads all of S^T(u) into registers at once and
//   writes P^T(u) as BF16 into columns [0,64) of the buffer: columns [64,128) are free from then on and take
//   the dQ block of unit u - 1.  Phase B writes dS^T(u) as BF16 into columns [0,64) of the dP block (operand of
//   dK) and into shared memory (operand of dQ, where the query index has to be the M dimension).
//   Because a part owns two runs of columns, its BF16 values land in its own first run; K step j of the
//   second-stage products therefore covers query rows 16 * (4 * (j & 1) + (j >> 1)) ... + 15.
#pragma once

#include "attn_bwd.cuh"

namespace b200attn {

struct OnePassCfg {
    static constexpr int D = 64;
    static constexpr int kStages = 3;                 // Q / dO tile pairs in flight
    static constexpr int kTileBytes = 128 * D * 2;    // 16 KB
    static constexpr int kDsBytes = 128 * 128 * 2;    // dS^T as BF16: two [128 keys][64 queries] boxes
    static constexpr int kVecBytes = kStages * 2 * 512;
    static constexpr int kBarBytes = 640;
    static constexpr int kSmemBytes = (4 + 2 * kStages) * kTileBytes + kDsBytes + kVecBytes + kBarBytes + 1024;
    static constexpr int kComputeThreads = 512;
    static constexpr int kDrainThreads = 128;
    static constexpr int kDrainWarp0 = 16, kProducerWarp = 20, kMmaWarp = 21;
    static constexpr int kThreads = 24 * 32;  // warps 22-23 only donate registers
    static constexpr int kRegsCompute = 88, kRegsDrain = 64, kRegsCtrl = 64;  // 512 * 88 + 256 * 64 = 768 * 80, the launch allocation
    static constexpr int kTmemCols = 512;
    static constexpr int kColS0 = 0, kColS1 = 128, kColDP = 256, kColDV = 384, kColDK = 448;
    __host__ __device__ static constexpr int col_s(int buf) { return buf ? kColS1 : kColS0; }
    static constexpr int kAccTileFloats = 128 * D;    // one query tile of the FP32 dQ accumulator
};

// Adds four consecutive FP32 values to global memory (16-byte aligned) without returning anything; the addition
// is performed in L2.
__device__ __forceinline__ void red_add_f32x4(float* dst, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(reinterpret_cast<uint64_t>(dst)), "r"(a), "r"(b),
                 "r"(c), "r"(d)
                 : "memory");
}

// D[tmem] (+)= A[tmem, BF16 pairs at a_col .. a_col + 64] * B[smem, MN-major, 128 rows]; K step j of A holds the
// values of B rows 16 * (4 * (j & 1) + (j >> 1)) ... (see the column ownership above).
__device__ __forceinline__ void onepass_ts(uint32_t d_tmem, uint32_t a_col, uint64_t b_desc, uint32_t idesc, bool accumulate) {
#pragma unroll
    for (int j = 0; j < 8; ++j)
        umma_ts(d_tmem, a_col + 8 * j, b_desc + uint64_t((4 * (j & 1) + (j >> 1)) * 128), idesc, accumulate || j > 0);
}

// ---------------------------------------------------------------------------------------
// In front of the one-pass kernel: per query row D = rowsum(O * dO) and L * log2(e) (+inf / 0 in the padding
// rows of the last tile), and the FP32 dQ accumulator cleared.  One CTA of 256 threads per 128-row tile.
// ---------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(256) attn_bwd_prep_kernel(const BwdParams p, float* dq_acc) {
    constexpr int LPR = D / 8;         // lanes per row (16 bytes each)
    constexpr int RPP = 256 / LPR;     // rows per pass
    const int tile = blockIdx.x % p.n_tiles, bh = blockIdx.x / p.n_tiles;
    const int b = bh / p.Hq, h = bh % p.Hq;
    const int q0 = tile * 128;
    grid_dep_wait();
    grid_dep_launch();
    const size_t base = size_t(b) * p.q_sb + size_t(h) * p.q_sh;
#pragma unroll
    for (int pass = 0; pass < 128 / RPP; ++pass) {
        const int r = pass * RPP + threadIdx.x / LPR;
        const int t = q0 + r;
        float acc = 0.f;
        if (t < p.T) {
            const size_t off = base + size_t(t) * p.q_st + (threadIdx.x % LPR) * 8;
            const uint4 a = *reinterpret_cast<const uint4*>(p.o + off);
            const uint4 g = *reinterpret_cast<const uint4*>(p.dout + off);
            const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
            const uint32_t gw[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                acc = fmaf(__uint_as_float(aw[e] << 16), __uint_as_float(gw[e] << 16), acc);
                acc = fmaf(__uint_as_float(aw[e] & 0xffff0000u), __uint_as_float(gw[e] & 0xffff0000u), acc);
            }
        }
#pragma unroll
        for (int o = LPR / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (threadIdx.x % LPR == 0) {
            const size_t vrow = size_t(bh) * p.Tpad + t;
            p.lse2_w[vrow] = t < p.T ? p.lse[size_t(bh) * p.T + t] * 1.4426950408889634f : INFINITY;
            p.dvec_w[vrow] = t < p.T ? acc : 0.f;
        }
    }
    float4* z = reinterpret_cast<float4*>(dq_acc + size_t(blockIdx.x) * (128 * D));
#pragma unroll
    for (int i = 0; i < 128 * D / 4 / 256; ++i) z[i * 256 + threadIdx.x] = make_float4(0.f, 0.f, 0.f, 0.f);
}

// ---------------------------------------------------------------------------------------
// Behind it: accumulator -> dq (times the softmax scale, BF16).  A tile of the accumulator is stored as
// [D / 4 column chunks][128 rows][4 floats] (what the drain warps write without bank conflicts).  One CTA of
// 128 threads per tile, thread = row.
// ---------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(128) attn_bwd_dq_convert_kernel(const BwdParams p, const float* dq_acc) {
    const int tile = blockIdx.x % p.n_tiles, bh = blockIdx.x / p.n_tiles;
    const int b = bh / p.Hq, h = bh % p.Hq;
    const int r = threadIdx.x, t = tile * 128 + r;
    grid_dep_wait();
    const float4* src = reinterpret_cast<const float4*>(dq_acc + size_t(blockIdx.x) * (128 * D)) + r;
    float4 v[D / 4];
#pragma unroll
    for (int c = 0; c < D / 4; ++c) v[c] = __ldcg(src + c * 128);
    if (t < p.T) {
        uint16_t* row = p.dq + size_t(b) * p.q_sb + size_t(h) * p.q_sh + size_t(t) * p.q_st;
#pragma unroll
        for (int c = 0; c < D / 8; ++c) {
            uint4 w;
            w.x = pack_bf16x2(v[2 * c].x * p.scale, v[2 * c].y * p.scale);
            w.y = pack_bf16x2(v[2 * c].z * p.scale, v[2 * c].w * p.scale);
            w.z = pack_bf16x2(v[2 * c + 1].x * p.scale, v[2 * c + 1].y * p.scale);
            w.w = pack_bf16x2(v[2 * c + 1].z * p.scale, v[2 * c + 1].w * p.scale);
            *reinterpret_cast<uint4*>(row + c * 8) = w;
        }
    }
}

// ---------------------------------------------------------------------------------------
// The one-pass kernel: persistent CTAs, one per SM; items and units as in attn_bwd_dkdv_kernel (item = one
// 128-key tile of one (batch, KV head); unit = (query head of the group, 128-query tile at or below the
// diagonal)).  p.lse2 / p.dvec are read; dq_acc is the FP32 accumulator [B * Hq][n_tiles][tile].
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(OnePassCfg::kThreads, 1)
attn_bwd_onepass_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                        const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
                        const BwdParams p, float* dq_acc) {
    using Cfg = OnePassCfg;
    constexpr int D = Cfg::D;
    constexpr int NST = Cfg::kStages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sK = smem;                          // [2]
    uint8_t* sV = sK + 2 * Cfg::kTileBytes;      // [2]
    uint8_t* sQ = sV + 2 * Cfg::kTileBytes;      // [NST]
    uint8_t* sdO = sQ + NST * Cfg::kTileBytes;   // [NST]
    uint8_t* sdS = sdO + NST * Cfg::kTileBytes;  // dS^T of the current unit
    float* sLse = reinterpret_cast<float*>(sdS + Cfg::kDsBytes);  // [NST][128]
    float* sDv = sLse + NST * 128;                                 // [NST][128]
    uint64_t* bars = reinterpret_cast<uint64_t*>(sdS + Cfg::kDsBytes + Cfg::kVecBytes);
    uint64_t* bar_kv = bars + 0;         // [2] K, V of an item have landed                           (phase: item / 2)
    uint64_t* bar_kv_free = bars + 2;    // [2] every product reading them is done                    (phase: item / 2)
    uint64_t* bar_s_full = bars + 4;     // [2] per S buffer: S^T complete                            (phase: unit / 2)
    uint64_t* bar_s_loaded = bars + 6;   // [2] per S buffer: S^T is in registers                     (phase: unit / 2)
    uint64_t* bar_p_full = bars + 8;     // [2] per S buffer: P^T written                             (phase: unit / 2)
    uint64_t* bar_pds_full = bars + 10;  // [2] by unit parity: dS^T written (TMEM and shared memory) (phase: unit / 2)
    uint64_t* bar_dp_full = bars + 12;   //                                                           (phase: unit)
    uint64_t* bar_ds_free = bars + 13;   // the dQ product has read dS^T from shared memory            (phase: unit)
    uint64_t* bar_dq_full = bars + 14;   // [2] by unit parity: dQ block complete                     (phase: unit / 2)
    uint64_t* bar_dq_free = bars + 16;   // [2] by unit parity: dQ block read by the drain warps      (phase: unit / 2)
    uint64_t* bar_acc = bars + 18;       // dV, dK of an item complete                                (phase: item)
    uint64_t* bar_acc_free = bars + 19;  // dV, dK read by the drain warps                            (phase: item)
    uint64_t* bar_full = bars + 20;      // [NST] Q, dO and the two row vectors of a unit have landed
    uint64_t* bar_free = bars + 20 + NST;  // [NST]  (NST <= 4)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 28);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 29);
    uint64_t* bar_item = bars + 32;      // [kItemRing]
    volatile int* item_ring = reinterpret_cast<volatile int*>(bars + 32 + kItemRing);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_bh = p.B * p.Hkv;
    const int n_items = p.n_tiles * n_bh;
    auto item_kt = [&](int id) { return int(fastdiv(unsigned(id), p.div_bhkv)); };
    auto item_rest = [&](int id) { return id - item_kt(id) * n_bh; };  // b * Hkv + hk
    auto item_b = [&](int id) { return int(fastdiv(unsigned(item_rest(id)), p.div_hkv)); };
    auto item_hk = [&](int id) { return item_rest(id) - item_b(id) * p.Hkv; };
    auto item_units = [&](int id) { return p.group * (p.n_tiles - item_kt(id)); };
    auto get_item = [&](int n) { return item_get(bar_item, item_ring, n, abort_flag, p.status); };

    B200ATTN_TRACE_BEGIN(2);
    if (warp == Cfg::kProducerWarp && lane == 0) {
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmdO);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bar_kv[i], 1);
            mbar_init(&bar_kv_free[i], 1);
            mbar_init(&bar_s_full[i], 1);
            mbar_init(&bar_s_loaded[i], Cfg::kComputeThreads);
            mbar_init(&bar_p_full[i], Cfg::kComputeThreads);
            mbar_init(&bar_pds_full[i], Cfg::kComputeThreads);
            mbar_init(&bar_dq_full[i], 1);
            mbar_init(&bar_dq_free[i], Cfg::kDrainThreads);
        }
        mbar_init(bar_dp_full, 1);
        mbar_init(bar_ds_free, 1);
        mbar_init(bar_acc, 1);
        mbar_init(bar_acc_free, Cfg::kDrainThreads);
        for (int s = 0; s < NST; ++s) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_free[s], 1);
        }
        for (int i = 0; i < kItemRing; ++i) mbar_init(&bar_item[i], 1);
        fence_mbar_init();
        grid_dep_wait();  // from here on the kernel in front (row vectors, cleared accumulator) has completed
        *abort_flag = *reinterpret_cast<volatile int*>(p.status);
    }
    if (warp == Cfg::kMmaWarp) {
        tmem_alloc(tmem_slot, Cfg::kTmemCols);
        tmem_relinquish();
    }
    grid_dep_wait();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (*abort_flag != 0) {
        // an earlier CTA already failed: fall through to the teardown
    } else if (warp == Cfg::kProducerWarp) {
        // ------------------------------------------------------------------ producer (whole warp, one lane issues)
        reg_dealloc<Cfg::kRegsCtrl>();
        int u = 0;
        bool ok = true;
        int id = blockIdx.x;
        int id_next = 0;
        if (lane == 0) {
            item_publish(bar_item, item_ring, 0, id);
            id_next = sched_fetch(p.sched2, 1, int(blockIdx.x), int(gridDim.x));
        }
        __syncwarp();
        for (int n = 0; ok; ++n) {
            const int kt = item_kt(id), hk = item_hk(id), b = item_b(id), k0 = kt * 128;
            const int n_i = p.n_tiles - kt, n_it = p.group * n_i;
            const int kb = n & 1;
            if (n >= 2) ok = mbar_wait_warp(&bar_kv_free[kb], uint32_t(n / 2 - 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_FREE);
            if (!ok) break;
            if (elect_one()) {
                mbar_arrive_expect_tx(&bar_kv[kb], 2 * Cfg::kTileBytes);
                tma_load_4d(sK + kb * Cfg::kTileBytes, &tmK, &bar_kv[kb], 0, k0, hk, b);
                tma_load_4d(sV + kb * Cfg::kTileBytes, &tmV, &bar_kv[kb], 0, k0, hk, b);
            }
            __syncwarp();
            const int j_next = max(min(n_it, NST) - 1, n_it - 2);
            int id_new = n_items;
            for (int it = 0, h = hk * p.group, i = kt; it < n_it; ++it, ++u, i = (i + 1 == p.n_tiles ? kt : i + 1), h += (i == kt)) {
                const int s = u % NST;
                if (u >= NST) ok = mbar_wait_warp(&bar_free[s], uint32_t(u / NST - 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_FREE);
                if (!ok) break;
                if (elect_one()) {
                    mbar_arrive_expect_tx(&bar_full[s], 2 * Cfg::kTileBytes + 1024);
                    tma_load_4d(sQ + s * Cfg::kTileBytes, &tmQ, &bar_full[s], 0, i * 128, h, b);
                    tma_load_4d(sdO + s * Cfg::kTileBytes, &tmdO, &bar_full[s], 0, i * 128, h, b);
                    const size_t voff = (size_t(b) * p.Hq + h) * p.Tpad + size_t(i) * 128;
                    bulk_load_1d(sLse + s * 128, p.lse2 + voff, 512, &bar_full[s]);
                    bulk_load_1d(sDv + s * 128, p.dvec + voff, 512, &bar_full[s]);
                }
                __syncwarp();
                if (it == j_next) {
                    id_new = __shfl_sync(0xffffffffu, id_next, 0);
                    if (lane == 0) {
                        item_publish(bar_item, item_ring, n + 1, id_new < n_items ? id_new : -1);
                        if (id_new < n_items) id_next = sched_fetch(p.sched2, n + 2, int(blockIdx.x), int(gridDim.x));
                    }
                    __syncwarp();
                }
            }
            if (!ok || id_new >= n_items) break;
            id = id_new;
        }
        if (ok && lane == 0) sched_finish(p.sched2, int(gridDim.x));
    } else if (warp == Cfg::kMmaWarp) {
        // ------------------------------------------------------------------ MMA issuer (whole warp, one lane issues)
        reg_dealloc<Cfg::kRegsCtrl>();
        constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);   // S^T, dP^T: K-major operands
        constexpr uint32_t idesc_acc = make_idesc_bf16(128, D, 0, 1);   // dV, dK: A in TMEM, B MN-major
        constexpr uint32_t idesc_dq = make_idesc_bf16(128, D, 1, 1);    // dQ: dS^T (M = query) and K both MN-major
        const uint64_t ds_desc = make_sdesc_sw128(smem_u32(sdS), 128 * 64 * 2, 1024);
        // Units of this CTA are numbered u = 0, 1, ... across its items.  Cursors: S^T two units ahead, dP^T one
        // unit ahead of the products that consume P^T and dS^T.
        struct Cursor {
            int n, it, n_it, u;
        };
        bool ok = true;
        auto cursor_start = [&](bool wait) {
            const int id = wait ? get_item(0) : item_ring[0];
            return Cursor{0, 0, id >= 0 ? item_units(id) : 0, 0};
        };
        auto cursor_next = [&](Cursor& c, bool wait) {
            ++c.u;
            if (++c.it == c.n_it) {
                ++c.n;
                c.it = 0;
                const int id = wait ? get_item(c.n) : item_ring[c.n % kItemRing];
                c.n_it = id >= 0 ? item_units(id) : 0;
            }
        };
        // S^T(u) = K Q^T into S buffer u & 1; the upper half of that buffer held the dQ block of unit u - 3
        auto issue_s = [&](const Cursor& c) {
            const int s = c.u % NST, kb = c.n & 1, buf = c.u & 1;
            if (c.it == 0) ok = mbar_wait_warp(&bar_kv[kb], uint32_t(c.n / 2) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_LOAD);
            if (ok) ok = mbar_wait_warp(&bar_full[s], uint32_t(c.u / NST) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_LOAD);
            if (ok && c.u >= 3)
                ok = mbar_wait_warp(&bar_dq_free[(c.u - 3) & 1], uint32_t((c.u - 3) >> 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_FREE);
            if (!ok) return;
            tc_fence_after_sync();
            if (elect_one()) {
                issue_ss_over_headdim<D>(tmem + Cfg::col_s(buf), kmajor_desc<D>(sK + kb * Cfg::kTileBytes),
                                         kmajor_desc<D>(sQ + s * Cfg::kTileBytes), idesc_s);
                umma_commit(&bar_s_full[buf]);
            }
            __syncwarp();
        };
        auto issue_dp = [&](const Cursor& c) {  // dP^T(u) = V dO^T; the unit's loads are known to be complete
            const int s = c.u % NST, kb = c.n & 1;
            if (elect_one()) {
                issue_ss_over_headdim<D>(tmem + Cfg::kColDP, kmajor_desc<D>(sV + kb * Cfg::kTileBytes),
                                         kmajor_desc<D>(sdO + s * Cfg::kTileBytes), idesc_s);
                umma_commit(bar_dp_full);
            }
            __syncwarp();
        };
        Cursor cs = cursor_start(true);
        Cursor cd = cs, ca = cs;
        if (cs.n_it > 0) {
            issue_s(cs);
            cursor_next(cs, true);
            if (ok) {
                issue_dp(cd);
                cursor_next(cd, false);
            }
            if (ok && cs.n_it > 0) {
                issue_s(cs);
                cursor_next(cs, true);
            }
        }
        int n_done = 0;
        int u_last_dq = -1;
        while (ok && ca.n_it > 0) {
            const int u = ca.u, s = u % NST, buf = u & 1, kb = ca.n & 1;
            const bool first = ca.it == 0, last = ca.it + 1 == ca.n_it;
            // dV += P^T dO as soon as P^T is there (it runs under phase B of the compute warps)
            ok = mbar_wait_warp(&bar_p_full[buf], uint32_t(u >> 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_SOFTMAX);
            if (ok && first && ca.n > 0)  // the accumulators belong to the previous item's epilogue until it has read them
                ok = mbar_wait_warp(bar_acc_free, uint32_t(ca.n - 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_SOFTMAX);
            if (!ok) break;
            B200ATTN_STAMP(lane == 0, 16 + 16 * u + 5);
            tc_fence_after_sync();
            if (elect_one())
                onepass_ts(tmem + Cfg::kColDV, tmem + Cfg::col_s(buf), mnmajor_desc<D>(sdO + s * Cfg::kTileBytes), idesc_acc, !first);
            __syncwarp();
            ok = mbar_wait_warp(&bar_pds_full[buf], uint32_t(u >> 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_SOFTMAX);
            if (!ok) break;
            B200ATTN_STAMP(lane == 0, 16 + 16 * u + 6);
            tc_fence_after_sync();
            if (elect_one()) {
                // dK += dS^T Q (dS^T sits in the first 64 columns of the dP block)
                onepass_ts(tmem + Cfg::kColDK, tmem + Cfg::kColDP, mnmajor_desc<D>(sQ + s * Cfg::kTileBytes), idesc_acc, !first);
                umma_commit(&bar_free[s]);
                if (last) umma_commit(bar_acc);
            }
            __syncwarp();
            if (last) ++n_done;
            // dP^T of the next unit: phase B of this unit has read the block, dK above reads it before this overwrites it
            if (cd.n_it > 0) {
                issue_dp(cd);
                cursor_next(cd, false);
            }
            B200ATTN_STAMP(lane == 0, 16 + 16 * u + 7);
            // dQ block of this unit = dS K into the upper half of the OTHER S buffer: S^T(u + 1), if there is one,
            // must be in registers, and the block of unit u - 2 must have been drained from there
            if (cd.u > u + 0 && cs.u > u + 1) {  // unit u + 1 exists and its S^T was issued
                ok = mbar_wait_warp(&bar_s_loaded[(u + 1) & 1], uint32_t((u + 1) >> 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_SOFTMAX);
                if (!ok) break;
            }
            if (u >= 2) {
                ok = mbar_wait_warp(&bar_dq_free[u & 1], uint32_t((u - 2) >> 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_FREE);
                if (!ok) break;
            }
            B200ATTN_STAMP(lane == 0, 16 + 16 * u + 8);
            tc_fence_after_sync();
            if (elect_one()) {
                const uint64_t k_desc = mnmajor_desc<D>(sK + kb * Cfg::kTileBytes);
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)
                    umma_ss(tmem + Cfg::col_s((u + 1) & 1) + 64, ds_desc + uint64_t(ks * 128), k_desc + uint64_t(ks * 128), idesc_dq, ks > 0);
                umma_commit(&bar_dq_full[u & 1]);
                umma_commit(bar_ds_free);
                if (last) umma_commit(&bar_kv_free[kb]);
            }
            __syncwarp();
            u_last_dq = u;
            B200ATTN_STAMP(lane == 0, 16 + 16 * u + 9);
            // S^T two units ahead, into this unit's S buffer (P^T was consumed by dV above)
            if (cs.n_it > 0) {
                issue_s(cs);
                cursor_next(cs, true);
            }
            B200ATTN_STAMP(lane == 0, 16 + 16 * u + 10);
            cursor_next(ca, false);
        }
        // nothing may be in flight when TMEM is freed: the last dQ block's barrier covers every product issued above
        if (ok && u_last_dq >= 0)
            mbar_wait_warp(&bar_dq_full[u_last_dq & 1], uint32_t(u_last_dq >> 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_MMA);
        (void)n_done;
    } else if (warp > Cfg::kMmaWarp) {
        reg_dealloc<Cfg::kRegsCtrl>();  // idle warps
    } else if (warp >= Cfg::kDrainWarp0) {
        // ------------------------------------------------------------------ drain warps
        reg_dealloc<Cfg::kRegsDrain>();
        const int wq = warp - Cfg::kDrainWarp0;
        const int row = wq * 32 + lane;
        const uint32_t lane_base = uint32_t(wq * 32) << 16;
        bool ok = true;
        int u = 0, n = 0;
        for (int id; ok && (id = get_item(n)) >= 0; ++n) {
            const int kt = item_kt(id), hk = item_hk(id), b = item_b(id);
            for (int hg = 0; hg < p.group && ok; ++hg) {
                const int h = hk * p.group + hg;
                for (int i = kt; i < p.n_tiles; ++i, ++u) {
                    const bool last = (hg + 1 == p.group) && (i + 1 == p.n_tiles);
                    if (last) {
                        // the item's dV and dK first (they complete before the last dQ block), so that the
                        // accumulators are free again when the next item's first products are due: each thread
                        // writes its key row, 16 columns (32 bytes) at a time
                        ok = mbar_wait_warp(bar_acc, uint32_t(n) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_MMA);
                        if (!ok) break;
                        tc_fence_after_sync();
                        const int t = kt * 128 + row;
                        const size_t off = size_t(b) * p.k_sb + size_t(hk) * p.k_sh + size_t(t) * p.k_st;
#pragma unroll
                        for (int c = 0; c < 8; ++c) {  // dV columns 0..63, then dK columns 0..63 (dK follows dV in TMEM)
                            uint32_t v[16];
                            tmem_ld_x16(tmem + lane_base + Cfg::kColDV + c * 16, v);
                            tmem_wait_ld();
                            if (c == 7) {
                                tc_fence_before_sync();
                                mbar_arrive(bar_acc_free);
                            }
                            if (t < p.T) {
                                const float mul = c < 4 ? 1.f : p.scale;
                                uint16_t* out = (c < 4 ? p.dv : p.dk) + off + (c & 3) * 16;
#pragma unroll
                                for (int g = 0; g < 2; ++g) {
                                    uint4 w;
                                    w.x = pack_bf16x2(__uint_as_float(v[g * 8 + 0]) * mul, __uint_as_float(v[g * 8 + 1]) * mul);
                                    w.y = pack_bf16x2(__uint_as_float(v[g * 8 + 2]) * mul, __uint_as_float(v[g * 8 + 3]) * mul);
                                    w.z = pack_bf16x2(__uint_as_float(v[g * 8 + 4]) * mul, __uint_as_float(v[g * 8 + 5]) * mul);
                                    w.w = pack_bf16x2(__uint_as_float(v[g * 8 + 6]) * mul, __uint_as_float(v[g * 8 + 7]) * mul);
                                    *reinterpret_cast<uint4*>(out + g * 8) = w;
                                }
                            }
                        }
                    }
                    // the dQ block of this unit: added to the accumulator tile, which is laid out
                    // [16 column chunks][128 rows][4 floats] so that a warp's 32 rows form 512 contiguous bytes
                    ok = mbar_wait_warp(&bar_dq_full[u & 1], uint32_t(u >> 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_MMA);
                    if (!ok) break;
                    B200ATTN_STAMP(tid == Cfg::kDrainWarp0 * 32, 16 + 16 * u + 11);
                    tc_fence_after_sync();
                    const uint32_t t_dq = tmem + lane_base + Cfg::col_s((u + 1) & 1) + 64;
                    float* dst = dq_acc + ((size_t(b) * p.Hq + h) * p.n_tiles + i) * Cfg::kAccTileFloats + row * 4;
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint32_t v[16];
                        tmem_ld_x16(t_dq + c * 16, v);
                        tmem_wait_ld();
                        if (c == 3) {
                            tc_fence_before_sync();
                            mbar_arrive(&bar_dq_free[u & 1]);
                        }
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            red_add_f32x4(dst + (c * 4 + e) * 512, v[4 * e], v[4 * e + 1], v[4 * e + 2], v[4 * e + 3]);
                    }
                    B200ATTN_STAMP(tid == Cfg::kDrainWarp0 * 32, 16 + 16 * u + 14);
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ compute
        reg_alloc<Cfg::kRegsCompute>();
        const int w4 = warp & 3, part = warp >> 2;
        const int row = w4 * 32 + lane;  // key row in the tile == TMEM lane
        const uint32_t lane_base = uint32_t(w4 * 32) << 16;
        const int c0 = part * 16;  // first query column of this thread's two runs (c0 and 64 + c0)
        bool ok = true;
        int u = 0, n = 0;
        for (int id; ok && (id = get_item(n)) >= 0; ++n) {
            const int n_i = p.n_tiles - item_kt(id);
            for (int it = p.group * n_i, i_in = 0; it > 0; --it, ++u, i_in = (i_in + 1 == n_i ? 0 : i_in + 1)) {
                const int s = u % NST, buf = u & 1;
                const uint32_t par2 = uint32_t(u >> 1) & 1;
                const bool diag = i_in == 0;
                const uint32_t t_s = tmem + lane_base + Cfg::col_s(buf) + c0;
                ok = mbar_wait_warp(&bar_s_full[buf], par2, abort_flag, p.status, DEV_WAIT_TIMEOUT_MMA);
                if (!ok) break;
                B200ATTN_STAMP(tid == 0, 16 + 16 * u + 0);
                tc_fence_after_sync();
                // phase A: all of S^T into registers (its buffer's upper half is free from here on), then P^T
                float pr[32];
                {
                    uint32_t sv[32];
                    tmem_ld_x16(t_s, sv);
                    tmem_ld_x16(t_s + 64, sv + 16);
                    tmem_wait_ld();
                    tc_fence_before_sync();
                    mbar_arrive(&bar_s_loaded[buf]);
                    B200ATTN_STAMP(tid == 0, 16 + 16 * u + 1);
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        const float4* lse4 = reinterpret_cast<const float4*>(sLse + s * 128 + hh * 64 + c0);
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            const float4 l4 = lse4[g];
                            float* q = &pr[hh * 16 + g * 4];
                            const uint32_t* x = &sv[hh * 16 + g * 4];
                            q[0] = ex2_approx(fmaf(__uint_as_float(x[0]), p.scale_log2, -l4.x));
                            q[1] = ex2_approx(fmaf(__uint_as_float(x[1]), p.scale_log2, -l4.y));
                            q[2] = ex2_approx(fmaf(__uint_as_float(x[2]), p.scale_log2, -l4.z));
                            q[3] = ex2_approx(fmaf(__uint_as_float(x[3]), p.scale_log2, -l4.w));
                        }
                    }
                }
                if (diag) {
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh)
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            if (hh * 64 + c0 + i < row) pr[hh * 16 + i] = 0.f;  // query above the key: masked
                }
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    uint32_t pk[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) pk[i] = pack_bf16x2(pr[hh * 16 + 2 * i], pr[hh * 16 + 2 * i + 1]);
                    tmem_st_x8(t_s + hh * 8, pk);
                }
                tmem_wait_st();
                tc_fence_before_sync();
                mbar_arrive(&bar_p_full[buf]);
                B200ATTN_STAMP(tid == 0, 16 + 16 * u + 2);
                ok = mbar_wait_warp(bar_dp_full, uint32_t(u) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_MMA);
                // the dQ product of the previous unit must have read dS^T from shared memory
                if (ok && u > 0) ok = mbar_wait_warp(bar_ds_free, uint32_t(u - 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_FREE);
                if (!ok) break;
                B200ATTN_STAMP(tid == 0, 16 + 16 * u + 3);
                tc_fence_after_sync();
                // phase B: dS^T = P^T (dP^T - D) as BF16 into the dP block's first half and into shared memory
                {
                    const uint32_t t_dp = tmem + lane_base + Cfg::kColDP + c0;
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        uint32_t dp[16];
                        tmem_ld_x16(t_dp + hh * 64, dp);
                        tmem_wait_ld();
                        const float4* dv4 = reinterpret_cast<const float4*>(sDv + s * 128 + hh * 64 + c0);
                        uint32_t pk[8];
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            const float4 d4 = dv4[g];
                            const float* q = &pr[hh * 16 + g * 4];
                            const uint32_t* x = &dp[g * 4];
                            pk[g * 2 + 0] = pack_bf16x2(q[0] * (__uint_as_float(x[0]) - d4.x), q[1] * (__uint_as_float(x[1]) - d4.y));
                            pk[g * 2 + 1] = pack_bf16x2(q[2] * (__uint_as_float(x[2]) - d4.z), q[3] * (__uint_as_float(x[3]) - d4.w));
                        }
                        B200ATTN_STAMP(tid == 0, 16 + 16 * u + 12 + hh);
                        tmem_st_x8(t_dp + hh * 8, pk);
                        // shared memory: box hh, key row `row`, query chunks 2 * part and 2 * part + 1 (8 queries each)
                        uint8_t* box = sdS + hh * (128 * 64 * 2) + row * 128;
                        *reinterpret_cast<uint4*>(box + (((2 * part) ^ (row & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                        *reinterpret_cast<uint4*>(box + (((2 * part + 1) ^ (row & 7)) << 4)) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
                    }
                }
                B200ATTN_STAMP(tid == 0, 16 + 16 * u + 15);
                fence_proxy_async_smem();
                tmem_wait_st();
                tc_fence_before_sync();
                mbar_arrive(&bar_pds_full[buf]);
                B200ATTN_STAMP(tid == 0, 16 + 16 * u + 4);
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == Cfg::kMmaWarp) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, Cfg::kTmemCols);
    }
    B200ATTN_TRACE_END(2);
}

}  // namespace b200attn
