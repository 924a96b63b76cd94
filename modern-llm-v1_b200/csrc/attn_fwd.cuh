// Causal grouped-query attention forward for sm_100a: O = softmax(scale * Q K^T) V and
// L = logsumexp of the scaled scores (natural log), the pair of outputs of the
// reference's flash_attn_forward (llm/src/model/flash_attn.h:25-28,
// llm/src/model/flash_attn.cu:28-131), computed tile-wise on the tensor cores.
//
// Persistent CTAs, two per SM.  A CTA walks a static list of work items (item = one 128-row
// query tile of one (batch, query head); items are ordered heaviest first and dealt by a host-built
// table, see ItemTable) and, per item, the 64-key tiles of K/V up to the diagonal (tiles above it are
// never loaded).  Every pipeline keeps running across item boundaries: the K/V ring prefetches
// the next item's tiles and the MMA warp issues the next item's first Q K^T products while the
// softmax warps write the previous item's output rows.  GQA is an index: the K/V tensor maps are
// addressed with h_kv = h_q / group (llm/src/model/attention.cu:406), nothing is replicated.
//
// Roles (256 threads = two warpgroups, so that setmaxnreg can move registers from the
// second group to the first):
//   warps 0-3  softmax + epilogue, thread r owns query row r == TMEM lane r
//   warp  4    TMA producer (converged warp, one elected lane issues)
//   warp  5    TMEM allocation and tcgen05.mma issue (converged warp, one elected lane issues)
//   warps 6-7  idle (they only donate registers)
// TMEM (256 columns): two S buffers of 64 FP32 columns, each re-used as P (BF16 pairs, 32 columns); the O
//   accumulator (FP32, D columns) behind them; for D = 64 two Q buffers of 32 columns behind that.
// Q in tensor memory (D = 64): every D = 64 kernel here is bound by the shared-memory data path (an SS product
//   M128 N64 K16 fetches 4 KB of A and 2 KB of B for 32 clocks of math), and Q is the same for all key tiles of an
//   item.  The softmax warps therefore copy an item's Q tile once from shared memory into tensor memory (the
//   128 bytes of row r are the 32 BF16-pair columns of lane r as they stand) and Q K^T is issued with the A
//   operand in tensor memory, like P V: per key tile the products then read 16 KB of shared memory instead of 32.
// The MMA warp's work is a chain softmax(g) -> P V(g) -> Q K^T(g + buffers) -> softmax(g + buffers);
// with several S buffers the products Q K^T run that many tiles ahead of the softmax, and P V of
// tile g runs under the softmax of tile g+1.
#pragma once

#include "ptx.cuh"

namespace b200attn {

struct FwdParams {
    int B, T, Hq, Hkv, group;
    int n_qtiles;
    int kv_off;        // keys in front of the first query row: query row t sees keys 0 .. kv_off + t (0 when q and k
                       // cover the same tokens; the cached tokens' count when a chunk of new tokens attends over a KV cache)
    float scale;       // softmax scale
    float scale_log2;  // scale * log2(e)
    float* lse;        // [B, Hq, T]
    uint16_t* o;       // output, BF16
    long long o_st, o_sh, o_sb;  // element strides of o: token, head, batch
    int* status;       // device status word
    int* sched;        // two words of the device-wide item counter (see ptx.cuh)
    FastDiv div_bh, div_h, div_group;  // division by B * Hq, by Hq and by the group size
};

template <int D>
struct FwdCfg {
    static constexpr int kKeys = 64;                  // keys per K/V tile
    static constexpr int kStages = (D == 64) ? 4 : 2;
    static constexpr int kQBufs = (D == 64) ? 2 : 1;  // Q tiles in shared memory (the next item's Q is prefetched)
    static constexpr int kQTileBytes = 128 * D * 2;
    static constexpr int kQBoxBytes = 128 * 64 * 2;   // Q TMA box: 128 rows x 64 bf16
    static constexpr int kKVTileBytes = kKeys * D * 2;
    static constexpr int kKVBoxBytes = kKeys * 64 * 2;  // K/V TMA box: 64 rows x 64 bf16
    static constexpr int kBoxes = D / 64;
    static constexpr int kBarBytes = 384;
    static constexpr bool kQInTmem = (D == 64);
    static constexpr int kSmemBytes = kQBufs * kQTileBytes + 2 * kStages * kKVTileBytes + kBarBytes + 1024;
    static constexpr int kTmemCols = 256;
    static constexpr int kSBufs = 2;
    static constexpr int kColO = kSBufs * 64;
    static constexpr int kColQ = kColO + D;  // D = 64 only: [192, 224) and [224, 256)
    __host__ __device__ static constexpr int col_s(int buf) { return buf * 64; }
};

// log2 of the growth of the row maximum that is tolerated before O and the row
// sum are rescaled; below it the stale maximum stays the exponent reference.
constexpr float kRescaleThresholdLog2 = 8.0f;

template <int D>
__global__ void __launch_bounds__(256, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const FwdParams p, const __grid_constant__ ItemTable tab) {
    using Cfg = FwdCfg<D>;
    constexpr int NST = Cfg::kStages;
    constexpr int NQB = Cfg::kQBufs;
    constexpr int NSB = Cfg::kSBufs;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;
    uint8_t* sK = sQ + NQB * Cfg::kQTileBytes;
    uint8_t* sV = sK + NST * Cfg::kKVTileBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sV + NST * Cfg::kKVTileBytes);
    uint64_t* bar_q = bars + 0;        // [2] per Q buffer: Q of an item has landed              (phase: item / NQB)
    uint64_t* bar_q_free = bars + 2;   // [2] per Q buffer: every Q K^T product of the item done (phase: item / NQB)
    uint64_t* bar_s_full = bars + 4;   // [NSB] per S buffer                                      (phase: tile / NSB)
    uint64_t* bar_p_full = bars + 7;   // [NSB] per S buffer: P written, O rescaled               (phase: tile / NSB)
    uint64_t* bar_pv_done = bars + 10; // P V of a tile is complete                               (phase: tile)
    uint64_t* bar_o_done = bars + 11;  // O of an item is complete                                (phase: item)
    uint64_t* bar_o_free = bars + 12;  // O has been read by the epilogue                         (phase: item)
    uint64_t* bar_k_full = bars + 13;            // [NST]
    uint64_t* bar_k_free = bars + 13 + NST;      // [NST]
    uint64_t* bar_v_full = bars + 13 + 2 * NST;  // [NST]
    uint64_t* bar_v_free = bars + 13 + 3 * NST;  // [NST]
    uint64_t* bar_item = bars + 32;    // [kItemRing] item ids handed out by the producer
    volatile int* item_ring = reinterpret_cast<volatile int*>(bars + 32 + kItemRing);
    uint64_t* bar_qs_free = bars + 44;  // [2] per Q buffer: the tile in shared memory has been copied (phase: item / NQB)
    uint64_t* bar_qt_full = bars + 46;  // [2] per Q buffer: Q of an item is in tensor memory          (phase: item / NQB)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 30);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 31);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;

    // item id -> (query tile, head, batch); ids are ordered by work, heaviest query tile first
    const int n_bh = p.B * p.Hq;
    const int n_items = p.n_qtiles * n_bh;
    auto get_item = [&](int n) { return item_get(bar_item, item_ring, n, abort_flag, p.status); };
    auto item_rest = [&](int id) { return id - int(fastdiv(unsigned(id), p.div_bh)) * n_bh; };  // b * Hq + h
    auto item_qt = [&](int id) { return p.n_qtiles - 1 - int(fastdiv(unsigned(id), p.div_bh)); };
    auto item_b = [&](int id) { return int(fastdiv(unsigned(item_rest(id)), p.div_h)); };
    auto item_h = [&](int id) { return item_rest(id) - item_b(id) * p.Hq; };
    auto item_nkv = [&](int id) { return (p.kv_off + min(p.T, item_qt(id) * 128 + 128) + Cfg::kKeys - 1) / Cfg::kKeys; };

    B200ATTN_TRACE_BEGIN(0);
    // Set-up with one CTA-wide barrier: one lane of the producer warp initialises every mbarrier while
    // the MMA warp allocates TMEM; nothing touches global memory before grid_dep_wait().
    if (warp == 4 && lane == 0) {
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bar_q[i], 1);
            mbar_init(&bar_q_free[i], 1);
            mbar_init(&bar_qs_free[i], 128);
            mbar_init(&bar_qt_full[i], 128);
        }
        for (int i = 0; i < NSB; ++i) {
            mbar_init(&bar_s_full[i], 1);
            mbar_init(&bar_p_full[i], 128);
        }
        mbar_init(bar_pv_done, 1);
        mbar_init(bar_o_done, 1);
        mbar_init(bar_o_free, 128);
        for (int s = 0; s < NST; ++s) {
            mbar_init(&bar_k_full[s], 1);
            mbar_init(&bar_k_free[s], 1);
            mbar_init(&bar_v_full[s], 1);
            mbar_init(&bar_v_free[s], 1);
        }
        for (int i = 0; i < kItemRing; ++i) mbar_init(&bar_item[i], 1);
        fence_mbar_init();
        grid_dep_wait();  // first global access of this CTA comes next
        *abort_flag = *reinterpret_cast<volatile int*>(p.status);
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

    if (*abort_flag != 0) {
        // an earlier CTA already failed: fall through to the teardown
    } else if (warp >= 6) {
        reg_dealloc<88>();  // idle warps
    } else if (warp == 4) {
        // ------------------------------------------------------------------ producer
        reg_dealloc<88>();
        int g = 0;  // key tiles issued so far by this CTA (ring position)
        bool ok = true;
        int id_next = 0;  // lane 0: the id fetched for the item after the next Q load
        // Q of this CTA's n-th item (item id `id`) into Q buffer n % NQB
        auto load_q = [&](int n, int id) {
            const int qb = n % NQB;
            if (n >= NQB)
                ok = mbar_wait_warp(Cfg::kQInTmem ? &bar_qs_free[qb] : &bar_q_free[qb], uint32_t(n / NQB - 1) & 1, abort_flag,
                                    p.status, DEV_WAIT_TIMEOUT_FREE);
            if (!ok) return;
            if (elect_one()) {
                mbar_arrive_expect_tx(&bar_q[qb], Cfg::kQTileBytes);
#pragma unroll
                for (int bx = 0; bx < Cfg::kBoxes; ++bx)
                    tma_load_4d(sQ + qb * Cfg::kQTileBytes + bx * Cfg::kQBoxBytes, &tmQ, &bar_q[qb], bx * 64,
                                item_qt(id) * 128, item_h(id), item_b(id));
            }
            __syncwarp();
        };
        int id = sched_first(tab, p.sched, int(blockIdx.x));  // the first item needs no fetch
        if (lane == 0) {
            item_publish(bar_item, item_ring, 0, id);
            id_next = sched_fetch(tab, p.sched, 1, int(blockIdx.x), int(gridDim.x));
        }
        __syncwarp();
        load_q(0, id);
        for (int n = 0; ok; ++n) {
            const int h = item_h(id), b = item_b(id), hk = int(fastdiv(unsigned(h), p.div_group)), n_kv = item_nkv(id);
            // The next item is taken, announced and its Q requested a few tiles before this item's loads end
            // (late, so that a CTA commits itself to little work ahead, but not before the ring has been
            // filled for this item); with one Q buffer, after this item's last tile (it is free only then).
            const int j_next = NQB > 1 ? max(min(n_kv, NST) - 1, n_kv - 3) : n_kv - 1;
            int id_new = n_items;
            for (int j = 0; j < n_kv; ++j, ++g) {
                const int s = g % NST;
                const uint32_t use = uint32_t(g / NST);
                if (g >= NST) ok = mbar_wait_warp(&bar_k_free[s], (use - 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_FREE);
                if (!ok) break;
                if (elect_one()) {
                    mbar_arrive_expect_tx(&bar_k_full[s], Cfg::kKVTileBytes);
#pragma unroll
                    for (int bx = 0; bx < Cfg::kBoxes; ++bx)
                        tma_load_4d(sK + s * Cfg::kKVTileBytes + bx * Cfg::kKVBoxBytes, &tmK, &bar_k_full[s], bx * 64,
                                    j * Cfg::kKeys, hk, b);
                }
                __syncwarp();
                if (g >= NST) ok = mbar_wait_warp(&bar_v_free[s], (use - 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_FREE);
                if (!ok) break;
                if (elect_one()) {
                    mbar_arrive_expect_tx(&bar_v_full[s], Cfg::kKVTileBytes);
#pragma unroll
                    for (int bx = 0; bx < Cfg::kBoxes; ++bx)
                        tma_load_4d(sV + s * Cfg::kKVTileBytes + bx * Cfg::kKVBoxBytes, &tmV, &bar_v_full[s], bx * 64,
                                    j * Cfg::kKeys, hk, b);
                }
                __syncwarp();
                if (j == j_next) {
                    id_new = __shfl_sync(0xffffffffu, id_next, 0);
                    const bool more = id_new < n_items;
                    if (lane == 0) {
                        item_publish(bar_item, item_ring, n + 1, more ? id_new : -1);
                        if (more) id_next = sched_fetch(tab, p.sched, n + 2, int(blockIdx.x), int(gridDim.x));
                    }
                    __syncwarp();
                    if (more) load_q(n + 1, id_new);
                    if (!ok) break;
                }
            }
            if (!ok || id_new >= n_items) break;
            id = id_new;
        }
        if (ok && lane == 0) sched_finish(p.sched, int(gridDim.x));
    } else if (warp == 5) {
        // ------------------------------------------------------------------ MMA issuer
        reg_dealloc<88>();
        constexpr uint32_t idesc_s = make_idesc_bf16(128, Cfg::kKeys, 0, 0);
        constexpr uint32_t idesc_o = make_idesc_bf16(128, D, 0, 1);
        // This CTA's key tiles are numbered g = 0, 1, ... across all its items: ring stage g % NST,
        // S buffer g % NSB.  The cursor `sc` walks that sequence for the products Q K^T, NSB tiles ahead
        // of the loop below that issues the products P V, also across item boundaries.
        struct Cursor {
            int id, n, j, n_kv, g;  // item id, items before it on this CTA, tile in item, tiles of item, global tile
        };
        Cursor sc{get_item(0), 0, 0, 0, 0};
        if (sc.id >= 0) sc.n_kv = item_nkv(sc.id);
        bool ok = true;
        auto issue_next_s = [&]() {
            if (sc.id < 0) return;
            const int s = sc.g % NST, qb = sc.n % NQB;
            if (sc.j == 0)
                ok = mbar_wait_warp(Cfg::kQInTmem ? &bar_qt_full[qb] : &bar_q[qb], uint32_t(sc.n / NQB) & 1, abort_flag, p.status,
                                    DEV_WAIT_TIMEOUT_LOAD);
            if (ok) ok = mbar_wait_warp(&bar_k_full[s], uint32_t(sc.g / NST) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_LOAD);
            if (!ok) return;
            tc_fence_after_sync();
            const uint64_t q_desc = make_sdesc_sw128(smem_u32(sQ + qb * Cfg::kQTileBytes), 16, 1024);
            const uint64_t k_desc = make_sdesc_sw128(smem_u32(sK + s * Cfg::kKVTileBytes), 16, 1024);
            const bool last = sc.j + 1 == sc.n_kv;  // no later MMA reads this item's Q
            if (elect_one()) {
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    if constexpr (Cfg::kQInTmem)
                        umma_ts(tmem + Cfg::col_s(sc.g % NSB), tmem + Cfg::kColQ + qb * 32 + ks * 8,
                                k_desc + kmajor_step(ks, Cfg::kKVBoxBytes), idesc_s, ks > 0);
                    else
                        umma_ss(tmem + Cfg::col_s(sc.g % NSB), q_desc + kmajor_step(ks, Cfg::kQBoxBytes),
                                k_desc + kmajor_step(ks, Cfg::kKVBoxBytes), idesc_s, ks > 0);
                }
                umma_commit(&bar_s_full[sc.g % NSB]);
                umma_commit(&bar_k_free[s]);
                if (last) umma_commit(&bar_q_free[qb]);
            }
            __syncwarp();
            ++sc.g;
            if (++sc.j == sc.n_kv) {
                sc.id = get_item(++sc.n);
                sc.j = 0;
                sc.n_kv = sc.id >= 0 ? item_nkv(sc.id) : 0;
            }
        };
        for (int i = 0; i < NSB && ok; ++i) issue_next_s();
        int g = 0, n = 0;
        // (this warp has already waited for the ring entry of item n: the cursor above is never behind)
        for (int id; ok && (id = item_ring[n % kItemRing]) >= 0; ++n) {
            const int n_kv = item_nkv(id);
            for (int j = 0; j < n_kv && ok; ++j, ++g) {
                const int s = g % NST;
                ok = mbar_wait_warp(&bar_p_full[g % NSB], uint32_t(g / NSB) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_SOFTMAX);
                if (!ok) break;
                B200ATTN_STAMP(lane == 0, 16 + 8 * g + 4);
                // the accumulator belongs to the previous item's epilogue until it has been read
                if (j == 0 && n > 0) {
                    ok = mbar_wait_warp(bar_o_free, uint32_t(n - 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_SOFTMAX);
                    if (!ok) break;
                }
                ok = mbar_wait_warp(&bar_v_full[s], uint32_t(g / NST) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_LOAD);
                if (!ok) break;
                tc_fence_after_sync();
                const uint64_t v_desc = make_sdesc_sw128(smem_u32(sV + s * Cfg::kKVTileBytes), Cfg::kKVBoxBytes, 1024);
                if (elect_one()) {
                    // O += P V : 64 keys = 4 K steps; P lives in the first 32 columns of its S buffer
#pragma unroll
                    for (int ks = 0; ks < Cfg::kKeys / 16; ++ks)
                        umma_ts(tmem + Cfg::kColO, tmem + Cfg::col_s(g % NSB) + ks * 8,
                                v_desc + uint64_t(ks * 128), idesc_o, (j > 0) || (ks > 0));
                    umma_commit(bar_pv_done);
                    umma_commit(&bar_v_free[s]);
                    if (j + 1 == n_kv) umma_commit(bar_o_done);
                }
                __syncwarp();
                B200ATTN_STAMP(lane == 0, 16 + 8 * g + 5);
                issue_next_s();  // tile g + NSB: its S buffer was read by the P V just issued
                B200ATTN_STAMP(lane == 0, 16 + 8 * g + 6);
            }
        }
        // nothing may be in flight when TMEM is freed: the last commit covers every MMA issued above
        if (ok && n > 0) mbar_wait_warp(bar_o_done, uint32_t(n - 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_MMA);
    } else {
        // ------------------------------------------------------------------ softmax + epilogue
        reg_alloc<168>();
        const int row = tid;                                   // query row inside the tile == TMEM lane
        const uint32_t lane_base = uint32_t(warp * 32) << 16;  // this warp's TMEM lane quadrant
        const uint32_t t_o = tmem + lane_base + Cfg::kColO;
        bool ok = true;
        // Epilogue of one item: O / l -> BF16 -> global memory, logsumexp.  (bar_pv_done cannot be used for
        // "O is complete": P V of the last TWO tiles may still be in flight, and a parity wait is only
        // unambiguous when the waiter is at most one phase behind; bar_o_done completes once per item.)
        auto epilogue = [&](int n_item, int id, float m_ref, float l) -> bool {
            B200ATTN_STAMP(tid == 0, 400 + 4 * n_item + 0);
            if (!mbar_wait_warp(bar_o_done, uint32_t(n_item) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_MMA)) return false;
            B200ATTN_STAMP(tid == 0, 400 + 4 * n_item + 1);
            tc_fence_after_sync();
            const float inv_l = 1.f / l;
            const int q0 = item_qt(id) * 128, b = item_b(id), h = item_h(id);
            const bool in_range = q0 + row < p.T;
            uint16_t* orow = p.o + size_t(b) * p.o_sb + size_t(h) * p.o_sh + size_t(q0 + row) * p.o_st;
            // every thread owns one contiguous row of D elements, written 64 columns at a time
#pragma unroll
            for (int hh = 0; hh < D / 64; ++hh) {
                uint32_t ow[32];  // 64 columns as BF16 pairs
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    uint32_t orr[32];
                    tmem_ld_x32(t_o + hh * 64 + c * 32, orr);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        ow[c * 16 + i] = pack_bf16x2(__uint_as_float(orr[2 * i]) * inv_l, __uint_as_float(orr[2 * i + 1]) * inv_l);
                }
                if (hh + 1 == D / 64) {
                    // the accumulator has been read: the next item's first P V may overwrite it
                    tc_fence_before_sync();
                    mbar_arrive(bar_o_free);
                }
                B200ATTN_STAMP(tid == 0, 440 + 4 * n_item + 0);
                if (in_range) {
#pragma unroll
                    for (int c = 0; c < 8; ++c)
                        *reinterpret_cast<uint4*>(orow + hh * 64 + c * 8) =
                            make_uint4(ow[c * 4], ow[c * 4 + 1], ow[c * 4 + 2], ow[c * 4 + 3]);
                }
            }
            B200ATTN_STAMP(tid == 0, 440 + 4 * n_item + 1);
            if (in_range) p.lse[(size_t(b) * p.Hq + h) * p.T + q0 + row] = m_ref * p.scale + logf(l);
            B200ATTN_STAMP(tid == 0, 400 + 4 * n_item + 2);
            return true;
        };
        // D = 64: Q of this CTA's n-th item from shared memory into Q buffer n % NQB of tensor memory.  The buffer
        // held Q of item n - NQB, whose last Q K^T product must have completed.
        auto copy_q = [&](int n_item) -> bool {
            const int qb = n_item % NQB;
            if (!mbar_wait_warp(&bar_q[qb], uint32_t(n_item / NQB) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_LOAD)) return false;
            if (n_item >= NQB &&
                !mbar_wait_warp(&bar_q_free[qb], uint32_t(n_item / NQB - 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_FREE))
                return false;
            tc_fence_after_sync();
            uint32_t qw[32];
            const uint8_t* qrow = sQ + qb * Cfg::kQTileBytes + row * 128;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const uint4 w = *reinterpret_cast<const uint4*>(qrow + ((c ^ (row & 7)) << 4));
                qw[4 * c] = w.x, qw[4 * c + 1] = w.y, qw[4 * c + 2] = w.z, qw[4 * c + 3] = w.w;
            }
            tmem_st_x32(tmem + lane_base + Cfg::kColQ + qb * 32, qw);
            fence_proxy_async_smem();  // ordinary reads before the async proxy (TMA) overwrites the tile
            mbar_arrive(&bar_qs_free[qb]);  // the values are in registers: the tile in shared memory may be reloaded
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(&bar_qt_full[qb]);
            return true;
        };
        if constexpr (Cfg::kQInTmem) {
            if (get_item(0) >= 0) ok = copy_q(0);
        }
        // The epilogue of an item is deferred until the softmax of the next item's first tile has been handed
        // to the MMA warp: the wait for the item's last P V then overlaps useful work.
        bool pending = false;
        int pend_id = 0;
        float pend_m = 0.f, pend_l = 1.f;
        int g = 0, n = 0;
        for (int id; ok && (id = get_item(n)) >= 0; ++n) {
            const int qt = item_qt(id), h = item_h(id), b = item_b(id), n_kv = item_nkv(id);
            const int q0 = qt * 128;
            float m_ref = -INFINITY;  // exponent reference (a past row maximum), raw score units
            float l = 0.f;            // running sum of exp2((s - m_ref) * scale_log2)
            for (int j = 0; j < n_kv; ++j, ++g) {
                if constexpr (Cfg::kQInTmem) {
                    // the next item's Q, a few tiles before the MMA warp wants it for that item's first products
                    if (j == max(0, n_kv - 3) && get_item(n + 1) >= 0) {
                        ok = copy_q(n + 1);
                        if (!ok) break;
                    }
                }
                const uint32_t t_s = tmem + lane_base + Cfg::col_s(g % NSB);
                ok = mbar_wait_warp(&bar_s_full[g % NSB], uint32_t(g / NSB) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_MMA);
                if (!ok) break;
                B200ATTN_STAMP(tid == 0, 16 + 8 * g + 0);
                tc_fence_after_sync();
                uint32_t sr[64];
                tmem_ld_x32(t_s, &sr[0]);
                tmem_ld_x32(t_s + 32, &sr[32]);
                tmem_wait_ld();
                const int kbase = j * Cfg::kKeys;  // first key of this tile
                if (kbase + Cfg::kKeys - 1 > q0 + p.kv_off) {
                    // tile touches the diagonal: key kbase + c is visible to query q0 + row iff it is <= the query's
                    // own position kv_off + q0 + row
                    const int lim = p.kv_off + q0 + row - kbase;  // columns c <= lim are visible
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
                B200ATTN_STAMP(tid == 0, 16 + 8 * g + 1);
                if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
                    // O must hold P V of the previous tile before it is rescaled.  (At most one phase of
                    // this barrier is outstanding here: P V of this tile cannot start before this
                    // warp has arrived on bar_p_full below.)
                    ok = mbar_wait_warp(bar_pv_done, uint32_t(g - 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_MMA);
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
                mbar_arrive(&bar_p_full[g % NSB]);
                B200ATTN_STAMP(tid == 0, 16 + 8 * g + 2);
                if (j == 0 && pending) {
                    ok = epilogue(n - 1, pend_id, pend_m, pend_l);
                    pending = false;
                    if (!ok) break;
                }
            }
            if (!ok) break;
            pending = true;
            pend_id = id, pend_m = m_ref, pend_l = l;
        }
        if (ok && pending) epilogue(n - 1, pend_id, pend_m, pend_l);
        tc_fence_before_sync();
    }

    // teardown: every role falls through to here, also after a wait that gave up
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 5) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, Cfg::kTmemCols);
    }
    B200ATTN_TRACE_END(0);
}

}  // namespace b200attn
