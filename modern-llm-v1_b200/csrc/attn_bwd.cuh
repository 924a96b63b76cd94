// Causal grouped-query attention backward for sm_100a, the three steps of the
// reference's flash_attn_backward (llm/src/model/flash_attn.cu:428-504, math :137-146):
//   1. preprocess  D[i] = sum_d O[i,d] dO[i,d]            (flash_attn_compute_D_kernel, :150-172)
//                  - done by the dQ pass for its own rows, no separate kernel
//   2. dQ pass     query tile stationary, walks key tiles  (flash_attn_dq_kernel, :175-274)
//   3. dK/dV pass  key tile stationary, walks query tiles  (flash_attn_dkdv_kernel, :277-379)
// with  P = exp(s - L),  dP = dO V^T,  dS = P (dP - D),  dQ = scale dS K,
//       dK = scale dS^T Q,  dV = P^T dO.
// Both passes recompute P from the saved logsumexp on the tensor cores; neither uses
// atomics, so results are bit-reproducible.  GQA: the dK/dV CTA of a KV head loops over
// the query heads of its group and keeps one accumulator, which replaces
// accumulate_kv_grads (llm/src/model/attention.cu:412-429,510-543).
//
// Roles in the dK/dV pass (576 threads; the dQ pass is described at its kernel):
//   warps 0-15  compute: thread owns TMEM lane (warp % 4) * 32 + lane and the 32 score
//               columns of its part (warp / 4); four warps per scheduler hide the TMEM and
//               MUFU latencies of one another
//   warp  16    TMA producer (converged warp, one elected lane issues)
//   warp  17    TMEM allocation and tcgen05.mma issue (converged warp, one elected lane issues)
// TMEM (512 columns), D = 64:  S buffer 0 [0,128), S buffer 1 [128,256), dP [256,384),
//   accumulators [384,448) and [448,512).  With two S buffers the next tile's QK^T product
//   is issued while the compute warps still work on the current tile.
//   D = 128: one S buffer [0,128), dP [128,256), accumulators [256,384) and [384,512).
// The compute step has two phases so that it can start on S before dP has arrived:
//   A: P = exp2(S * scale*log2e - L*log2e)   (kept in registers; the dK/dV pass also stores it)
//   B: dS = P * (dP - D)                      (stored over dP as BF16)
// The BF16 operands of the second-stage MMAs overwrite the FP32 values they were computed
// from: part q of a 128-wide block keeps its 32 BF16 values in the first 16 columns of its
// own 32-column range.
#pragma once

#include "ptx.cuh"

namespace b200attn {

struct BwdParams {
    int B, T, Tpad, Hq, Hkv, group, n_tiles;
    float scale, scale_log2;
    const float* lse2;  // [B, Hq, Tpad]  logsumexp * log2(e); +inf in the padding rows   (read by the dK/dV pass)
    const float* dvec;  // [B, Hq, Tpad]  rowsum(O * dO);       0 in the padding rows     (read by the dK/dV pass)
    float* lse2_w;      // the same two vectors, written by the dQ pass
    float* dvec_w;
    const float* lse;       // [B, Hq, T]
    const uint16_t* o;      // forward output, q layout
    const uint16_t* dout;   // upstream gradient, q layout
    uint16_t* dq;           // q layout
    long long q_st, q_sh, q_sb;  // element strides of the q layout: token, head, batch
    int* status;
    uint16_t* dk;           // k layout
    uint16_t* dv;           // k layout
    long long k_st, k_sh, k_sb;  // element strides of the k layout: token, head, batch
    int* sched;   // two words of the device-wide item counter of the persistent dQ pass (see ptx.cuh), or nullptr
    int* sched2;  // the same for the dK/dV pass
    FastDiv div_bhq, div_hq, div_bhkv, div_hkv, div_group;  // division by B * Hq, Hq, B * Hkv, Hkv and the group size
};

template <int D>
struct BwdCfg {
    static constexpr bool kDoubleS = (D == 64);
    static constexpr int kStages = kDoubleS ? 3 : 2;  // streamed operand pairs in shared memory
    static constexpr int kTileBytes = 128 * D * 2;
    static constexpr int kBoxBytes = 128 * 64 * 2;
    static constexpr int kBoxes = D / 64;
    static constexpr int kVecBytes = kStages * 2 * 512;  // per stage (lse2, dvec) of 128 rows
    static constexpr int kBarBytes = 512;
    static constexpr int kKvBufs = kDoubleS ? 2 : 1;       // K/V tile pairs in shared memory (the next item's are prefetched)
    static constexpr int kOutTiles = kDoubleS ? 2 : 0;     // staging tiles for dV, dK (D = 128 has no room: direct stores)
    static constexpr int kParts = 4;                       // compute warpgroups: each owns 128 / kParts score columns
    static constexpr int kPartCols = 128 / kParts;         // 32
    static constexpr int kComputeThreads = 128 * kParts;   // 512
    static constexpr int kThreads = kComputeThreads + 64;  // + producer warp + MMA warp
    static constexpr int kSmemBytes = (2 * kKvBufs + 2 * kStages + kOutTiles) * kTileBytes + kVecBytes + kBarBytes + 1024;
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
// rows 0..15).  The A operand lives in kParts pieces: part q keeps its kPartCols BF16 values in
// the first kPartCols / 2 columns of its own FP32 column range, which starts at a_col + q * kPartCols.
template <int D>
__device__ __forceinline__ void issue_ts_over_rows(uint32_t d_tmem, uint32_t a_col, uint64_t b_desc, uint32_t idesc,
                                                   bool accumulate) {
    constexpr int kStepsPerPart = BwdCfg<D>::kPartCols / 16;  // K steps (16 rows of B) per part
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
        const uint32_t a = a_col + (ks / kStepsPerPart) * BwdCfg<D>::kPartCols + (ks % kStepsPerPart) * 8;
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
// dQ pass (D = 64): persistent CTAs, two per SM.  A CTA walks a list of work items (item = one 128-row query tile
// of one (batch, query head); items are ordered heaviest first), and every pipeline keeps running across item
// boundaries.  The O tile travels with Q and dO, so the preprocess D = rowsum(O * dO)
// (flash_attn_compute_D_kernel, llm/src/model/flash_attn.cu:150-172) is shared-memory work at the head of each
// item; D and L * log2(e) are also left in the workspace for the dK/dV pass, which therefore has to run after this
// kernel.
//
// Q and dO in tensor memory.  Every D = 64 kernel here is bound by the shared-memory data path (a product M128 N64
// K16 with both operands in shared memory fetches 4 KB of A and 2 KB of B for 32 clocks of math), and Q and dO are
// the A operands of every S = Q K^T and dP = dO V^T product of an item.  The compute warps therefore copy the two
// tiles once per item from shared memory into tensor memory (the 128 bytes of row r are the 32 BF16-pair columns
// of lane r as they stand), all three products of a key tile take their A operand from tensor memory, and the
// shared-memory tiles are free for the NEXT item's loads while this item is still being worked on.
//
// Roles (320 threads): warps 0-7 compute (thread owns query row (warp % 4) * 32 + lane == TMEM lane and the 32 key
// columns of its part warp / 4), warp 8 TMA producer, warp 9 TMEM allocation + MMA issue (converged warps, one
// elected lane issues).
// TMEM (256 columns): S [0,64), dP [64,128) (dS as BF16 over the first 16 columns of each part's range), dQ
// accumulator [128,192), Q [192,224), dO [224,256).  There is one S buffer: the compute warps read a tile's scores
// into registers in one go and hand the buffer back at once, so the next tile's Q K^T runs under this tile's
// exponentials; dS overwrites dP, so the next dP product follows the dQ product that consumes it.
// ---------------------------------------------------------------------------------------
template <int D>
struct DqCfg {
    static constexpr int kKeys = 64;
    static constexpr int kStages = 3;
    static constexpr int kQTileBytes = 128 * D * 2;
    static constexpr int kQBoxBytes = 128 * 64 * 2;
    static constexpr int kKVTileBytes = kKeys * D * 2;
    static constexpr int kKVBoxBytes = kKeys * 64 * 2;
    static constexpr int kBoxes = D / 64;
    static constexpr int kSmemBytes = 3 * kQTileBytes + 2 * kStages * kKVTileBytes + 512 + 1024;  // Q, dO, O + ring + barriers
    static constexpr int kTmemCols = 256;
    static constexpr int kCtasPerSm = 2;
    static constexpr int kColS = 0, kColDP = 64, kColAcc = 128, kColQ = 192, kColDO = 224;
    static constexpr int kParts = 2;
    static constexpr int kPartCols = kKeys / kParts;  // 32
    static constexpr int kComputeThreads = 128 * kParts;
    static constexpr int kThreads = kComputeThreads + 64;
    static constexpr int kProducerWarp = 4 * kParts, kMmaWarp = 4 * kParts + 1;
};

template <int D>
__global__ void __launch_bounds__(DqCfg<D>::kThreads, DqCfg<D>::kCtasPerSm)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                   const __grid_constant__ CUtensorMap tmO, const BwdParams p, const __grid_constant__ ItemTable tab) {
    static_assert(D == 64, "the persistent dQ pass keeps Q and dO in 64 tensor-memory columns: D = 64 only");
    using Cfg = DqCfg<D>;
    constexpr int NST = Cfg::kStages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;
    uint8_t* sdO = sQ + Cfg::kQTileBytes;
    uint8_t* sO = sdO + Cfg::kQTileBytes;
    uint8_t* sK = sO + Cfg::kQTileBytes;         // [NST]
    uint8_t* sV = sK + NST * Cfg::kKVTileBytes;  // [NST]
    uint64_t* bars = reinterpret_cast<uint64_t*>(sV + NST * Cfg::kKVTileBytes);
    uint64_t* bar_q = bars + 0;         // Q, dO, O of an item have landed in shared memory      (phase: item)
    uint64_t* bar_qs_free = bars + 1;   // the compute warps have read those three tiles          (phase: item)
    uint64_t* bar_qt_full = bars + 2;   // Q and dO of an item are in tensor memory               (phase: item)
    uint64_t* bar_s_full = bars + 3;    //                                                         (phase: tile)
    uint64_t* bar_s_loaded = bars + 4;  // S is in registers: the buffer may be overwritten       (phase: tile)
    uint64_t* bar_dp_full = bars + 5;   //                                                         (phase: tile)
    uint64_t* bar_ds_full = bars + 6;   // dS written over dP                                      (phase: tile)
    uint64_t* bar_acc = bars + 8;       // dQ accumulator of an item complete                      (phase: item)
    uint64_t* bar_acc_free = bars + 9;  // dQ accumulator read by the epilogue                     (phase: item)
    uint64_t* bar_kv_full = bars + 14;        // [NST]
    uint64_t* bar_kv_free = bars + 14 + NST;  // [NST]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14 + 2 * NST);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 15 + 2 * NST);
    uint64_t* bar_item = bars + 24;     // [kItemRing] item ids handed out by the producer
    volatile int* item_ring = reinterpret_cast<volatile int*>(bars + 24 + kItemRing);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_bh = p.B * p.Hq;
    const int n_items = p.n_tiles * n_bh;
    // item id -> (query tile, head, batch); ids are ordered by work, heaviest query tile first
    auto item_rest = [&](int id) { return id - int(fastdiv(unsigned(id), p.div_bhq)) * n_bh; };  // b * Hq + h
    auto item_qt = [&](int id) { return p.n_tiles - 1 - int(fastdiv(unsigned(id), p.div_bhq)); };
    auto item_b = [&](int id) { return int(fastdiv(unsigned(item_rest(id)), p.div_hq)); };
    auto item_h = [&](int id) { return item_rest(id) - item_b(id) * p.Hq; };
    auto item_nkv = [&](int id) { return (min(p.T, item_qt(id) * 128 + 128) + Cfg::kKeys - 1) / Cfg::kKeys; };
    auto get_item = [&](int n) { return item_get(bar_item, item_ring, n, abort_flag, p.status); };

    B200ATTN_TRACE_BEGIN(1);
    if (warp == Cfg::kProducerWarp && lane == 0) {
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
        tma_prefetch_desc(&tmdO);
        tma_prefetch_desc(&tmO);
        mbar_init(bar_q, 1);
        mbar_init(bar_qs_free, Cfg::kComputeThreads);
        mbar_init(bar_qt_full, Cfg::kComputeThreads);
        mbar_init(bar_s_full, 1);
        mbar_init(bar_s_loaded, Cfg::kComputeThreads);
        mbar_init(bar_dp_full, 1);
        mbar_init(bar_ds_full, Cfg::kComputeThreads);
        mbar_init(bar_acc, 1);
        mbar_init(bar_acc_free, Cfg::kComputeThreads);
        for (int s = 0; s < NST; ++s) {
            mbar_init(&bar_kv_full[s], 1);
            mbar_init(&bar_kv_free[s], 1);
        }
        for (int i = 0; i < kItemRing; ++i) mbar_init(&bar_item[i], 1);
        fence_mbar_init();
        grid_dep_wait();  // first global access of this CTA comes next
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
        // ------------------------------------------------------------------ producer
        int g = 0;  // tiles issued so far by this CTA (ring position)
        bool ok = true;
        int id = sched_first(tab, p.sched, int(blockIdx.x));  // the first item needs no fetch
        int id_next = 0;      // lane 0: the id fetched for the next item
        if (lane == 0) {
            item_publish(bar_item, item_ring, 0, id);
            id_next = sched_fetch(tab, p.sched, 1, int(blockIdx.x), int(gridDim.x));
        }
        __syncwarp();
        for (int n = 0; ok; ++n) {
            const int qt = item_qt(id), h = item_h(id), b = item_b(id), hk = int(fastdiv(unsigned(h), p.div_group)), n_kv = item_nkv(id);
            // the next item is taken and announced shortly before this item's loads end, but not before the
            // ring has been filled for this item
            const int j_next = max(min(n_kv, NST) - 1, n_kv - 2);
            int id_new = n_items;
            // the three tiles in shared memory are free as soon as the previous item has been copied out of them
            if (n > 0) ok = mbar_wait_warp(bar_qs_free, (n - 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_FREE);
            if (!ok) break;
            if (elect_one()) {
                mbar_arrive_expect_tx(bar_q, 3 * Cfg::kQTileBytes);
                tma_load_4d(sQ, &tmQ, bar_q, 0, qt * 128, h, b);
                tma_load_4d(sdO, &tmdO, bar_q, 0, qt * 128, h, b);
                tma_load_4d(sO, &tmO, bar_q, 0, qt * 128, h, b);
            }
            __syncwarp();
            for (int j = 0; j < n_kv; ++j, ++g) {
                const int s = g % NST;
                if (g >= NST) ok = mbar_wait_warp(&bar_kv_free[s], ((g / NST) - 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_FREE);
                if (!ok) break;
                if (elect_one()) {
                    mbar_arrive_expect_tx(&bar_kv_full[s], 2 * Cfg::kKVTileBytes);
                    tma_load_4d(sK + s * Cfg::kKVTileBytes, &tmK, &bar_kv_full[s], 0, j * Cfg::kKeys, hk, b);
                    tma_load_4d(sV + s * Cfg::kKVTileBytes, &tmV, &bar_kv_full[s], 0, j * Cfg::kKeys, hk, b);
                }
                __syncwarp();
                if (j == j_next) {
                    id_new = __shfl_sync(0xffffffffu, id_next, 0);
                    if (lane == 0) {
                        item_publish(bar_item, item_ring, n + 1, id_new < n_items ? id_new : -1);
                        if (id_new < n_items) id_next = sched_fetch(tab, p.sched, n + 2, int(blockIdx.x), int(gridDim.x));
                    }
                    __syncwarp();
                }
            }
            if (!ok || id_new >= n_items) break;
            id = id_new;
        }
        if (ok && lane == 0) sched_finish(p.sched, int(gridDim.x));
    } else if (warp == Cfg::kMmaWarp) {
        // ------------------------------------------------------------------ MMA issuer
        constexpr uint32_t idesc_s = make_idesc_bf16(128, Cfg::kKeys, 0, 0);  // A in TMEM, B (K or V tile) K-major
        constexpr uint32_t idesc_acc = make_idesc_bf16(128, D, 0, 1);         // A in TMEM, B (K tile) MN-major
        // g numbers this CTA's key tiles across all its items: ring stage g % NST
        auto issue_s = [&](int g) -> bool {  // S(g) = Q K^T; the buffer still holds S(g - 1) until it has been read
            const int s = g % NST;
            if (g > 0 && !mbar_wait_warp(bar_s_loaded, uint32_t(g - 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_SOFTMAX))
                return false;
            if (!mbar_wait_warp(&bar_kv_full[s], (g / NST) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_LOAD)) return false;
            tc_fence_after_sync();
            const uint64_t k_desc = make_sdesc_sw128(smem_u32(sK + s * Cfg::kKVTileBytes), 16, 1024);
            if (elect_one()) {
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks)
                    umma_ts(tmem + Cfg::kColS, tmem + Cfg::kColQ + ks * 8, k_desc + kmajor_step(ks, Cfg::kKVBoxBytes), idesc_s, ks > 0);
                umma_commit(bar_s_full);
            }
            __syncwarp();
            return true;
        };
        // dP(g) = dO V^T; tile g's loads have landed (S(g) was issued), and the product that read dS(g - 1) out of
        // this block was issued before (the products execute in order)
        auto issue_dp = [&](int g) {
            const int s = g % NST;
            const uint64_t v_desc = make_sdesc_sw128(smem_u32(sV + s * Cfg::kKVTileBytes), 16, 1024);
            if (elect_one()) {
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks)
                    umma_ts(tmem + Cfg::kColDP, tmem + Cfg::kColDO + ks * 8, v_desc + kmajor_step(ks, Cfg::kKVBoxBytes), idesc_s, ks > 0);
                umma_commit(bar_dp_full);
            }
            __syncwarp();
        };
        int g0 = 0, n = 0;
        bool ok = true;
        for (int id; ok && (id = get_item(n)) >= 0; ++n) {
            const int n_kv = item_nkv(id);
            B200ATTN_STAMP(lane == 0, 440 + 2 * n);
            ok = mbar_wait_warp(bar_qt_full, n & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_LOAD);
            B200ATTN_STAMP(lane == 0, 441 + 2 * n);
            if (ok) ok = issue_s(g0);
            if (!ok) break;
            issue_dp(g0);
            for (int j = 0; j < n_kv && ok; ++j) {
                const int g = g0 + j;
                const int s = g % NST;
                if (j + 1 < n_kv) {
                    ok = issue_s(g + 1);  // as soon as S(g) is in registers
                    if (!ok) break;
                }
                ok = mbar_wait_warp(bar_ds_full, uint32_t(g) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_SOFTMAX);
                if (!ok) break;
                B200ATTN_STAMP(lane == 0, 240 + 8 * g + 5);
                // the accumulator still belongs to the previous item's epilogue until it has been read
                if (j == 0 && n > 0) {
                    ok = mbar_wait_warp(bar_acc_free, (n - 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_SOFTMAX);
                    if (!ok) break;
                }
                tc_fence_after_sync();
                const uint64_t kmn_desc = make_sdesc_sw128(smem_u32(sK + s * Cfg::kKVTileBytes), Cfg::kKVBoxBytes, 1024);
                if (elect_one()) {
                    // dQ += dS K : 64 keys = 4 K steps; part q keeps its BF16 dS in the first 16 columns of its range
#pragma unroll
                    for (int ks = 0; ks < Cfg::kKeys / 16; ++ks) {
                        constexpr int kStepsPerPart = Cfg::kPartCols / 16;
                        const uint32_t a_col = Cfg::kColDP + (ks / kStepsPerPart) * Cfg::kPartCols + (ks % kStepsPerPart) * 8;
                        umma_ts(tmem + Cfg::kColAcc, tmem + a_col, kmn_desc + uint64_t(ks * 128), idesc_acc, (j > 0) || (ks > 0));
                    }
                    umma_commit(&bar_kv_free[s]);
                    if (j + 1 == n_kv) umma_commit(bar_acc);
                }
                __syncwarp();
                B200ATTN_STAMP(lane == 0, 240 + 8 * g + 6);
                if (j + 1 < n_kv) issue_dp(g + 1);
            }
            g0 += n_kv;
        }
        // drain: nothing may be in flight when TMEM is freed
        if (ok && n > 0) mbar_wait_warp(bar_acc, (n - 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_MMA);
    } else {
        // ------------------------------------------------------------------ compute
        const int w4 = warp & 3, part = warp >> 2;
        const int row = w4 * 32 + lane;  // query row in the tile == TMEM lane
        const uint32_t lane_base = uint32_t(w4 * 32) << 16;
        const int c0 = part * Cfg::kPartCols;  // first key column of this thread's part
        bool ok = true;
        float dv = 0.f, lse2 = INFINITY;  // of the item whose Q and dO are in tensor memory
        // Head of this CTA's n-th item: the preprocess of this row from the tiles in shared memory
        // (D = rowsum(O * dO); L * log2(e)), and Q (part 0) / dO (part 1) into tensor memory.  All S and dP products
        // of the previous item have completed when this runs (their results were waited for).
        auto item_head = [&](int n_item, int id) -> bool {
            const int q0 = item_qt(id) * 128, h = item_h(id), b = item_b(id);
            const bool in_range = q0 + row < p.T;
            // (issued here and first used after the wait below, so that its latency overlaps the wait)
            const float lse_raw = in_range ? p.lse[(size_t(b) * p.Hq + h) * p.T + q0 + row] : 0.f;
            B200ATTN_STAMP(tid == 0, 400 + 4 * n_item + 0);
            if (!mbar_wait_warp(bar_q, n_item & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_LOAD)) return false;
            B200ATTN_STAMP(tid == 0, 400 + 4 * n_item + 1);
            tc_fence_after_sync();
            float acc = 0.f;
            uint32_t tw[32];  // this row of Q (part 0) or dO (part 1) as it goes into tensor memory
#pragma unroll
            for (int c = 0; c < D / 8; ++c) {
                const uint32_t off = row * 128 + ((c ^ (row & 7)) << 4);
                const uint4 a = *reinterpret_cast<const uint4*>(sO + off);
                const uint4 gq = *reinterpret_cast<const uint4*>(sdO + off);
                const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
                const uint32_t gw[4] = {gq.x, gq.y, gq.z, gq.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    acc = fmaf(__uint_as_float(aw[e] << 16), __uint_as_float(gw[e] << 16), acc);
                    acc = fmaf(__uint_as_float(aw[e] & 0xffff0000u), __uint_as_float(gw[e] & 0xffff0000u), acc);
                }
                if (part == 0) {
                    const uint4 qv = *reinterpret_cast<const uint4*>(sQ + off);
                    tw[4 * c] = qv.x, tw[4 * c + 1] = qv.y, tw[4 * c + 2] = qv.z, tw[4 * c + 3] = qv.w;
                } else {
                    tw[4 * c] = gq.x, tw[4 * c + 1] = gq.y, tw[4 * c + 2] = gq.z, tw[4 * c + 3] = gq.w;
                }
            }
            // The tiles were read with ordinary loads and will be overwritten by TMA, which works through the async
            // proxy: without this fence the producer's next load, issued the moment the last thread has arrived, may
            // overtake reads that are still in flight (the producer is parked at the barrier whenever the item before
            // was short; dQ rows of whole warps, sometimes of single lanes, then came out wrong once in a few launches).
            fence_proxy_async_smem();
            mbar_arrive(bar_qs_free);  // the three tiles may be overwritten by the next item's loads
            tmem_st_x32(tmem + lane_base + (part == 0 ? Cfg::kColQ : Cfg::kColDO), tw);
            // exp2(x - inf) = 0: padding query rows contribute nothing
            lse2 = in_range ? lse_raw * 1.4426950408889634f : INFINITY;
            dv = in_range ? acc : 0.f;
            if (part == 0) {
                const size_t vrow = (size_t(b) * p.Hq + h) * p.Tpad + q0 + row;
                p.lse2_w[vrow] = lse2;
                p.dvec_w[vrow] = dv;
            }
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(bar_qt_full);
            return true;
        };
        int g0 = 0, n = 0;
        int id = get_item(0);
        if (id >= 0) ok = item_head(0, id);
        while (ok && id >= 0) {
            const int qt = item_qt(id), h = item_h(id), b = item_b(id), n_kv = item_nkv(id);
            const int q0 = qt * 128;
            for (int j = 0; j < n_kv; ++j) {
                const int g = g0 + j;
                ok = mbar_wait_warp(bar_s_full, uint32_t(g) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_MMA);
                if (!ok) break;
                B200ATTN_STAMP(tid == 0, 240 + 8 * g + 0);
                tc_fence_after_sync();
                // phase A: P from S (the scores leave tensor memory in one go)
                float pr[32];
                {
                    uint32_t sv[32];
                    tmem_ld_x32(tmem + lane_base + Cfg::kColS + c0, sv);
                    tmem_wait_ld();
                    tc_fence_before_sync();
                    mbar_arrive(bar_s_loaded);
#pragma unroll
                    for (int i = 0; i < 32; ++i) pr[i] = ex2_approx(fmaf(__uint_as_float(sv[i]), p.scale_log2, -lse2));
                }
                const int kbase = j * Cfg::kKeys;
                if (kbase + Cfg::kKeys - 1 > q0) {
                    const int lim = q0 + row - kbase - c0;  // columns i <= lim of this part are visible
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (i > lim) pr[i] = 0.f;
                }
                B200ATTN_STAMP(tid == 0, 240 + 8 * g + 1);
                ok = mbar_wait_warp(bar_dp_full, uint32_t(g) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_MMA);
                if (!ok) break;
                B200ATTN_STAMP(tid == 0, 240 + 8 * g + 2);
                tc_fence_after_sync();
                // phase B: dS = P (dP - D), written as BF16 over the part's first 16 columns of the dP block
                {
                    uint32_t dp[32], pk[16];
                    const uint32_t t_dp = tmem + lane_base + Cfg::kColDP + c0;
                    tmem_ld_x32(t_dp, dp);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        pk[i] = pack_bf16x2(pr[2 * i] * (__uint_as_float(dp[2 * i]) - dv),
                                            pr[2 * i + 1] * (__uint_as_float(dp[2 * i + 1]) - dv));
                    tmem_st_x16(t_dp, pk);
                }
                tmem_wait_st();
                tc_fence_before_sync();
                mbar_arrive(bar_ds_full);
                B200ATTN_STAMP(tid == 0, 240 + 8 * g + 3);
            }
            if (!ok) break;
            g0 += n_kv;
            // The next item's head before this item's epilogue: its first products then run while the dQ rows are
            // written.  (dv and lse2 change here; the epilogue below needs neither.)
            const int id_next = get_item(n + 1);
            if (id_next >= 0) {
                ok = item_head(n + 1, id_next);
                if (!ok) break;
            }
            // epilogue of the item: dQ rows (times scale) -> BF16 -> global memory; each part writes D / 2 columns
            ok = mbar_wait_warp(bar_acc, n & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_MMA);
            if (!ok) break;
            B200ATTN_STAMP(tid == 0, 400 + 4 * n + 2);
            tc_fence_after_sync();
            constexpr int kCols = D / Cfg::kParts;
            uint32_t v[kCols];
            tmem_ld_x32(tmem + lane_base + Cfg::kColAcc + part * kCols, v);
            tmem_wait_ld();
            tc_fence_before_sync();
            mbar_arrive(bar_acc_free);  // the MMA warp may start the next item's accumulation
            if (q0 + row < p.T) {
                uint16_t* dqrow = p.dq + size_t(b) * p.q_sb + size_t(h) * p.q_sh + size_t(q0 + row) * p.q_st + part * kCols;
#pragma unroll
                for (int gq = 0; gq < kCols / 8; ++gq) {
                    uint4 w;
                    w.x = pack_bf16x2(__uint_as_float(v[gq * 8 + 0]) * p.scale, __uint_as_float(v[gq * 8 + 1]) * p.scale);
                    w.y = pack_bf16x2(__uint_as_float(v[gq * 8 + 2]) * p.scale, __uint_as_float(v[gq * 8 + 3]) * p.scale);
                    w.z = pack_bf16x2(__uint_as_float(v[gq * 8 + 4]) * p.scale, __uint_as_float(v[gq * 8 + 5]) * p.scale);
                    w.w = pack_bf16x2(__uint_as_float(v[gq * 8 + 6]) * p.scale, __uint_as_float(v[gq * 8 + 7]) * p.scale);
                    *reinterpret_cast<uint4*>(dqrow + gq * 8) = w;
                }
            }
            B200ATTN_STAMP(tid == 0, 400 + 4 * n + 3);
            id = id_next;
            ++n;
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == Cfg::kMmaWarp) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, Cfg::kTmemCols);
    }
    B200ATTN_TRACE_END(1);
}

// ---------------------------------------------------------------------------------------
// dQ pass for D = 128: one CTA per item (128-row query tile of one (batch, query head)), 128-key tiles, eight
// compute warps (thread owns a row and 64 of the 128 score columns), one CTA per SM.  As in the D = 64 kernel, Q
// and dO are copied once from shared memory into tensor memory, so that S = Q K^T, dP = dO V^T and dQ += dS K all
// take their A operand from there (a 128-wide product with A in shared memory fetches 4 KB of A and 4 KB of B per
// K step), and the one S buffer is handed back as soon as the scores are in registers: the next tile's Q K^T runs
// under this tile's exponentials, and the next dP product follows the dQ product that consumes dS out of the dP
// block.
// Shared memory: the Q and dO staging tiles (64 KB; re-used as the third K/V ring stage once they have been copied
// into tensor memory, and at the very end as the staging tile of the dQ store) and two more K/V stages.
// TMEM (512 columns): S [0,128), dP [128,256) (dS as BF16 over the first 32 columns of each half's range), dQ
// accumulator [256,384), Q [384,448), dO [448,512).
// ---------------------------------------------------------------------------------------
template <int D>
struct DqWideCfg {
    static constexpr int kStages = 3;  // K/V tile pairs in flight; the third one lives where Q and dO were staged
    static constexpr int kTileBytes = 128 * D * 2;
    static constexpr int kBoxBytes = 128 * 64 * 2;
    static constexpr int kBoxes = D / 64;
    static constexpr int kSmemBytes = 2 * kStages * kTileBytes + 256 + 1024;
    static constexpr int kTmemCols = 512;
    static constexpr int kColS = 0, kColDP = 128, kColAcc = 256, kColQ = 384, kColDO = 448;
};

// D[tmem] = A[tmem, BF16 pairs] * B[smem, K-major]^T over the head dimension (b_desc describes K step 0)
template <int D>
__device__ __forceinline__ void wide_ts_headdim(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc) {
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) umma_ts(d_tmem, a_tmem + ks * 8, b_desc + kmajor_step(ks, 16384), idesc, ks > 0);
}
// A in two 32-column pieces at a_col and a_col + 64 (one per column half)
template <int D>
__device__ __forceinline__ void wide_ts(uint32_t d_tmem, uint32_t a_col, uint64_t b_desc, uint32_t idesc, bool accumulate) {
#pragma unroll
    for (int ks = 0; ks < 8; ++ks)
        umma_ts(d_tmem, a_col + (ks < 4 ? ks * 8 : 64 + (ks - 4) * 8), b_desc + uint64_t(ks * 128), idesc,
                accumulate || ks > 0);
}
template <int D>
__global__ void __launch_bounds__(320, 1)
attn_bwd_dq_wide_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                   const __grid_constant__ CUtensorMap tmdQ, const BwdParams p) {
    static_assert(D == 128, "Q and dO take 2 x 64 tensor-memory columns: D = 128 only");
    using Cfg = DqWideCfg<D>;
    constexpr int NST = Cfg::kStages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;
    uint8_t* sdO = sQ + Cfg::kTileBytes;
    uint8_t* sK01 = sdO + Cfg::kTileBytes;      // K of ring stages 0 and 1
    uint8_t* sV01 = sK01 + 2 * Cfg::kTileBytes; // V of ring stages 0 and 1
    // ring stage 2 re-uses the two tiles Q and dO were staged in (free once they are in tensor memory)
    auto stage_k = [&](int st) { return st < 2 ? sK01 + st * Cfg::kTileBytes : sQ; };
    auto stage_v = [&](int st) { return st < 2 ? sV01 + st * Cfg::kTileBytes : sdO; };
    uint64_t* bars = reinterpret_cast<uint64_t*>(sV01 + 2 * Cfg::kTileBytes);
    uint64_t* bar_q = bars + 0;         // Q and dO have landed in shared memory
    uint64_t* bar_qt_full = bars + 1;   // Q and dO are in tensor memory
    uint64_t* bar_s_full = bars + 2;    //                                                     (phase: tile)
    uint64_t* bar_s_loaded = bars + 3;  // S is in registers: the buffer may be overwritten   (phase: tile)
    uint64_t* bar_dp_full = bars + 4;   //                                                     (phase: tile)
    uint64_t* bar_ds_full = bars + 5;   // dS written over dP                                  (phase: tile)
    uint64_t* bar_acc = bars + 6;
    uint64_t* bar_kv_full = bars + 7;          // [NST]
    uint64_t* bar_kv_free = bars + 7 + NST;    // [NST]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 17);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_bh = p.B * p.Hq;
    const int qt = p.n_tiles - 1 - int(blockIdx.x) / n_bh;
    const int h = (int(blockIdx.x) % n_bh) % p.Hq, b = (int(blockIdx.x) % n_bh) / p.Hq;
    const int hk = h / p.group;
    const int q0 = qt * 128;
    const int n_kv = qt + 1;

    B200ATTN_TRACE_BEGIN(1);
    // launched with programmatic stream serialization: wait for the previous kernel before any global access
    grid_dep_launch();
    grid_dep_wait();
    if (tid == 0) *abort_flag = *reinterpret_cast<volatile int*>(p.status);
    __syncthreads();
    if (*abort_flag != 0) return;
    __syncthreads();

    if (tid == 0) {
        mbar_init(bar_q, 1);
        mbar_init(bar_qt_full, 256);
        mbar_init(bar_s_full, 1);
        mbar_init(bar_s_loaded, 256);
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
            // the first use of stage 2 overwrites Q and dO in shared memory: they must be in tensor memory by then
            if (j == 2 && !mbar_wait_warp(bar_qt_full, 0, abort_flag, p.status, DEV_WAIT_TIMEOUT_FREE)) break;
            if (elect_one()) {
                mbar_arrive_expect_tx(&bar_kv_full[s], 2 * Cfg::kTileBytes);
#pragma unroll
                for (int bx = 0; bx < Cfg::kBoxes; ++bx) {
                    tma_load_4d(stage_k(s) + bx * Cfg::kBoxBytes, &tmK, &bar_kv_full[s], bx * 64, j * 128, hk, b);
                    tma_load_4d(stage_v(s) + bx * Cfg::kBoxBytes, &tmV, &bar_kv_full[s], bx * 64, j * 128, hk, b);
                }
            }
            __syncwarp();
        }
    } else if (warp == 9) {
        // ------------------------------------------------------------------ MMA issuer (whole warp, one lane issues)
        constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);   // A in TMEM, B (K or V tile) K-major
        constexpr uint32_t idesc_acc = make_idesc_bf16(128, D, 0, 1);   // A in TMEM, B (K tile) MN-major
        bool ok = mbar_wait_warp(bar_qt_full, 0, abort_flag, p.status, DEV_WAIT_TIMEOUT_LOAD);
        // S(j) = Q K_j^T; the buffer still holds S(j - 1) until it has been read into registers
        auto issue_s = [&](int j) -> bool {
            const int s = j % NST;
            if (j > 0 && !mbar_wait_warp(bar_s_loaded, uint32_t(j - 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_SOFTMAX))
                return false;
            if (!mbar_wait_warp(&bar_kv_full[s], (j / NST) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_LOAD)) return false;
            tc_fence_after_sync();
            if (elect_one()) {
                wide_ts_headdim<D>(tmem + Cfg::kColS, tmem + Cfg::kColQ, kmajor_desc<D>(stage_k(s)), idesc_s);
                umma_commit(bar_s_full);
            }
            __syncwarp();
            return true;
        };
        // dP(j) = dO V_j^T; the tile's loads are known to be complete (S(j) was issued), and the product that read
        // dS(j - 1) out of this block was issued before
        auto issue_dp = [&](int j) {
            const int s = j % NST;
            if (elect_one()) {
                wide_ts_headdim<D>(tmem + Cfg::kColDP, tmem + Cfg::kColDO, kmajor_desc<D>(stage_v(s)), idesc_s);
                umma_commit(bar_dp_full);
            }
            __syncwarp();
        };
        if (ok) ok = issue_s(0);
        if (ok) issue_dp(0);
        for (int j = 0; j < n_kv && ok; ++j) {
            const int s = j % NST;
            if (j + 1 < n_kv) {
                ok = issue_s(j + 1);  // as soon as S(j) is in registers
                if (!ok) break;
            }
            ok = mbar_wait_warp(bar_ds_full, uint32_t(j) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_SOFTMAX);
            if (!ok) break;
            tc_fence_after_sync();
            if (elect_one()) {
                // dQ += dS K_j
                wide_ts<D>(tmem + Cfg::kColAcc, tmem + Cfg::kColDP, mnmajor_desc<D>(stage_k(s)), idesc_acc, j > 0);
                umma_commit(&bar_kv_free[s]);
            }
            __syncwarp();
            if (j + 1 < n_kv) issue_dp(j + 1);
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
        // preprocess for the warp's 32 rows (both halves compute it, half 0 stores it for the dK/dV pass)
        float lse2 = INFINITY, dv = 0.f;
        {
            constexpr int LPR = D / 8, RPP = 32 / LPR;
            const size_t tile_off = size_t(b) * p.q_sb + size_t(h) * p.q_sh;
#pragma unroll
            for (int i = 0; i < LPR; ++i) {
                const int r = q0 + w4 * 32 + i * RPP + lane / LPR;
                float acc = 0.f;
                if (r < p.T) {
                    const size_t off = tile_off + size_t(r) * p.q_st + (lane % LPR) * 8;
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
                const float v = __shfl_sync(0xffffffffu, acc, (lane % RPP) * LPR);
                if (lane / RPP == i) dv = v;
            }
            if (q0 + row < p.T) lse2 = p.lse[(size_t(b) * p.Hq + h) * p.T + q0 + row] * 1.4426950408889634f;
            if (half == 0) {
                p.lse2_w[vrow] = lse2;
                p.dvec_w[vrow] = dv;
            }
        }
        // this row of Q (half 0) or dO (half 1) from the swizzled tile in shared memory into tensor memory: the 256
        // bytes of the row are the 64 BF16-pair columns of lane `row` as they stand
        bool ok = mbar_wait_warp(bar_q, 0, abort_flag, p.status, DEV_WAIT_TIMEOUT_LOAD);
        if (ok) {
            const uint8_t* tile = half == 0 ? sQ : sdO;
#pragma unroll
            for (int bx = 0; bx < Cfg::kBoxes; ++bx) {
                uint32_t tw[32];
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const uint4 w = *reinterpret_cast<const uint4*>(tile + bx * Cfg::kBoxBytes + row * 128 + ((c ^ (row & 7)) << 4));
                    tw[4 * c] = w.x, tw[4 * c + 1] = w.y, tw[4 * c + 2] = w.z, tw[4 * c + 3] = w.w;
                }
                tmem_st_x32(tmem + lane_base + (half == 0 ? Cfg::kColQ : Cfg::kColDO) + bx * 32, tw);
            }
            tmem_wait_st();
            tc_fence_before_sync();
            // the producer re-uses the two tiles as a K/V stage once this barrier completes: the ordinary reads
            // above are ordered before the async proxy's (TMA) writes
            fence_proxy_async_smem();
            mbar_arrive(bar_qt_full);
        }
        for (int j = 0; j < n_kv && ok; ++j) {
            ok = mbar_wait_warp(bar_s_full, uint32_t(j) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_MMA);
            if (!ok) break;
            tc_fence_after_sync();
            // phase A: P from S (the scores leave tensor memory in one go)
            float pr[64];
            {
                uint32_t sv[64];
                tmem_ld_x32(tmem + lane_base + Cfg::kColS + c0, sv);
                tmem_ld_x32(tmem + lane_base + Cfg::kColS + c0 + 32, sv + 32);
                tmem_wait_ld();
                tc_fence_before_sync();
                mbar_arrive(bar_s_loaded);
#pragma unroll
                for (int i = 0; i < 64; ++i) pr[i] = ex2_approx(fmaf(__uint_as_float(sv[i]), p.scale_log2, -lse2));
            }
            if (j == qt) {
#pragma unroll
                for (int i = 0; i < 64; ++i)
                    if (c0 + i > row) pr[i] = 0.f;  // key above the diagonal
            }
            ok = mbar_wait_warp(bar_dp_full, uint32_t(j) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_MMA);
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
                tmem_ld_x32(tmem + lane_base + Cfg::kColAcc + col, v);
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
    B200ATTN_TRACE_END(1);
}


// ---------------------------------------------------------------------------------------
// dK/dV pass: persistent CTAs, one per SM.  An item is one 128-key tile of one (batch, KV head); its
// units are the (query head of the group, 128-query tile at or below the diagonal) pairs, each a
// 128 x 128 block of scores.  Items are ordered heaviest first (key tile 0 sees every query tile) and
// handed out as described in ptx.cuh.  All pipelines run across item boundaries: the next item's K and V
// tiles (second buffer, D = 64) and its first Q / dO tiles are loaded, and its first S^T and dP^T
// products issued, while the compute warps still drain the accumulators of the previous item.
// ---------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(BwdCfg<D>::kThreads, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                     const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
                     const __grid_constant__ CUtensorMap tmdK, const __grid_constant__ CUtensorMap tmdV,
                     const BwdParams p) {
    using Cfg = BwdCfg<D>;
    constexpr int NST = Cfg::kStages;
    constexpr int NKV = Cfg::kKvBufs;
    constexpr bool DBL = Cfg::kDoubleS;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sK = smem;                         // [NKV]
    uint8_t* sV = sK + NKV * Cfg::kTileBytes;   // [NKV]
    uint8_t* sQ = sV + NKV * Cfg::kTileBytes;   // [NST]
    uint8_t* sdO = sQ + NST * Cfg::kTileBytes;  // [NST]
    uint8_t* sOut = sdO + NST * Cfg::kTileBytes;  // [2] staging of dV and dK for the TMA store (D = 64 only)
    float* sLse = reinterpret_cast<float*>(sOut + Cfg::kOutTiles * Cfg::kTileBytes);  // [NST][128]
    float* sDv = sLse + NST * 128;                                         // [NST][128]
    uint64_t* bars = reinterpret_cast<uint64_t*>(sOut + Cfg::kOutTiles * Cfg::kTileBytes + Cfg::kVecBytes);
    uint64_t* bar_kv = bars + 0;        // [2] per K/V buffer: K, V of an item have landed      (phase: item / NKV)
    uint64_t* bar_kv_free = bars + 2;   // [2] per K/V buffer: every MMA reading them is done   (phase: item / NKV)
    uint64_t* bar_s_full = bars + 4;    // [2] per S buffer                                      (phase: unit / 2 or unit)
    uint64_t* bar_dp_full = bars + 6;   //                                                       (phase: unit)
    uint64_t* bar_dp_free = bars + 7;   // dP^T has been read into registers                     (phase: unit)
    uint64_t* bar_pds_full = bars + 8;  // [2] by unit parity: P^T and dS^T written              (phase: unit / 2)
    uint64_t* bar_acc = bars + 10;      // accumulators of an item complete                      (phase: item)
    uint64_t* bar_acc_free = bars + 11; // accumulators read by the epilogue                     (phase: item)
    uint64_t* bar_full = bars + 12;        // [NST] Q, dO and the two row vectors of a unit have landed
    uint64_t* bar_free = bars + 12 + NST;  // [NST]
    uint64_t* bar_s_loaded = bars + 22;  // one S buffer (D = 128): S^T is in registers, the buffer is free (phase: unit)
    uint64_t* bar_out_free = bars + 20;  // the TMA store of the previous item has read the staging tiles (phase: item)
    uint64_t* bar_out_full = bars + 21;  // every compute thread has staged its part of dV / dK        (phase: item)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 18);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 19);
    uint64_t* bar_item = bars + 24;     // [kItemRing] item ids handed out by the producer
    volatile int* item_ring = reinterpret_cast<volatile int*>(bars + 24 + kItemRing);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    constexpr int kProducerWarp = Cfg::kParts * 4, kMmaWarp = Cfg::kParts * 4 + 1;
    // item id -> (key tile, KV head, batch); ids are ordered by work: key tile 0 has the most query tiles below it
    const int n_bh = p.B * p.Hkv;
    const int n_items = p.n_tiles * n_bh;
    auto item_kt = [&](int id) { return int(fastdiv(unsigned(id), p.div_bhkv)); };
    auto item_rest = [&](int id) { return id - item_kt(id) * n_bh; };  // b * Hkv + hk
    auto item_b = [&](int id) { return int(fastdiv(unsigned(item_rest(id)), p.div_hkv)); };
    auto item_hk = [&](int id) { return item_rest(id) - item_b(id) * p.Hkv; };
    auto item_units = [&](int id) { return p.group * (p.n_tiles - item_kt(id)); };
    auto get_item = [&](int n) { return item_get(bar_item, item_ring, n, abort_flag, p.status); };

    B200ATTN_TRACE_BEGIN(2);
    if (warp == kProducerWarp && lane == 0) {
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmdO);
        tma_prefetch_desc(&tmdK);
        tma_prefetch_desc(&tmdV);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bar_kv[i], 1);
            mbar_init(&bar_kv_free[i], 1);
            mbar_init(&bar_s_full[i], 1);
            mbar_init(&bar_pds_full[i], Cfg::kComputeThreads);
        }
        mbar_init(bar_dp_full, 1);
        mbar_init(bar_dp_free, Cfg::kComputeThreads);
        mbar_init(bar_acc, 1);
        mbar_init(bar_acc_free, Cfg::kComputeThreads);
        mbar_init(bar_out_free, 1);
        mbar_init(bar_out_full, Cfg::kComputeThreads);
        mbar_init(bar_s_loaded, Cfg::kComputeThreads);
        for (int s = 0; s < NST; ++s) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_free[s], 1);
        }
        for (int i = 0; i < kItemRing; ++i) mbar_init(&bar_item[i], 1);
        fence_mbar_init();
        // Everything above touched no global memory.  From here on the previous kernel of the stream
        // (the dQ pass, which writes the two per-row vectors) must have completed.
        grid_dep_wait();
        *abort_flag = *reinterpret_cast<volatile int*>(p.status);
    }
    if (warp == kMmaWarp) {
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
    } else if (warp == kProducerWarp) {
        // ------------------------------------------------------------------ producer (whole warp, one lane issues)
        int u = 0;  // units issued so far by this CTA (ring position)
        bool ok = true;
        int id = blockIdx.x;  // the first item needs no fetch
        int id_next = 0;      // lane 0: the id fetched for the next item
        if (lane == 0) {
            item_publish(bar_item, item_ring, 0, id);
            id_next = sched_fetch(p.sched2, 1, int(blockIdx.x), int(gridDim.x));
        }
        __syncwarp();
        for (int n = 0; ok; ++n) {
            const int kt = item_kt(id), hk = item_hk(id), b = item_b(id), k0 = kt * 128;
            const int n_i = p.n_tiles - kt, n_it = p.group * n_i;
            const int kb = n % NKV;
            if (n >= NKV) ok = mbar_wait_warp(&bar_kv_free[kb], uint32_t(n / NKV - 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_FREE);
            if (!ok) break;
            if (elect_one()) {
                mbar_arrive_expect_tx(&bar_kv[kb], 2 * Cfg::kTileBytes);
#pragma unroll
                for (int bx = 0; bx < Cfg::kBoxes; ++bx) {
                    tma_load_4d(sK + kb * Cfg::kTileBytes + bx * Cfg::kBoxBytes, &tmK, &bar_kv[kb], bx * 64, k0, hk, b);
                    tma_load_4d(sV + kb * Cfg::kTileBytes + bx * Cfg::kBoxBytes, &tmV, &bar_kv[kb], bx * 64, k0, hk, b);
                }
            }
            __syncwarp();
            // the next item is taken and announced shortly before this item's loads end, but not before the
            // ring has been filled for this item
            const int j_next = max(min(n_it, NST) - 1, n_it - 2);
            int id_new = n_items;
            for (int it = 0, h = hk * p.group, i = kt; it < n_it; ++it, ++u, i = (i + 1 == p.n_tiles ? kt : i + 1), h += (i == kt)) {
                const int s = u % NST;
                if (u >= NST) ok = mbar_wait_warp(&bar_free[s], uint32_t(u / NST - 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_FREE);
                if (!ok) break;
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
    } else if (warp == kMmaWarp) {
        // ------------------------------------------------------------------ MMA issuer (whole warp, one lane issues)
        constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
        constexpr uint32_t idesc_acc = make_idesc_bf16(128, D, 0, 1);
        // This CTA's units are numbered u = 0, 1, ... across all its items: ring stage u % NST, S buffer u & 1
        // (two S buffers).  Three cursors walk that sequence: S^T = K Q^T runs two units ahead (one with a
        // single S buffer) and dP^T = V dO^T one unit ahead of the products into the accumulators.
        struct Cursor {
            int n, it, n_it, u;  // items before this one on this CTA, unit in item, units of item (0: list ended), unit number
        };
        bool ok = true;
        // `wait`: the first cursor to reach an item waits for its id; the others find it in the ring
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
        auto issue_s = [&](const Cursor& c) {  // S^T(u) = K Q^T
            const int s = c.u % NST, kb = c.n % NKV;
            // one S buffer: it still holds S^T of the unit before until the compute warps have read it into registers
            if (!DBL && c.u > 0) ok = mbar_wait_warp(bar_s_loaded, uint32_t(c.u - 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_SOFTMAX);
            if (ok && c.it == 0) ok = mbar_wait_warp(&bar_kv[kb], uint32_t(c.n / NKV) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_LOAD);
            if (ok) ok = mbar_wait_warp(&bar_full[s], uint32_t(c.u / NST) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_LOAD);
            if (!ok) return;
            tc_fence_after_sync();
            const int buf = DBL ? (c.u & 1) : 0;
            if (elect_one()) {
                issue_ss_over_headdim<D>(tmem + Cfg::col_s(buf), kmajor_desc<D>(sK + kb * Cfg::kTileBytes),
                                         kmajor_desc<D>(sQ + s * Cfg::kTileBytes), idesc_s);
                umma_commit(&bar_s_full[buf]);
            }
            __syncwarp();
        };
        // dP^T(u) = V dO^T; the loads of the unit are known to be complete (S^T of the unit was issued before).
        // After the item's last unit no MMA reads its K and V any more.
        auto issue_dp = [&](const Cursor& c) {
            const int s = c.u % NST, kb = c.n % NKV;
            if (elect_one()) {
                issue_ss_over_headdim<D>(tmem + Cfg::kColDP, kmajor_desc<D>(sV + kb * Cfg::kTileBytes),
                                         kmajor_desc<D>(sdO + s * Cfg::kTileBytes), idesc_s);
                umma_commit(bar_dp_full);
                if (c.it + 1 == c.n_it) umma_commit(&bar_kv_free[kb]);
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
            if (ok && DBL && cs.n_it > 0) {
                issue_s(cs);
                cursor_next(cs, true);
            }
        }
        int n_done = 0;  // items whose accumulators have been completed
        while (ok && ca.n_it > 0) {
            const int s = ca.u % NST;
            const int buf = DBL ? (ca.u & 1) : 0;
            // dP^T of the next unit as soon as the compute warps have read this one into registers
            // (dS^T is written next to P^T inside the S buffer, so the dP block is free): the MMA round trip
            // runs under their arithmetic.  (With a single S buffer, D = 128, the loads of the next unit
            // may still be in flight: there dP^T follows S^T below instead.)
            if (!DBL && cs.n_it > 0 && cs.it != 0) {
                // one S buffer (D = 128): S^T of the next unit as soon as this unit's scores are in registers, so that
                // it runs under this unit's exponentials.  (Not across an item boundary: the next item's K and V are
                // only loaded once this item's last dP^T product has run; that S^T follows the products below.)
                issue_s(cs);
                cursor_next(cs, true);
                if (!ok) break;
            }
            if (DBL && cd.n_it > 0) {
                ok = mbar_wait_warp(bar_dp_free, uint32_t(ca.u) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_SOFTMAX);
                if (!ok) break;
                tc_fence_after_sync();
                issue_dp(cd);
                cursor_next(cd, false);
            }
            ok = mbar_wait_warp(&bar_pds_full[ca.u & 1], uint32_t(ca.u >> 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_SOFTMAX);
            if (!ok) break;
            B200ATTN_STAMP(lane == 0, 16 + 8 * ca.u + 4);
            // the accumulators belong to the previous item's epilogue until it has read them
            if (ca.it == 0 && ca.n > 0) {
                ok = mbar_wait_warp(bar_acc_free, uint32_t(ca.n - 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_SOFTMAX);
                if (!ok) break;
            }
            tc_fence_after_sync();
            if (elect_one()) {
                // dV += P^T dO ; dK += dS^T Q   (P^T and dS^T sit side by side: in S buffer `buf`, or, with one S
                // buffer, over the dP block, which the compute warps have read by then)
                const uint32_t a_pds = tmem + (DBL ? Cfg::col_s(buf) : Cfg::kColDP);
                issue_ts_over_rows<D>(tmem + Cfg::kColAcc0, a_pds, mnmajor_desc<D>(sdO + s * Cfg::kTileBytes), idesc_acc, ca.it > 0);
                issue_ts_over_rows<D>(tmem + Cfg::kColAcc1, a_pds + Cfg::kPartCols / 2, mnmajor_desc<D>(sQ + s * Cfg::kTileBytes),
                                      idesc_acc, ca.it > 0);
                umma_commit(&bar_free[s]);
                if (ca.it + 1 == ca.n_it) umma_commit(bar_acc);
            }
            __syncwarp();
            B200ATTN_STAMP(lane == 0, 16 + 8 * ca.u + 5);
            if (ca.it + 1 == ca.n_it) ++n_done;
            if (!DBL && cs.n_it > 0 && cs.u == ca.u + 1) {  // S^T of the next unit is still to come (item boundary)
                issue_s(cs);
                cursor_next(cs, true);
                if (!ok) break;
            }
            if (!DBL && cd.n_it > 0) {
                // dP^T of the next unit overwrites P^T and dS^T of this one: behind the two products just issued
                issue_dp(cd);
                cursor_next(cd, false);
            }
            if (DBL && cs.n_it > 0) {
                issue_s(cs);
                cursor_next(cs, true);
            }
            B200ATTN_STAMP(lane == 0, 16 + 8 * ca.u + 6);
            cursor_next(ca, false);
        }
        // nothing may be in flight when TMEM is freed: the last commit covers every MMA issued above
        if (ok && n_done > 0) mbar_wait_warp(bar_acc, uint32_t(n_done - 1) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_MMA);
    } else {
        // ------------------------------------------------------------------ compute
        const int w4 = warp & 3, part = warp >> 2;
        const int row = w4 * 32 + lane;  // key row in the tile == TMEM lane
        const uint32_t lane_base = uint32_t(w4 * 32) << 16;
        const int c0 = part * Cfg::kPartCols;  // first query column of this thread's part
        bool ok = true;
        // Epilogue of an item.  It is deferred until the first unit of the next item has been handed to the MMA
        // warp, so that the wait for the item's last products overlaps that unit's arithmetic.
        auto epilogue = [&](int n_item, int id_item) -> bool {
            // epilogue of the item: parts 0,1 write dV, parts 2,3 write dK (times scale); each part takes D / 2
            // of the accumulator's columns of its key row, which is contiguous in global memory
            B200ATTN_STAMP(tid == 0, 460 + 4 * n_item + 0);
            ok = mbar_wait_warp(bar_acc, uint32_t(n_item) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_MMA);
            if (!ok) return false;
            B200ATTN_STAMP(tid == 0, 460 + 4 * n_item + 1);
            tc_fence_after_sync();
            // (the values below are derived from copies the compiler cannot see through, so that it does not
            // compute them ahead of the unit loop and keep them in registers there)
            int part_e = part, id_e = id_item;
            asm volatile("" : "+r"(part_e), "+r"(id_e));
            constexpr int kHalfParts = Cfg::kParts / 2;
            constexpr int kColsPerPart = D / kHalfParts;
            const bool is_dk = part_e >= kHalfParts;
            const uint32_t acc = is_dk ? Cfg::kColAcc1 : Cfg::kColAcc0;
            const float mul = is_dk ? p.scale : 1.f;
            const int col0 = (part_e % kHalfParts) * kColsPerPart;
            const int k0 = item_kt(id_e) * 128;
            if constexpr (Cfg::kOutTiles > 0) {
                // through shared memory and a TMA store, so that no compute thread waits on the memory system:
                // the previous item's store must have read the staging tiles before they are rewritten
                // (mbarriers with bounded waits rather than bar.sync: a warp that has given up never arrives)
                if (tid == 0) {
                    tma_store_wait_read0();
                    mbar_arrive(bar_out_free);
                }
                ok = mbar_wait_warp(bar_out_free, uint32_t(n_item) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_FREE);
                if (!ok) return false;
#pragma unroll
                for (int c = 0; c < kColsPerPart / 32; ++c) {
                    uint32_t v[32];
                    tmem_ld_x32(tmem + lane_base + acc + col0 + c * 32, v);
                    tmem_wait_ld();
                    if (c + 1 == kColsPerPart / 32) {
                        tc_fence_before_sync();
                        mbar_arrive(bar_acc_free);  // the MMA warp may start the next item's accumulation
                    }
                    stage_row_chunk<D>(sOut + (is_dk ? Cfg::kTileBytes : 0), row, col0 + c * 32, v, mul);
                }
                fence_proxy_async_smem();
                mbar_arrive(bar_out_full);
                if (warp == 0) {
                    ok = mbar_wait_warp(bar_out_full, uint32_t(n_item) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_FREE);
                    if (!ok) return false;
                }
                if (tid == 0) {
#pragma unroll
                    for (int bx = 0; bx < Cfg::kBoxes; ++bx) {
                        tma_store_4d(&tmdV, sOut + bx * Cfg::kBoxBytes, bx * 64, k0, item_hk(id_e), item_b(id_e));
                        tma_store_4d(&tmdK, sOut + Cfg::kTileBytes + bx * Cfg::kBoxBytes, bx * 64, k0, item_hk(id_e), item_b(id_e));
                    }
                    tma_store_commit();
                }
            } else {
                const bool in_range = k0 + row < p.T;
                uint16_t* out = (is_dk ? p.dk : p.dv) + size_t(item_b(id_e)) * p.k_sb + size_t(item_hk(id_e)) * p.k_sh +
                                size_t(k0 + row) * p.k_st + col0;
#pragma unroll
                for (int c = 0; c < kColsPerPart / 32; ++c) {
                    uint32_t v[32];
                    tmem_ld_x32(tmem + lane_base + acc + col0 + c * 32, v);
                    tmem_wait_ld();
                    if (c + 1 == kColsPerPart / 32) {
                        tc_fence_before_sync();
                        mbar_arrive(bar_acc_free);  // the MMA warp may start the next item's accumulation
                    }
                    if (in_range) {
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            uint4 w;
                            w.x = pack_bf16x2(__uint_as_float(v[g * 8 + 0]) * mul, __uint_as_float(v[g * 8 + 1]) * mul);
                            w.y = pack_bf16x2(__uint_as_float(v[g * 8 + 2]) * mul, __uint_as_float(v[g * 8 + 3]) * mul);
                            w.z = pack_bf16x2(__uint_as_float(v[g * 8 + 4]) * mul, __uint_as_float(v[g * 8 + 5]) * mul);
                            w.w = pack_bf16x2(__uint_as_float(v[g * 8 + 6]) * mul, __uint_as_float(v[g * 8 + 7]) * mul);
                            *reinterpret_cast<uint4*>(out + c * 32 + g * 8) = w;
                        }
                    }
                }
            }
            B200ATTN_STAMP(tid == 0, 460 + 4 * n_item + 2);
            return true;
        };
        bool pending = false;
        int pend_id = 0;
        int u = 0, n = 0;
        for (int id; ok && (id = get_item(n)) >= 0; ++n) {
            const int n_i = p.n_tiles - item_kt(id);
            // units of the item: for each query head of the group, the query tiles from the diagonal down
            for (int it = p.group * n_i, i_in = 0; it > 0; --it, ++u, i_in = (i_in + 1 == n_i ? 0 : i_in + 1)) {
                const int s = u % NST;
                const int buf = DBL ? (u & 1) : 0;
                const uint32_t s_par = DBL ? ((u >> 1) & 1) : (u & 1);
                const bool diag = i_in == 0;
                ok = mbar_wait_warp(&bar_s_full[buf], s_par, abort_flag, p.status, DEV_WAIT_TIMEOUT_MMA);
                if (!ok) break;
                B200ATTN_STAMP(tid == 0, 16 + 8 * u + 0);
                tc_fence_after_sync();
                const float4* lse4 = reinterpret_cast<const float4*>(sLse + s * 128 + c0);
                const float4* dv4 = reinterpret_cast<const float4*>(sDv + s * 128 + c0);
                float pr[32];
                if constexpr (DBL) {
                // phase A: P^T from S^T (kept in registers and stored over S^T as BF16), 16 columns at a time
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    uint32_t sv[16], pk[8];
                    tmem_ld_x16(tmem + lane_base + Cfg::col_s(buf) + c0 + hh * 16, sv);
                    tmem_wait_ld();
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        const float4 l4 = lse4[hh * 4 + g];
                        float* q = &pr[hh * 16 + g * 4];
                        q[0] = ex2_approx(fmaf(__uint_as_float(sv[g * 4 + 0]), p.scale_log2, -l4.x));
                        q[1] = ex2_approx(fmaf(__uint_as_float(sv[g * 4 + 1]), p.scale_log2, -l4.y));
                        q[2] = ex2_approx(fmaf(__uint_as_float(sv[g * 4 + 2]), p.scale_log2, -l4.z));
                        q[3] = ex2_approx(fmaf(__uint_as_float(sv[g * 4 + 3]), p.scale_log2, -l4.w));
                    }
                    if (diag) {
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            if (c0 + hh * 16 + i < row) pr[hh * 16 + i] = 0.f;  // query above the key: masked
                    }
#pragma unroll
                    for (int i = 0; i < 8; ++i) pk[i] = pack_bf16x2(pr[hh * 16 + 2 * i], pr[hh * 16 + 2 * i + 1]);
                    tmem_st_x8(tmem + lane_base + Cfg::col_s(buf) + c0 + hh * 8, pk);
                }
                } else {
                // phase A with one S buffer: the scores leave tensor memory in one go and the buffer goes back to the
                // MMA warp at once; P^T stays in registers until phase B
                {
                    uint32_t sv[32];
                    tmem_ld_x16(tmem + lane_base + Cfg::kColS0 + c0, sv);
                    tmem_ld_x16(tmem + lane_base + Cfg::kColS0 + c0 + 16, sv + 16);
                    tmem_wait_ld();
                    tc_fence_before_sync();
                    mbar_arrive(bar_s_loaded);
#pragma unroll
                    for (int g = 0; g < 8; ++g) {
                        const float4 l4 = lse4[g];
                        float* q = &pr[g * 4];
                        q[0] = ex2_approx(fmaf(__uint_as_float(sv[g * 4 + 0]), p.scale_log2, -l4.x));
                        q[1] = ex2_approx(fmaf(__uint_as_float(sv[g * 4 + 1]), p.scale_log2, -l4.y));
                        q[2] = ex2_approx(fmaf(__uint_as_float(sv[g * 4 + 2]), p.scale_log2, -l4.z));
                        q[3] = ex2_approx(fmaf(__uint_as_float(sv[g * 4 + 3]), p.scale_log2, -l4.w));
                    }
                }
                if (diag) {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (c0 + i < row) pr[i] = 0.f;  // query above the key: masked
                }
                }
                B200ATTN_STAMP(tid == 0, 16 + 8 * u + 1);
                ok = mbar_wait_warp(bar_dp_full, uint32_t(u) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_MMA);
                if (!ok) break;
                B200ATTN_STAMP(tid == 0, 16 + 8 * u + 2);
                tc_fence_after_sync();
                if constexpr (DBL) {
                // phase B: dS^T = P^T (dP^T - D), stored as BF16 next to P^T in the S buffer
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    uint32_t dp[16], pk[8];
                    tmem_ld_x16(tmem + lane_base + Cfg::kColDP + c0 + hh * 16, dp);
                    tmem_wait_ld();
                    if (hh == 1) {
                        tc_fence_before_sync();
                        mbar_arrive(bar_dp_free);  // dP^T is in registers: the next product may overwrite the block
                    }
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        const float4 d4 = dv4[hh * 4 + g];
                        const float* q = &pr[hh * 16 + g * 4];
                        pk[g * 2 + 0] = pack_bf16x2(q[0] * (__uint_as_float(dp[g * 4 + 0]) - d4.x),
                                                    q[1] * (__uint_as_float(dp[g * 4 + 1]) - d4.y));
                        pk[g * 2 + 1] = pack_bf16x2(q[2] * (__uint_as_float(dp[g * 4 + 2]) - d4.z),
                                                    q[3] * (__uint_as_float(dp[g * 4 + 3]) - d4.w));
                    }
                    tmem_st_x8(tmem + lane_base + Cfg::col_s(buf) + c0 + Cfg::kPartCols / 2 + hh * 8, pk);
                }
                } else {
                // phase B with one S buffer: all of this thread's dP^T into registers, then P^T and dS^T as BF16 side by
                // side over the part's own 32 columns of the dP block (P^T in the first 16, dS^T in the second 16)
                {
                    uint32_t dp[32], pp[16], pd[16];
                    const uint32_t t_dp = tmem + lane_base + Cfg::kColDP + c0;
                    tmem_ld_x16(t_dp, dp);
                    tmem_ld_x16(t_dp + 16, dp + 16);
                    tmem_wait_ld();
#pragma unroll
                    for (int g = 0; g < 8; ++g) {
                        const float4 d4 = dv4[g];
                        const float* q = &pr[g * 4];
                        pp[g * 2 + 0] = pack_bf16x2(q[0], q[1]);
                        pp[g * 2 + 1] = pack_bf16x2(q[2], q[3]);
                        pd[g * 2 + 0] = pack_bf16x2(q[0] * (__uint_as_float(dp[g * 4 + 0]) - d4.x),
                                                    q[1] * (__uint_as_float(dp[g * 4 + 1]) - d4.y));
                        pd[g * 2 + 1] = pack_bf16x2(q[2] * (__uint_as_float(dp[g * 4 + 2]) - d4.z),
                                                    q[3] * (__uint_as_float(dp[g * 4 + 3]) - d4.w));
                    }
                    tmem_st_x16(t_dp, pp);
                    tmem_st_x16(t_dp + 16, pd);
                }
                }
                tmem_wait_st();
                tc_fence_before_sync();
                // the unit's two row vectors were read from shared memory with ordinary loads; the stage goes back
                // to TMA (async proxy) through the products this arrival lets go
                fence_proxy_async_smem();
                mbar_arrive(&bar_pds_full[u & 1]);
                B200ATTN_STAMP(tid == 0, 16 + 8 * u + 3);
                if (pending) {  // first unit of this item: now the previous item's epilogue
                    pending = false;
                    ok = epilogue(n - 1, pend_id);
                    if (!ok) break;
                }
            }
            if (!ok) break;
            pending = true;
            pend_id = id;
        }
        if (ok && pending) epilogue(n - 1, pend_id);
        // the staging tiles must outlive the last store's reads
        if (Cfg::kOutTiles > 0 && tid == 0) tma_store_wait_read0();
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == kMmaWarp) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, Cfg::kTmemCols);
    }
    B200ATTN_TRACE_END(2);
}

}  // namespace b200attn
