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
// Roles (160 threads): warps 0-3 compute with warp-level BF16 MMAs (m16n8k16: the 16 rows are
// the query heads of the group), each warp on its own 32 keys of a tile; warp 4 = TMA producer.
// Each split writes an un-normalised partial (m, l, O); a small combine kernel merges them.
#pragma once

#include "ptx.cuh"

namespace b200attn {

struct DecodeParams {
    int B, L, Hq, Hkv, group;
    int G;         // query heads served per CTA (a divisor of group, <= 16)
    int n_chunks;  // group / G
    int n_splits;
    int tiles_per_split;
    float scale, scale_log2;
    const int* lens;    // [B] cache length per sequence (1 <= lens[b]; clamped to L), or nullptr: every sequence has L
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
    static constexpr int kMaxG = 16;                    // query heads per CTA = rows of the m16n8k16 MMA
    static constexpr int kQBytes = 16 * D * 2;          // q rows as BF16, zero padded to 16 rows, swizzled
    // the end-of-kernel merge scratch (per warp 16 rows x (O row, m, l) as FP32) re-uses the K ring
    static constexpr int kSmemBytes = 2 * kStages * kTileBytes + kQBytes + 256 + 1024;
};

// ---- warp-level tensor-core pieces (mma.sync is enough here: the kernel is bound by HBM, and the
// ---- 16-row MMA shape matches "all query heads of a KV group against one key tile")
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// Byte offset of the 16-byte chunk `chunk` (8 BF16 of the head dimension) of row `r` inside a tile of
// [rows][64]-boxes written by TMA with the 128-byte swizzle.
__device__ __forceinline__ uint32_t swz_off(int r, int chunk, int box_bytes) {
    return uint32_t((chunk >> 3) * box_bytes + r * 128 + (((chunk & 7) ^ (r & 7)) << 4));
}

// One CTA = (split of the cache, KV head x head chunk, batch).  Warps 0-3 compute, each on its own
// 32 keys of every 128-key tile and with its own running (m, l, O), so there is no CTA-wide
// synchronisation inside the loop; the four states are merged once at the end.  Warp 4 is the TMA
// producer.  S = Q K^T and O += P V run as m16n8k16 BF16 MMAs whose 16 rows are the G <= 16 query
// heads that share this KV head (rows >= G are zero padding).
template <int D>
__global__ void __launch_bounds__(160)
attn_decode_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                   const DecodeParams p) {
    using Cfg = DecodeCfg<D>;
    constexpr int NST = Cfg::kStages;
    constexpr int KS = D / 16;  // k-steps of Q K^T
    constexpr int DT = D / 8;   // 8-column output tiles of P V
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sK = smem;
    uint8_t* sV = sK + NST * Cfg::kTileBytes;
    uint8_t* sQ = sV + NST * Cfg::kTileBytes;                        // [16 rows][D] BF16, swizzled like a tile
    float* sRed = reinterpret_cast<float*>(sK);  // [4 warps][16 rows][D + 2], used after the last tile only
    uint64_t* bars = reinterpret_cast<uint64_t*>(sQ + Cfg::kQBytes);
    uint64_t* bar_full = bars;        // [NST]
    uint64_t* bar_free = bars + NST;  // [NST]
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * NST);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = p.G;
    const int split = blockIdx.x;
    const int hk = int(blockIdx.y) / p.n_chunks;
    const int chunk = int(blockIdx.y) % p.n_chunks;
    const int b = blockIdx.z;
    const int h0 = hk * p.group + chunk * G;  // first query head served here
    const int tile0 = split * p.tiles_per_split;

    if (tid == 0) {
        for (int s = 0; s < NST; ++s) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_free[s], 128);
        }
        fence_mbar_init();
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
    }
    // launched with programmatic stream serialization: everything above overlaps the previous kernel's end (the
    // cache append that wrote q and the newest K / V row); nothing in global memory is touched before this wait
    grid_dep_wait();
    if (tid == 0) *abort_flag = *reinterpret_cast<volatile int*>(p.status);
    __syncthreads();
    if (*abort_flag != 0) return;
    // this sequence's length: a split that lies beyond it writes an empty partial (m = -inf, l = 0)
    const int L = p.lens ? max(1, min(__ldg(p.lens + b), p.L)) : p.L;
    const int n_all = (L + 127) / 128;
    const int n_tiles = max(0, min(p.tiles_per_split, n_all - tile0));
    // q rows of the G heads -> shared memory (BF16, 16-byte chunks, swizzled); rows >= G are zero
    for (int i = tid; i < 16 * (D / 8); i += blockDim.x) {
        const int r = i / (D / 8), c = i % (D / 8);
        uint4 val = make_uint4(0u, 0u, 0u, 0u);
        if (r < G) val = *reinterpret_cast<const uint4*>(p.q + (size_t(b) * p.Hq + h0 + r) * D + c * 8);
        *reinterpret_cast<uint4*>(sQ + swz_off(r, c, 16 * 128)) = val;
    }
    __syncthreads();

    if (warp == 4) {
        if (lane == 0) {
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
    // A fragments of Q (rows = heads): one ldmatrix.x4 per k-step
    uint32_t aq[KS][4];
    {
        const uint32_t q_base = smem_u32(sQ);
        const int r = (lane & 7) + ((lane >> 3) & 1) * 8;  // matrices 0,2: rows 0-7; 1,3: rows 8-15
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const int c = ks * 2 + (lane >> 4);  // matrices 0,1: k 0-7; 2,3: k 8-15
            ldsm_x4(q_base + swz_off(r, c, 16 * 128), aq[ks][0], aq[ks][1], aq[ks][2], aq[ks][3]);
        }
    }
    // this thread holds rows r0 = lane / 4 and r1 = r0 + 8 (query heads), key / head-dim columns (lane % 4) * 2 + {0, 1}
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    float o[DT][4];
#pragma unroll
    for (int dt = 0; dt < DT; ++dt) o[dt][0] = o[dt][1] = o[dt][2] = o[dt][3] = 0.f;
    const int kw = warp * 32;  // this warp's keys inside a tile
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
        const int s = j % NST;
        ok = mbar_wait_warp(&bar_full[s], (j / NST) & 1, abort_flag, p.status, DEV_WAIT_TIMEOUT_LOAD);
        if (!ok) break;
        const uint32_t k_base = smem_u32(sK + s * Cfg::kTileBytes);
        const uint32_t v_base = smem_u32(sV + s * Cfg::kTileBytes);
        // ---- S[16 heads x 32 keys] = Q K^T
        float sc[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
            const int key = kw + nt * 8 + (lane & 7);
#pragma unroll
            for (int kk = 0; kk < KS / 2; ++kk) {
                uint32_t b0, b1, b2, b3;  // chunks 4kk .. 4kk+3 of the key rows: two k-steps
                ldsm_x4(k_base + swz_off(key, kk * 4 + (lane >> 3), Cfg::kBoxBytes), b0, b1, b2, b3);
                mma_bf16_16816(sc[nt], aq[2 * kk], b0, b1);
                mma_bf16_16816(sc[nt], aq[2 * kk + 1], b2, b3);
            }
        }
        // ---- mask keys beyond the cache length (last tile only)
        const int key0 = (tile0 + j) * 128 + kw + (lane & 3) * 2;
        if ((tile0 + j) * 128 + 128 > L) {
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                if (key0 + nt * 8 >= L) sc[nt][0] = sc[nt][2] = -INFINITY;
                if (key0 + nt * 8 + 1 >= L) sc[nt][1] = sc[nt][3] = -INFINITY;
            }
        }
        // ---- online softmax per head row (rows r0 and r1), over this warp's 32 keys
        float mx0 = fmaxf(fmaxf(sc[0][0], sc[0][1]), fmaxf(sc[1][0], sc[1][1]));
        float mx1 = fmaxf(fmaxf(sc[0][2], sc[0][3]), fmaxf(sc[1][2], sc[1][3]));
        mx0 = fmaxf(mx0, fmaxf(fmaxf(sc[2][0], sc[2][1]), fmaxf(sc[3][0], sc[3][1])));
        mx1 = fmaxf(mx1, fmaxf(fmaxf(sc[2][2], sc[2][3]), fmaxf(sc[3][2], sc[3][3])));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        // a warp whose 32 keys are all beyond the cache has mn = -inf: keep its state neutral
        const float a0 = (mn0 == -INFINITY) ? 1.f : ex2_approx((m0 - mn0) * p.scale_log2);
        const float a1 = (mn1 == -INFINITY) ? 1.f : ex2_approx((m1 - mn1) * p.scale_log2);
        const float nb0 = (mn0 == -INFINITY) ? 0.f : -mn0 * p.scale_log2;
        const float nb1 = (mn1 == -INFINITY) ? 0.f : -mn1 * p.scale_log2;
        m0 = mn0;
        m1 = mn1;
        float rs0 = 0.f, rs1 = 0.f;
        uint32_t ap[2][4];  // P as A fragments: k-step kk covers keys 16 kk .. 16 kk + 15
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            const float p0 = ex2_approx(fmaf(sc[nt][0], p.scale_log2, nb0));
            const float p1 = ex2_approx(fmaf(sc[nt][1], p.scale_log2, nb0));
            const float p2 = ex2_approx(fmaf(sc[nt][2], p.scale_log2, nb1));
            const float p3 = ex2_approx(fmaf(sc[nt][3], p.scale_log2, nb1));
            rs0 += p0 + p1;
            rs1 += p2 + p3;
            ap[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16x2(p0, p1);
            ap[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16x2(p2, p3);
        }
        l0 = l0 * a0 + rs0;
        l1 = l1 * a1 + rs1;
        // ---- O[16 x D] = alpha O + P V
#pragma unroll
        for (int dt = 0; dt < DT; ++dt) {
            o[dt][0] *= a0;
            o[dt][1] *= a0;
            o[dt][2] *= a1;
            o[dt][3] *= a1;
        }
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
            const int key = kw + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;  // matrices 0,2: keys 0-7; 1,3: 8-15
#pragma unroll
            for (int dp = 0; dp < DT / 2; ++dp) {
                uint32_t b0, b1, b2, b3;  // head-dim chunks 2dp (matrices 0,1) and 2dp+1 (matrices 2,3)
                ldsm_x4_trans(v_base + swz_off(key, dp * 2 + (lane >> 4), Cfg::kBoxBytes), b0, b1, b2, b3);
                mma_bf16_16816(o[2 * dp], ap[kk], b0, b1);
                mma_bf16_16816(o[2 * dp + 1], ap[kk], b2, b3);
            }
        }
        // ordinary (ldmatrix) reads of a stage that TMA will overwrite: ordered before the async proxy's write
        fence_proxy_async_smem();
        mbar_arrive(&bar_free[s]);
    }
    // ---- merge the four warps' states and write the split's partial (un-normalised O, m, l)
    named_bar_sync(1, 128);  // every compute thread, also after a wait that gave up
    if (*abort_flag != 0) return;
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    constexpr int RS = D + 2;  // row stride of the scratch: O row, then m, then l
    float* mine = sRed + warp * 16 * RS;
    const int r0 = lane >> 2, r1 = r0 + 8, cq = (lane & 3) * 2;
#pragma unroll
    for (int dt = 0; dt < DT; ++dt) {
        mine[r0 * RS + dt * 8 + cq] = o[dt][0];
        mine[r0 * RS + dt * 8 + cq + 1] = o[dt][1];
        mine[r1 * RS + dt * 8 + cq] = o[dt][2];
        mine[r1 * RS + dt * 8 + cq + 1] = o[dt][3];
    }
    if ((lane & 3) == 0) {
        mine[r0 * RS + D] = m0;
        mine[r0 * RS + D + 1] = l0;
        mine[r1 * RS + D] = m1;
        mine[r1 * RS + D + 1] = l1;
    }
    named_bar_sync(1, 128);
    for (int i = tid; i < G * D; i += 128) {
        const int g = i / D, d = i % D;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) m = fmaxf(m, sRed[(w * 16 + g) * RS + D]);
        float acc = 0.f, l = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = sRed[(w * 16 + g) * RS + D];
            const float f = (mw == -INFINITY) ? 0.f : ex2_approx((mw - m) * p.scale_log2);
            acc += f * sRed[(w * 16 + g) * RS + d];
            l += f * sRed[(w * 16 + g) * RS + D + 1];
        }
        const size_t idx = (size_t(b) * p.Hq + h0 + g) * p.n_splits + split;
        p.part_o[idx * D + d] = acc;
        if (d == 0) {
            p.part_m[idx] = m;
            p.part_l[idx] = l;
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
    grid_dep_wait();  // the partials come from the kernel before this one
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
