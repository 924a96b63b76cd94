// Inline-PTX building blocks for the sm_100a attention kernels: mbarriers with
// bounded waits, TMA tiled loads/stores, TMEM allocation, tcgen05 MMA issue,
// commit and TMEM load/store, plus the shared-memory and instruction
// descriptors those MMAs consume.
//
// Every wait in this file is bounded.  A wait that runs out records a code in
// a device status word and returns false; callers unwind to their teardown
// (TMEM is freed, no thread is left spinning).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200attn {

// ---------------------------------------------------------------------------
// Status codes written by kernels into the device status word.
// ---------------------------------------------------------------------------
enum DeviceStatus : int {
    DEV_OK = 0,
    DEV_WAIT_TIMEOUT_LOAD = 101,   // a TMA-load barrier never completed
    DEV_WAIT_TIMEOUT_MMA = 102,    // a tcgen05.commit barrier never completed
    DEV_WAIT_TIMEOUT_SOFTMAX = 103,// a softmax->MMA hand-off barrier never completed
    DEV_WAIT_TIMEOUT_FREE = 104,   // a stage/TMEM "free" barrier never completed
    DEV_KV_CACHE_OVERFLOW = 105,   // kv_append with per-sequence positions: a position + n_new exceeds the capacity
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// Makes generic-proxy writes to shared memory visible to the async proxy
// (TMA stores, tcgen05.mma operand reads).
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Spin budget: the clock is sampled every 256 failed probes; a wait gives up
// after ~2^31 SM clocks (about a second at B200 clocks).
constexpr long long kWaitBudgetClocks = 1ll << 31;

// Bounded wait.  `abort_flag` is a CTA-shared word: once any thread of the CTA
// has given up, every other wait in the CTA returns false at its next probe.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          int* status, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    long long t0 = clock64();
    uint32_t spins = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++spins & 255u) == 0) {
            if (*abort_flag != 0) return false;
            if (clock64() - t0 > kWaitBudgetClocks) {
                *abort_flag = code;
                atomicCAS(status, 0, code);
                return false;
            }
        }
    }
}

// ---------------------------------------------------------------------------
// TMA (cp.async.bulk.tensor), no multicast anywhere.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1, int c2,
                                            int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, "
        "%6}], [%2];" ::"r"(smem_u32(dst)),
        "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
// Untiled bulk copy global -> shared; both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_load_1d(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* m, const void* src, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(
                     reinterpret_cast<uint64_t>(m)),
                 "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until the bulk stores of this thread have finished READING shared memory.
__device__ __forceinline__ void tma_store_wait_read0() {
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
// Waits until the bulk stores of this thread are complete (global writes done).
__device__ __forceinline__ void tma_store_wait0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ---------------------------------------------------------------------------
// TMEM allocation (one warp, converged).
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------------------
// Descriptors
// ---------------------------------------------------------------------------
// Instruction descriptor for tcgen05.mma kind::f16 with BF16 A/B and FP32 D.
// Bit layout: [4,6) D format (1 = F32), [7,10) A format (1 = BF16), [10,13) B
// format, [15] A major (0 = K-major, 1 = MN-major), [16] B major, [17,23)
// N >> 3, [24,29) M >> 4.
__host__ __device__ constexpr uint32_t make_idesc_bf16(int M, int N, int a_mn_major, int b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(a_mn_major) << 15) | (uint32_t(b_mn_major) << 16) |
           (uint32_t(N >> 3) << 17) | (uint32_t(M >> 4) << 24);
}

// Shared-memory matrix descriptor, 128-byte swizzle, sm_100 version field = 1.
// start/LBO/SBO are byte quantities (16-byte granular).
//  * K-major operand  ([rows][64 bf16], 128 B per row): SBO = 1024 (stride
//    between 8-row groups); LBO unused (1).  Step along K by +32 B per 16
//    elements inside the 128-byte row.
//  * MN-major operand ([k rows][64 bf16 of M/N], 128 B per k row): SBO = 1024
//    (stride between 8-k-row groups), LBO = stride between 64-element chunks
//    along M/N.  Step along K by +2048 B per 16 k rows.
__device__ __forceinline__ uint64_t make_sdesc_sw128(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= uint64_t((smem_addr & 0x3FFFFu) >> 4);
    d |= uint64_t((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= uint64_t((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= uint64_t(1) << 46;  // descriptor version (Blackwell)
    d |= uint64_t(2) << 61;  // SWIZZLE_128B
    return d;
}

// Programmatic dependent launch: a kernel launched with the programmatic-stream-serialization
// attribute may become resident while the previous kernel of the stream is still draining.
// grid_dep_launch() lets the NEXT kernel start its own set-up early; grid_dep_wait() blocks
// until the PREVIOUS kernel has completed and its writes are visible.  Every kernel here does
// its set-up (barriers, TMEM, tensor-map prefetch) first and calls grid_dep_wait() before its
// first access to global memory, so only set-up and launch latency overlap.  The persistent
// kernels do not call grid_dep_launch(): all their CTAs start at once, so the call would release
// the next kernel at this one's very beginning, and a dependent grid queued behind a kernel for
// its whole run time measured slower (2 %) than one released as the CTAs exit, which is what
// happens without the call.
__device__ __forceinline__ void grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }


// Elects one lane of a fully converged warp.  The MMA and TMA issuing warps run their loops
// with all 32 lanes (so that addresses and descriptors stay in the uniform datapath) and
// guard only the issuing instructions with this.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred = 0;
    asm volatile(
        "{\n\t"
        ".reg .pred P;\n\t"
        "elect.sync _|P, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t"
        "}\n"
        : "=r"(pred));
    return pred != 0;
}

// Bounded wait executed by a whole warp; the result is made warp-uniform.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status,
                                               int code) {
    return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag, status, code));
}

// ---------------------------------------------------------------------------
// Division of n < 2^31 by a divisor fixed per launch, through one multiply-high and one shift (the round-up
// method of Granlund and Montgomery: mul = ceil(2^(31 + ceil(log2 d)) / d), shr = ceil(log2 d) - 1).  The
// kernels turn item and row numbers into (tile, head, batch) with it; a hardware division by a run-time
// value costs some twenty dependent instructions and sat in front of every item's first load.
// ---------------------------------------------------------------------------
struct FastDiv {
    unsigned d, mul, shr;
};
inline FastDiv fastdiv_make(unsigned d) {
    FastDiv f = {d, 0u, 0u};
    if (d <= 1) return f;
    unsigned lg = 0;
    while ((1u << lg) < d) ++lg;
    const unsigned p = 31 + lg;
    f.mul = static_cast<unsigned>(((1ull << p) + d - 1) / d);
    f.shr = p - 32;
    return f;
}
__device__ __forceinline__ unsigned fastdiv(unsigned n, const FastDiv& f) {
    return f.d == 1 ? n : (__umulhi(n, f.mul) >> f.shr);
}

// ---------------------------------------------------------------------------
// Work distribution of the persistent kernels.  Items are numbered by decreasing cost.  A CTA
// starts with item blockIdx.x; every further item comes from a device-wide counter (sched[0]), so
// that whichever CTA is free takes the most expensive item left.  The producer warp of a CTA
// fetches the ids one item ahead and hands them to the other warps through a ring of kItemRing
// entries in shared memory, one mbarrier per entry; the entry of the CTA's n-th item is n % kItemRing
// and completes phase n / kItemRing of its barrier.  (No warp is ever more than a few items behind
// the producer, because the producer's loads wait for the buffers those warps release, so an entry
// is never rewritten before every warp has read it, and a waiter is never more than one phase
// behind.)  An id of -1 ends the list.  When a CTA's list has ended it counts itself in sched[1]; the
// last CTA to do so clears both words for the next launch that uses them.
// ---------------------------------------------------------------------------
constexpr int kItemRing = 8;

// Producer, lane 0 only: hand item `id` (or -1) to the CTA as its n-th item.
__device__ __forceinline__ void item_publish(uint64_t* bar_item, volatile int* ring, int n, int id) {
    ring[n % kItemRing] = id;
    mbar_arrive(&bar_item[n % kItemRing]);  // release: the id is visible to whoever sees the phase complete
}
// Any warp: the id of this CTA's n-th item, -1 at the end of the list or after a wait that gave up.
__device__ __forceinline__ int item_get(uint64_t* bar_item, volatile int* ring, int n, volatile int* abort_flag,
                                        int* status) {
    if (!mbar_wait_warp(&bar_item[n % kItemRing], uint32_t(n / kItemRing) & 1, abort_flag, status, DEV_WAIT_TIMEOUT_LOAD))
        return -1;
    return ring[n % kItemRing];
}
// Producer, lane 0 only: the id of this CTA's n-th item (n >= 1) from the device-wide counter (ids below
// n_ctas are the CTAs' first items).  Without a counter (sched == nullptr) the items are dealt statically
// in rounds, every other round in reverse CTA order, so that the CTA that got the most expensive item
// of one round gets the cheapest of the next.
__device__ __forceinline__ int sched_fetch(int* sched, int n, int cta, int n_ctas) {
    if (sched == nullptr) return n * n_ctas + ((n & 1) ? n_ctas - 1 - cta : cta);
    return n_ctas + atomicAdd(&sched[0], 1);
}
// A static deal prepared on the host (a kernel parameter): CTA c takes ids[c * per_cta + n] as its n-th item,
// kItemTableEnd ends its list.  The host balances the lists by their work (longest processing time first) and
// hands the heavier lists to the lower block indices: with two CTAs per SM the hardware places block i and block
// i + n_SMs on the same SM (measured: every SM got one block of each half in every launch), so an SM's two lists
// are one heavy and one light one and all SMs finish together; the formula above leaves some SMs with two heavy
// lists.  per_cta == 0: no table, use the formula (or the counter).
constexpr int kItemTableCtas = 296, kItemTableMaxPerCta = 8;
constexpr unsigned short kItemTableEnd = 0xffffu;
struct ItemTable {
    int per_cta;
    unsigned short ids[kItemTableCtas * kItemTableMaxPerCta];
};
__device__ __forceinline__ int sched_fetch(const ItemTable& tab, int* sched, int n, int cta, int n_ctas) {
    if (sched != nullptr || tab.per_cta == 0) return sched_fetch(sched, n, cta, n_ctas);
    if (n >= tab.per_cta) return 0x7fffffff;
    const unsigned short id = tab.ids[cta * tab.per_cta + n];
    return id == kItemTableEnd ? 0x7fffffff : int(id);
}
// the CTA's first item: its block index, unless a table says otherwise
__device__ __forceinline__ int sched_first(const ItemTable& tab, int* sched, int cta) {
    return (sched != nullptr || tab.per_cta == 0) ? cta : int(tab.ids[cta * tab.per_cta]);
}
// Producer, lane 0 only, after its last sched_fetch: count this CTA; the last one resets the counters.
__device__ __forceinline__ void sched_finish(int* sched, int n_ctas) {
    if (sched == nullptr) return;
    __threadfence();
    if (atomicAdd(&sched[1], 1) == n_ctas - 1) {
        __threadfence();
        sched[0] = 0;
        sched[1] = 0;
    }
}

// Descriptor offset (in the 16-byte units of the start-address field) of K step `ks` of a
// K-major operand made of [128 rows][64] boxes of `box_bytes`.
__host__ __device__ constexpr uint32_t kmajor_step(int ks, int box_bytes) {
    return uint32_t(((ks / 4) * box_bytes + (ks % 4) * 32) >> 4);
}

// ---------------------------------------------------------------------------
// tcgen05.mma (issued by ONE thread), cta_group::1, kind::f16.
// ---------------------------------------------------------------------------
// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Makes `bar` receive one arrival when all MMAs issued so far by this thread
// have completed (implies tcgen05.fence::before_thread_sync).
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// ---------------------------------------------------------------------------
// TMEM <-> registers, shape 32x32b: thread t of the warp touches lane
// (lane_base + t), 32-bit column (col + i) for register i.
// ---------------------------------------------------------------------------
#define B200ATTN_R8(v, o) \
    "=r"(v[o + 0]), "=r"(v[o + 1]), "=r"(v[o + 2]), "=r"(v[o + 3]), "=r"(v[o + 4]), "=r"(v[o + 5]), "=r"(v[o + 6]), \
        "=r"(v[o + 7])
#define B200ATTN_W8(v, o) \
    "r"(v[o + 0]), "r"(v[o + 1]), "r"(v[o + 2]), "r"(v[o + 3]), "r"(v[o + 4]), "r"(v[o + 5]), "r"(v[o + 6]), \
        "r"(v[o + 7])

__device__ __forceinline__ void tmem_ld_x8(uint32_t taddr, uint32_t* v) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : B200ATTN_R8(v, 0)
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld_x16(uint32_t taddr, uint32_t* v) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : B200ATTN_R8(v, 0), B200ATTN_R8(v, 8)
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t* v) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
        "%29,%30,%31}, [%32];"
        : B200ATTN_R8(v, 0), B200ATTN_R8(v, 8), B200ATTN_R8(v, 16), B200ATTN_R8(v, 24)
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st_x8(uint32_t taddr, const uint32_t* v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr),
                 B200ATTN_W8(v, 0)
                 : "memory");
}
__device__ __forceinline__ void tmem_st_x16(uint32_t taddr, const uint32_t* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(
            taddr),
        B200ATTN_W8(v, 0), B200ATTN_W8(v, 8)
        : "memory");
}
__device__ __forceinline__ void tmem_st_x32(uint32_t taddr, const uint32_t* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,"
        "%30,%31,%32};" ::"r"(taddr),
        B200ATTN_W8(v, 0), B200ATTN_W8(v, 8), B200ATTN_W8(v, 16), B200ATTN_W8(v, 24)
        : "memory");
}

// Packs two floats to a bf16x2 word, `lo` in bits [0,16).
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Register re-balancing between warpgroups (each executed by all four warps of a group).
template <int N>
__device__ __forceinline__ void reg_alloc() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void reg_dealloc() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

// Optional phase timestamps for tuning (compiled in only with -DB200ATTN_PROBE): the first
// CTA of a launch records clock64() at numbered points into a device array.
#ifdef B200ATTN_PROBE
__device__ long long g_probe[512];
#define B200ATTN_STAMP(cond, idx)                                                      \
    do {                                                                               \
        if ((cond) && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (idx) < 512) \
            g_probe[(idx)] = clock64();                                                \
    } while (0)
// Per-CTA trace: SM id and begin/end times (ns) of the first 2048 CTAs of a launch, kept per kernel
// (k = 0 forward, 1 dQ pass, 2 dK/dV pass).
__device__ unsigned long long g_trace[8192 * 3];
__device__ long long g_trace_clk[8192 * 2];  // clock64() at the same two points
__device__ __forceinline__ unsigned long long b200attn_globaltimer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ unsigned b200attn_smid() {
    unsigned r;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(r));
    return r;
}
#define B200ATTN_TRACE_BEGIN(k)                                                                     \
    do {                                                                                            \
        const unsigned lin_ = (k) * 2048 + blockIdx.x;                                              \
        if (threadIdx.x == 0 && blockIdx.x < 2048) {                                                \
            g_trace[lin_ * 3 + 0] = b200attn_smid();                                                \
            g_trace[lin_ * 3 + 1] = b200attn_globaltimer();                                         \
            g_trace_clk[lin_ * 2 + 0] = clock64();                                                  \
        }                                                                                           \
    } while (0)
#define B200ATTN_TRACE_END(k)                                                                       \
    do {                                                                                            \
        const unsigned lin_ = (k) * 2048 + blockIdx.x;                                              \
        if (threadIdx.x == 0 && blockIdx.x < 2048) {                                                \
            g_trace[lin_ * 3 + 2] = b200attn_globaltimer();                                         \
            g_trace_clk[lin_ * 2 + 1] = clock64();                                                  \
        }                                                                                           \
    } while (0)
#else
#define B200ATTN_TRACE_BEGIN(k) \
    do {                        \
    } while (0)
#define B200ATTN_TRACE_END(k) \
    do {                      \
    } while (0)
#define B200ATTN_STAMP(cond, idx) \
    do {                          \
    } while (0)
#endif

// Named barrier among a subset of the CTA's warps.
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

}  // namespace b200attn
