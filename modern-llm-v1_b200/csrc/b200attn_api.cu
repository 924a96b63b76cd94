// C-ABI launcher for the sm_100a attention kernels (see include/b200attn.h for
// the contract).  Host side only validates, builds TMA tensor maps and enqueues.
#include "../../include/b200attn.h"
#include "b200attn_debug.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <functional>
#include <queue>
#include <utility>
#include <vector>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>

#include "attn_bwd.cuh"
#include "attn_bwd_onepass.cuh"
#include "attn_decode.cuh"
#include "attn_fwd.cuh"
#include "kv_cache.cuh"
#include "rope_norm.cuh"
#include "tmap.h"

using namespace b200attn;

namespace {

// One status word per device, living in the library's device image.
__device__ int g_status_word;

constexpr int kMaxDevices = 64;
int* g_status_ptr[kMaxDevices] = {nullptr};

// Item counters of the persistent kernels (two words per launch, see ptx.cuh), also in the device
// image (zero at load).  A kernel leaves its two words zero again when it ends, so one pair would do
// for launches that follow each other on one stream; consecutive launches take consecutive pairs so
// that launches running at the same time on different streams do not share one.  (Two launches
// kSchedSlots launches apart that overlap in time, or one captured graph replayed concurrently with
// itself, would share a pair: serialise those.)  A kernel that gave up on a wait may leave its pair
// non-zero; b200attn_last_device_status clears all pairs when it reports such a failure, and until
// then every kernel exits at once because the status word is set.
constexpr int kSchedSlots = 64;
__device__ int g_sched_words[2 * kSchedSlots];
int* g_sched_ptr[kMaxDevices] = {nullptr};
std::atomic<unsigned> g_sched_seq{0};

// Returns the device address of the status word of the current device (resolved once per device).
int* status_ptr(int* err) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        *err = B200ATTN_ERR_NO_DEVICE;
        return nullptr;
    }
    if (!g_status_ptr[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) {
            cudaGetLastError();
            *err = B200ATTN_ERR_NO_DEVICE;
            return nullptr;
        }
        if (cudaMemset(p, 0, sizeof(int)) != cudaSuccess) {
            cudaGetLastError();
            *err = B200ATTN_ERR_CUDA;
            return nullptr;
        }
        void* sp = nullptr;
        if (cudaGetSymbolAddress(&sp, g_sched_words) != cudaSuccess) {
            cudaGetLastError();
            *err = B200ATTN_ERR_NO_DEVICE;
            return nullptr;
        }
        g_sched_ptr[dev] = static_cast<int*>(sp);
        g_status_ptr[dev] = static_cast<int*>(p);
    }
    return g_status_ptr[dev];
}

// The counter pair for the next launch of a persistent kernel on the current device (status_ptr()
// has resolved the device's addresses before).
// Returns nullptr when the items should be dealt statically: with only a few items per CTA a static
// deal in rounds of alternating direction balances better than first come, first served, because a CTA
// takes its next item before it has finished the current one.  (B200ATTN_ITEMS=static|dynamic overrides.)
int* next_sched_pair(long long n_items, unsigned n_ctas) {
    static const int forced = [] {
        const char* e = getenv("B200ATTN_ITEMS");
        return !e ? 0 : (e[0] == 's' ? 1 : (e[0] == 'd' ? 2 : 0));
    }();
    if (forced == 1 || (forced == 0 && n_items < 4LL * n_ctas)) return nullptr;
    int dev = 0;
    cudaGetDevice(&dev);
    return g_sched_ptr[dev] + 2 * (g_sched_seq.fetch_add(1, std::memory_order_relaxed) % kSchedSlots);
}

// The static deal of the forward and the dQ pass (two CTAs per SM) as a table: items (ids are heaviest first;
// item id covers query tile n_qtiles - 1 - id / n_groups, i.e. that many 64-key tiles plus item_cost half tiles
// for its loads and epilogue; the deal at the training shapes is the same for costs from 1 to 8) go, longest first, to the list with the least work; then the lists are handed out by
// falling work, so that block i (one of the first n_SMs blocks) and block i + n_SMs, which share an SM, get a
// heavy and a light list.  Returns a table with per_cta == 0 when the deal does not fit the table (the kernel
// then uses the closed formula) or when B200ATTN_ITEMS=static asks for the formula.
const ItemTable& item_table_for(long long n_items, unsigned n_ctas, int n_groups, int n_qtiles, int T, int item_cost) {
    static const ItemTable none = [] {
        ItemTable t;
        t.per_cta = 0;
        return t;
    }();
    static const bool formula = [] {
        const char* e = getenv("B200ATTN_ITEMS");
        return e && e[0] == 's';
    }();
    if (formula || n_ctas > (unsigned)kItemTableCtas || n_items >= 0xffff || n_items < (long long)n_ctas) return none;
    struct Entry {
        long long n_items = -1;
        unsigned n_ctas = 0;
        int n_groups = 0, n_qtiles = 0, T = 0, cost = 0;
        ItemTable tab;
    };
    thread_local Entry cache[4];
    thread_local unsigned next = 0;
    for (Entry& e : cache)
        if (e.n_items == n_items && e.n_ctas == n_ctas && e.n_groups == n_groups && e.n_qtiles == n_qtiles && e.T == T &&
            e.cost == item_cost)
            return e.tab.per_cta >= 0 ? e.tab : none;
    Entry& e = cache[next++ % 4];
    e.n_items = n_items, e.n_ctas = n_ctas, e.n_groups = n_groups, e.n_qtiles = n_qtiles, e.T = T, e.cost = item_cost;
    // longest processing time first; work in half tiles: an item costs its tiles plus half a tile
    std::vector<std::vector<unsigned short>> lists(n_ctas);
    std::vector<long long> load(n_ctas, 0);
    using Slot = std::pair<long long, unsigned>;  // (work, list), least work first, then lowest index
    std::priority_queue<Slot, std::vector<Slot>, std::greater<Slot>> heap;
    for (unsigned c = 0; c < n_ctas; ++c) heap.push({0, c});
    size_t longest = 0;
    for (long long id = 0; id < n_items; ++id) {
        const int qt = n_qtiles - 1 - (int)(id / n_groups);
        const int rows = std::min(T, qt * 128 + 128);
        const long long work = 2 * ((rows + 63) / 64) + item_cost;
        const Slot s = heap.top();
        heap.pop();
        lists[s.second].push_back((unsigned short)id);
        load[s.second] = s.first + work;
        heap.push({load[s.second], s.second});
        longest = std::max(longest, lists[s.second].size());
    }
    if (longest > (size_t)kItemTableMaxPerCta) {
        e.tab.per_cta = -1;  // remembered as "no table"
        return none;
    }
    std::vector<unsigned> order(n_ctas);
    for (unsigned c = 0; c < n_ctas; ++c) order[c] = c;
    std::stable_sort(order.begin(), order.end(), [&](unsigned a, unsigned b) { return load[a] > load[b]; });
    e.tab.per_cta = (int)longest;
    for (unsigned c = 0; c < n_ctas; ++c)
        for (size_t n = 0; n < longest; ++n)
            e.tab.ids[c * longest + n] = n < lists[order[c]].size() ? lists[order[c]][n] : kItemTableEnd;
    return e.tab;
}

// SM count of the current device (cached per device).
int sm_count() {
    static int cached[kMaxDevices] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

struct Strides {
    long long t, h, b;  // element strides
};

inline Strides strides_for(int layout, int H, int T, int D) {
    Strides s;
    if (layout == B200ATTN_LAYOUT_BHTD) {
        s.t = D;
        s.h = (long long)T * D;
        s.b = (long long)H * T * D;
    } else {
        s.t = (long long)H * D;
        s.h = D;
        s.b = (long long)T * H * D;
    }
    return s;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int check_common(int B, int T, int Hq, int Hkv, int D, int layout) {
    if (B <= 0 || T <= 0 || Hq <= 0 || Hkv <= 0 || D <= 0) return B200ATTN_ERR_INVALID_ARG;
    if (Hq % Hkv != 0) return B200ATTN_ERR_INVALID_ARG;
    if (layout != B200ATTN_LAYOUT_BHTD && layout != B200ATTN_LAYOUT_BTHD) return B200ATTN_ERR_INVALID_ARG;
    if (D != 64 && D != 128) return B200ATTN_ERR_UNSUPPORTED;
    return B200ATTN_OK;
}

// Launch with programmatic stream serialization: the kernel may become resident while the
// previous kernel of the stream drains; it calls griddepcontrol.wait before touching global memory.
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, unsigned block, size_t smem, cudaStream_t st,
                       Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(block, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <int D>
int launch_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FwdParams& p,
               cudaStream_t st) {
    using Cfg = FwdCfg<D>;
    static bool attr_set[kMaxDevices] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_set[dev]) {
        if (cudaFuncSetAttribute(attn_fwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) !=
            cudaSuccess) {
            cudaGetLastError();
            return B200ATTN_ERR_CUDA;
        }
        attr_set[dev] = true;
    }
    // persistent CTAs, two per SM, each walking a heaviest-first list of (query tile, head, batch) items
    const long long items = (long long)p.n_qtiles * p.Hq * p.B;
    const unsigned grid = (unsigned)std::min<long long>(items, 2LL * sm_count());
    FwdParams pl = p;
    pl.sched = next_sched_pair(items, grid);
    pl.div_bh = fastdiv_make((unsigned)(p.B * p.Hq));
    pl.div_h = fastdiv_make((unsigned)p.Hq);
    pl.div_group = fastdiv_make((unsigned)p.group);
    const ItemTable& tab = item_table_for(pl.sched ? -1 : items, grid, p.B * p.Hq, p.n_qtiles, p.T, 1);
    if (launch_pdl(attn_fwd_kernel<D>, grid, 256, Cfg::kSmemBytes, st, tq, tk, tv, pl, tab) != cudaSuccess) {
        cudaGetLastError();
        return B200ATTN_ERR_CUDA;
    }
    return B200ATTN_OK;
}

}  // namespace

namespace {

// The forward with K and V at their own strides (sk): the training call passes the strides of `layout`, the
// prefill over a KV cache those of the cache.
int fwd_run(const void* q, const void* k, const void* v, void* o, float* lse, int B, int T, int kv_off, int Hq, int Hkv, int D,
            int layout, const Strides& sk, float softmax_scale, void* stream) {
    int rc = check_common(B, T, Hq, Hkv, D, layout);
    if (rc) return rc;
    if (!q || !k || !v || !o || !lse) return B200ATTN_ERR_INVALID_ARG;
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o)) return B200ATTN_ERR_ALIGNMENT;
    int* status = status_ptr(&rc);
    if (!status) return rc;
    const Strides sq = strides_for(layout, Hq, T, D);
    CUtensorMap tq, tk, tv;
    if (!make_tmap_bf16_4d(&tq, q, D, T, Hq, B, sq.t, sq.h, sq.b, 128) ||
        !make_tmap_bf16_4d(&tk, k, D, kv_off + T, Hkv, B, sk.t, sk.h, sk.b, 64) ||
        !make_tmap_bf16_4d(&tv, v, D, kv_off + T, Hkv, B, sk.t, sk.h, sk.b, 64))
        return B200ATTN_ERR_TENSOR_MAP;
    FwdParams p;
    p.B = B;
    p.T = T;
    p.Hq = Hq;
    p.Hkv = Hkv;
    p.group = Hq / Hkv;
    p.n_qtiles = (T + 127) / 128;
    p.kv_off = kv_off;
    p.scale = softmax_scale > 0.f ? softmax_scale : 1.f / sqrtf((float)D);
    p.scale_log2 = p.scale * 1.4426950408889634f;
    p.lse = lse;
    p.o = static_cast<uint16_t*>(o);
    p.o_st = sq.t;
    p.o_sh = sq.h;
    p.o_sb = sq.b;
    p.status = status;
    p.sched = nullptr;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return D == 64 ? launch_fwd<64>(tq, tk, tv, p, st) : launch_fwd<128>(tq, tk, tv, p, st);
}

}  // namespace

extern "C" int b200attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int T, int Hq,
                            int Hkv, int D, int layout, float softmax_scale, void* stream) {
    if (T <= 0 || Hkv <= 0 || D <= 0) return B200ATTN_ERR_INVALID_ARG;
    return fwd_run(q, k, v, o, lse, B, T, 0, Hq, Hkv, D, layout, strides_for(layout, Hkv, T, D), softmax_scale, stream);
}

extern "C" int b200attn_fwd_kvcache(const void* q, const void* kcache, const void* vcache, void* o, float* lse, int B,
                                    int T, int L_cap, int Hq, int Hkv, int D, int q_layout, float softmax_scale,
                                    void* stream) {
    return b200attn_fwd_kvcache_at(q, kcache, vcache, o, lse, B, T, 0, L_cap, Hq, Hkv, D, q_layout, softmax_scale, stream);
}

extern "C" int b200attn_fwd_kvcache_at(const void* q, const void* kcache, const void* vcache, void* o, float* lse, int B,
                                       int T, int pos0, int L_cap, int Hq, int Hkv, int D, int q_layout,
                                       float softmax_scale, void* stream) {
    if (T <= 0 || pos0 < 0 || Hkv <= 0 || D <= 0 || (long long)pos0 + T > L_cap) return B200ATTN_ERR_INVALID_ARG;
    return fwd_run(q, kcache, vcache, o, lse, B, T, pos0, Hq, Hkv, D, q_layout,
                   strides_for(B200ATTN_LAYOUT_BHTD, Hkv, L_cap, D), softmax_scale, stream);
}

namespace {

inline size_t bwd_vec_elems(int B, int T, int Hq) { return (size_t)B * Hq * (size_t)((T + 127) / 128 * 128); }

template <typename K>
int set_smem_once(K kernel, int bytes, bool* done) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (!done[dev]) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) {
            cudaGetLastError();
            return B200ATTN_ERR_CUDA;
        }
        done[dev] = true;
    }
    return B200ATTN_OK;
}

cudaEvent_t g_bwd_events[4] = {nullptr, nullptr, nullptr, nullptr};

inline void record_bwd_event(int i, cudaStream_t st) {
    if (g_bwd_events[i]) cudaEventRecord(g_bwd_events[i], st);
}

// Which backward runs.  The one-pass kernel (attn_bwd_onepass.cuh) exists for D = 64; it needs the FP32 dQ
// accumulator behind the two row vectors in the workspace.  AUTO is the two-pass backward: measured on B200 the
// one-pass kernel moves as many bytes through shared memory per block of scores as the two passes together (the
// limiter of every D = 64 kernel here) and pays two HBM-bound kernels around it, so it only draws level from
// T = 4096 on.  The environment variable B200ATTN_BWD=two_pass|one_pass overrides AUTO.
inline size_t bwd_acc_bytes(int B, int T, int Hq, int D) { return bwd_vec_elems(B, T, Hq) * (size_t)D * sizeof(float); }
inline size_t bwd_vec_bytes_padded(int B, int T, int Hq) { return (2 * bwd_vec_elems(B, T, Hq) * sizeof(float) + 255) & ~(size_t)255; }

int bwd_resolve_mode(int mode, int B, int T, int Hq, int D) {
    static const int forced = [] {
        const char* e = getenv("B200ATTN_BWD");
        return !e ? 0 : (e[0] == 't' ? B200ATTN_BWD_TWO_PASS : (e[0] == 'o' ? B200ATTN_BWD_ONE_PASS : 0));
    }();
    if (mode == B200ATTN_BWD_AUTO) {
        mode = forced ? forced : B200ATTN_BWD_TWO_PASS;
        if (D != 64) mode = B200ATTN_BWD_TWO_PASS;
        (void)B, (void)T, (void)Hq;
    }
    return mode;
}

// One-pass backward (D = 64): row vectors + cleared accumulator, the fused kernel, accumulator -> dq.
int launch_bwd_onepass(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdo,
                       const BwdParams& p, float* dq_acc, cudaStream_t st) {
    static bool set[kMaxDevices] = {false};
    int rc = set_smem_once(attn_bwd_onepass_kernel, OnePassCfg::kSmemBytes, set);
    if (rc) return rc;
    record_bwd_event(0, st);
    const unsigned q_tiles = (unsigned)(p.n_tiles * p.Hq * p.B);
    if (launch_pdl(attn_bwd_prep_kernel<64>, q_tiles, 256, 0, st, p, dq_acc) != cudaSuccess) {
        cudaGetLastError();
        return B200ATTN_ERR_CUDA;
    }
    record_bwd_event(1, st);
    const unsigned kv_items = (unsigned)(p.n_tiles * p.Hkv * p.B);
    const unsigned kv_grid = std::min(kv_items, (unsigned)sm_count());
    BwdParams pk = p;
    pk.sched2 = next_sched_pair(kv_items, kv_grid);
    if (launch_pdl(attn_bwd_onepass_kernel, kv_grid, OnePassCfg::kThreads, OnePassCfg::kSmemBytes, st, tk, tv, tq, tdo, pk,
                   dq_acc) != cudaSuccess) {
        cudaGetLastError();
        return B200ATTN_ERR_CUDA;
    }
    record_bwd_event(2, st);
    const float* acc_c = dq_acc;
    if (launch_pdl(attn_bwd_dq_convert_kernel<64>, q_tiles, 128, 0, st, p, acc_c) != cudaSuccess) {
        cudaGetLastError();
        return B200ATTN_ERR_CUDA;
    }
    record_bwd_event(3, st);
    return B200ATTN_OK;
}

template <int D>
int launch_bwd(const CUtensorMap& tq, const CUtensorMap& tk64, const CUtensorMap& tv64, const CUtensorMap& tk,
               const CUtensorMap& tv, const CUtensorMap& tdo, const CUtensorMap& to, const CUtensorMap& tdq,
               const CUtensorMap& tdk, const CUtensorMap& tdv, const BwdParams& p, cudaStream_t st) {
    static bool dq_set[kMaxDevices] = {false}, dkdv_set[kMaxDevices] = {false};
    // D = 64: 64-key tiles, two CTAs per SM.  D = 128: 128-key tiles, one CTA per SM (tensor-pipe bound).
    constexpr bool kWide = (D == 128);
    int rc;
    if constexpr (kWide) rc = set_smem_once(attn_bwd_dq_wide_kernel<D>, DqWideCfg<D>::kSmemBytes, dq_set);
    else rc = set_smem_once(attn_bwd_dq_kernel<D>, DqCfg<D>::kSmemBytes, dq_set);
    if (rc) return rc;
    rc = set_smem_once(attn_bwd_dkdv_kernel<D>, BwdCfg<D>::kSmemBytes, dkdv_set);
    if (rc) return rc;
    record_bwd_event(0, st);
    // the dQ pass also writes the two per-row vectors the dK/dV pass reads
    const unsigned dq_items = (unsigned)(p.n_tiles * p.Hq * p.B);
    cudaError_t e;
    if constexpr (kWide) {
        e = launch_pdl(attn_bwd_dq_wide_kernel<D>, dq_items, 320, DqWideCfg<D>::kSmemBytes, st, tq, tk, tv, tdo, tdq, p);
    } else {
        // the D = 64 kernel is persistent: two CTAs per SM walk the item list
        const unsigned dq_grid = std::min(dq_items, 2u * (unsigned)sm_count());
        BwdParams pq = p;
        pq.sched = next_sched_pair(dq_items, dq_grid);
        e = launch_pdl(attn_bwd_dq_kernel<D>, dq_grid, DqCfg<D>::kThreads, DqCfg<D>::kSmemBytes, st, tq, tk64, tv64, tdo, to, pq,
                       item_table_for(pq.sched ? -1 : (long long)dq_items, dq_grid, p.B * p.Hq, p.n_tiles, p.T, 4));
    }
    if (e != cudaSuccess) {
        cudaGetLastError();
        return B200ATTN_ERR_CUDA;
    }
    record_bwd_event(1, st);
    // the dK/dV pass is persistent too: one CTA per SM walks the list of (key tile, KV head, batch) items
    const unsigned kv_items = (unsigned)(p.n_tiles * p.Hkv * p.B);
    const unsigned kv_grid = std::min(kv_items, (unsigned)sm_count());
    BwdParams pk = p;
    pk.sched2 = next_sched_pair(kv_items, kv_grid);
    if (launch_pdl(attn_bwd_dkdv_kernel<D>, kv_grid, BwdCfg<D>::kThreads, BwdCfg<D>::kSmemBytes, st, tk, tv, tq, tdo,
                   tdk, tdv, pk) != cudaSuccess) {
        cudaGetLastError();
        return B200ATTN_ERR_CUDA;
    }
    record_bwd_event(2, st);
    return B200ATTN_OK;
}

}  // namespace

// ---------------------------------------------------------------------------------------
// Fused RoPE + QK-Norm (rope_norm.cuh)
// ---------------------------------------------------------------------------------------
namespace {

constexpr int kRopeNormMaxCtasPerSm = 8;  // 2048 threads per SM / 256

int rope_norm_check(int B, int T, int H, int D, int x_dtype, int x_layout, int y_layout) {
    if (B <= 0 || T <= 0 || H <= 0 || D <= 0) return B200ATTN_ERR_INVALID_ARG;
    if (x_dtype != B200ATTN_DTYPE_BF16 && x_dtype != B200ATTN_DTYPE_F32) return B200ATTN_ERR_INVALID_ARG;
    for (int l : {x_layout, y_layout})
        if (l != B200ATTN_LAYOUT_BHTD && l != B200ATTN_LAYOUT_BTHD) return B200ATTN_ERR_INVALID_ARG;
    if (D != 64 && D != 128) return B200ATTN_ERR_UNSUPPORTED;
    if ((long long)B * T * H >= (1LL << 31)) return B200ATTN_ERR_TOO_LARGE;  // rows are counted in 32 bits
    return B200ATTN_OK;
}

// grid: as many CTAs as the device keeps resident at once (asked of the runtime once per kernel and device), never
// more than the rows need
template <typename K>
unsigned rope_norm_grid(K kernel, long long rows, int rows_per_cta_iter, int* cached_occ, int dyn_smem = 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= kMaxDevices) dev = 0;
    if (cached_occ[dev] == 0) {
        int occ = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kernel, kRopeNormThreads, dyn_smem) != cudaSuccess || occ <= 0) {
            cudaGetLastError();
            occ = 1;
        }
        cached_occ[dev] = occ;
    }
    const long long need = (rows + rows_per_cta_iter - 1) / rows_per_cta_iter;
    const long long cap = (long long)cached_occ[dev] * sm_count();
    return (unsigned)std::max<long long>(1, std::min(need, cap));
}

template <int D, bool F32>
void rope_norm_launch_fwd(const RopeNormParams& p0, const RopeNormParams& p1, int n_tensors, long long rows,
                          cudaStream_t st) {
    static int occ[kMaxDevices] = {0};
    const unsigned grid = rope_norm_grid(rope_norm_fwd_kernel<D, F32>, rows, (kRopeNormThreads / 32) * kFwdSteps * (256 / D), occ);
    launch_pdl(rope_norm_fwd_kernel<D, F32>, dim3(grid, 1, 1), kRopeNormThreads, 0, st, p0, p1, n_tensors);
}
template <int D, bool F32>
void rope_norm_launch_bwd(RopeNormParams p0, RopeNormParams p1, int n_tensors, long long rows, float* workspace,
                          cudaStream_t st) {
    static int occ[kMaxDevices] = {0};
    static bool smem_set[kMaxDevices] = {false};
    constexpr int kSmem = kRopeNormBwdSmemBytes<F32>;
    if (set_smem_once(rope_norm_bwd_kernel<D, F32>, kSmem, smem_set) != B200ATTN_OK) return;
    unsigned grid = rope_norm_grid(rope_norm_bwd_kernel<D, F32>, rows, (kRopeNormThreads / 32) * kBwdSteps * (256 / D), occ, kSmem);
    grid = std::min(grid, (unsigned)(kRopeNormMaxCtasPerSm * sm_count()));  // the workspace holds that many partial sums
    p0.partial = workspace;
    p1.partial = workspace + (size_t)kRopeNormMaxCtasPerSm * sm_count() * D;
    launch_pdl(rope_norm_bwd_kernel<D, F32>, dim3(grid, 1, 1), kRopeNormThreads, kSmem, st, p0, p1, n_tensors);
    const float* part0 = p0.partial;
    const float* part1 = p1.partial;
    launch_pdl(rope_norm_dgamma_kernel<D>, dim3(n_tensors * D, 1, 1), 32, 0, st, part0, p0.d_gamma, part1, p1.d_gamma,
               (int)grid);
}

void rope_norm_fill(RopeNormParams& p, int B, int T, int H, int D, int x_layout, int y_layout) {
    const Strides sx = strides_for(x_layout, H, T, D), sy = strides_for(y_layout, H, T, D);
    p.B = B;
    p.T = T;
    p.H = H;
    p.x_st = sx.t, p.x_sh = sx.h, p.x_sb = sx.b;
    p.y_st = sy.t, p.y_sh = sy.h, p.y_sb = sy.b;
    p.div_h = fastdiv_make((unsigned)H);
    p.div_t = fastdiv_make((unsigned)T);
}

struct RopeNormTensor {  // what differs between q and k
    const void* x;
    void* y;            // forward: y; backward: d_x
    const void* dy;     // backward only
    float* rstd;
    const float* gamma;
    float* d_gamma;     // backward only
    int H;
};

int rope_norm_run(bool backward, const RopeNormTensor* t, int n_tensors, int x_dtype, int x_layout, int y_layout,
                  const float* cos_t, const float* sin_t, int B, int T, int D, float eps, void* workspace,
                  size_t workspace_bytes, void* stream) {
    RopeNormParams p[2] = {};
    long long rows = 0;
    for (int i = 0; i < n_tensors; ++i) {
        int rc = rope_norm_check(B, T, t[i].H, D, x_dtype, x_layout, y_layout);
        if (rc) return rc;
        if (!t[i].x || !t[i].y || !t[i].rstd || !t[i].gamma || (backward && (!t[i].dy || !t[i].d_gamma)))
            return B200ATTN_ERR_INVALID_ARG;
        if (!aligned16(t[i].x) || !aligned16(t[i].y) || (backward && !aligned16(t[i].dy))) return B200ATTN_ERR_ALIGNMENT;
        rope_norm_fill(p[i], B, T, t[i].H, D, x_layout, y_layout);
        // rows are walked in the order of the tensor that is written (y forward, d_x backward): dense stores
        p[i].walk_bthd = (backward ? x_layout : y_layout) == B200ATTN_LAYOUT_BTHD;
        p[i].x = t[i].x;
        p[i].y = t[i].y;
        p[i].dy = static_cast<const uint16_t*>(t[i].dy);
        p[i].rstd = t[i].rstd;
        p[i].gamma = t[i].gamma;
        p[i].d_gamma = t[i].d_gamma;
        p[i].cos_t = cos_t;
        p[i].sin_t = sin_t;
        p[i].eps = eps;
        rows = std::max(rows, (long long)B * T * t[i].H);
    }
    if (!cos_t || !sin_t) return B200ATTN_ERR_INVALID_ARG;
    if (backward && (!workspace || workspace_bytes < b200attn_rope_norm_bwd_workspace_bytes(D) ||
                     (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0))
        return B200ATTN_ERR_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool f32 = x_dtype == B200ATTN_DTYPE_F32;
    float* ws = static_cast<float*>(workspace);
    if (!backward) {
        if (D == 64) {
            if (f32) rope_norm_launch_fwd<64, true>(p[0], p[1], n_tensors, rows, st);
            else rope_norm_launch_fwd<64, false>(p[0], p[1], n_tensors, rows, st);
        } else {
            if (f32) rope_norm_launch_fwd<128, true>(p[0], p[1], n_tensors, rows, st);
            else rope_norm_launch_fwd<128, false>(p[0], p[1], n_tensors, rows, st);
        }
    } else {
        if (D == 64) {
            if (f32) rope_norm_launch_bwd<64, true>(p[0], p[1], n_tensors, rows, ws, st);
            else rope_norm_launch_bwd<64, false>(p[0], p[1], n_tensors, rows, ws, st);
        } else {
            if (f32) rope_norm_launch_bwd<128, true>(p[0], p[1], n_tensors, rows, ws, st);
            else rope_norm_launch_bwd<128, false>(p[0], p[1], n_tensors, rows, ws, st);
        }
    }
    if (cudaGetLastError() != cudaSuccess) return B200ATTN_ERR_CUDA;
    return B200ATTN_OK;
}

}  // namespace

extern "C" int b200attn_rope_table(int T, int D, float base, float* cos_host, float* sin_host) {
    if (T <= 0 || D <= 0 || (D & 1) || !cos_host || !sin_host || !(base > 0.f)) return B200ATTN_ERR_INVALID_ARG;
    const int half = D / 2;
    // the same single-precision arithmetic as make_rope_cache (llm/src/model/rope.cu:112-128)
    for (int t = 0; t < T; ++t)
        for (int i = 0; i < half; ++i) {
            const float theta = powf(base, -static_cast<float>(2 * i) / static_cast<float>(D));
            const float angle = static_cast<float>(t) * theta;
            cos_host[(size_t)t * half + i] = cosf(angle);
            sin_host[(size_t)t * half + i] = sinf(angle);
        }
    return B200ATTN_OK;
}

extern "C" size_t b200attn_rope_norm_bwd_workspace_bytes(int D) {
    if (D <= 0) return 0;
    return (size_t)2 * kRopeNormMaxCtasPerSm * sm_count() * D * sizeof(float);  // partial sums for up to two tensors
}

extern "C" int b200attn_rope_norm_fwd(const void* x, int x_dtype, int x_layout, void* y, int y_layout, float* rstd,
                                      const float* gamma, const float* cos_t, const float* sin_t, int B, int T, int H,
                                      int D, float eps, void* stream) {
    const RopeNormTensor t = {x, y, nullptr, rstd, gamma, nullptr, H};
    return rope_norm_run(false, &t, 1, x_dtype, x_layout, y_layout, cos_t, sin_t, B, T, D, eps, nullptr, 0, stream);
}

extern "C" int b200attn_rope_norm_bwd(const void* dy, int y_layout, const void* x, int x_dtype, int x_layout,
                                      const float* rstd, const float* gamma, const float* cos_t, const float* sin_t,
                                      void* dx, float* d_gamma, int B, int T, int H, int D, void* workspace,
                                      size_t workspace_bytes, void* stream) {
    const RopeNormTensor t = {x, dx, dy, const_cast<float*>(rstd), gamma, d_gamma, H};
    return rope_norm_run(true, &t, 1, x_dtype, x_layout, y_layout, cos_t, sin_t, B, T, D, 0.f, workspace, workspace_bytes,
                         stream);
}

extern "C" int b200attn_rope_norm_fwd_qk(const void* xq, const void* xk, int x_dtype, int x_layout, void* yq, void* yk,
                                         int y_layout, float* rstd_q, float* rstd_k, const float* gamma_q,
                                         const float* gamma_k, const float* cos_t, const float* sin_t, int B, int T,
                                         int Hq, int Hkv, int D, float eps, void* stream) {
    const RopeNormTensor t[2] = {{xq, yq, nullptr, rstd_q, gamma_q, nullptr, Hq}, {xk, yk, nullptr, rstd_k, gamma_k, nullptr, Hkv}};
    return rope_norm_run(false, t, 2, x_dtype, x_layout, y_layout, cos_t, sin_t, B, T, D, eps, nullptr, 0, stream);
}

extern "C" int b200attn_rope_norm_bwd_qk(const void* dyq, const void* dyk, int y_layout, const void* xq, const void* xk,
                                         int x_dtype, int x_layout, const float* rstd_q, const float* rstd_k,
                                         const float* gamma_q, const float* gamma_k, const float* cos_t,
                                         const float* sin_t, void* dxq, void* dxk, float* d_gamma_q, float* d_gamma_k,
                                         int B, int T, int Hq, int Hkv, int D, void* workspace, size_t workspace_bytes,
                                         void* stream) {
    const RopeNormTensor t[2] = {{xq, dxq, dyq, const_cast<float*>(rstd_q), gamma_q, d_gamma_q, Hq},
                                 {xk, dxk, dyk, const_cast<float*>(rstd_k), gamma_k, d_gamma_k, Hkv}};
    return rope_norm_run(true, t, 2, x_dtype, x_layout, y_layout, cos_t, sin_t, B, T, D, 0.f, workspace, workspace_bytes,
                         stream);
}

extern "C" int b200attn_set_bwd_profile_events4(void* e0, void* e1, void* e2, void* e3) {
    void* ev[4] = {e0, e1, e2, e3};
    const int n_set = (e0 != nullptr) + (e1 != nullptr) + (e2 != nullptr);
    if (n_set != 0 && n_set != 3) return B200ATTN_ERR_INVALID_ARG;
    if (n_set == 0 && e3 != nullptr) return B200ATTN_ERR_INVALID_ARG;
    for (int i = 0; i < 4; ++i) g_bwd_events[i] = static_cast<cudaEvent_t>(ev[i]);
    return B200ATTN_OK;
}

extern "C" int b200attn_set_bwd_profile_events(void* e0, void* e1, void* e2) {
    return b200attn_set_bwd_profile_events4(e0, e1, e2, nullptr);
}

extern "C" size_t b200attn_bwd_workspace_bytes_mode(int B, int T, int Hq, int Hkv, int D, int mode) {
    (void)Hkv;
    if (B <= 0 || T <= 0 || Hq <= 0 || D <= 0) return 0;
    if (mode != B200ATTN_BWD_AUTO && mode != B200ATTN_BWD_TWO_PASS && mode != B200ATTN_BWD_ONE_PASS) return 0;
    if (bwd_resolve_mode(mode, B, T, Hq, D) == B200ATTN_BWD_ONE_PASS) return bwd_vec_bytes_padded(B, T, Hq) + bwd_acc_bytes(B, T, Hq, D);
    return 2 * bwd_vec_elems(B, T, Hq) * sizeof(float);
}

extern "C" size_t b200attn_bwd_workspace_bytes(int B, int T, int Hq, int Hkv, int D) {
    return b200attn_bwd_workspace_bytes_mode(B, T, Hq, Hkv, D, B200ATTN_BWD_AUTO);
}

extern "C" int b200attn_bwd(const void* q, const void* k, const void* v, const void* o, const float* lse,
                            const void* dout, void* dq, void* dk, void* dv, int B, int T, int Hq, int Hkv, int D,
                            int layout, float softmax_scale, void* workspace, size_t workspace_bytes, void* stream) {
    return b200attn_bwd_mode(q, k, v, o, lse, dout, dq, dk, dv, B, T, Hq, Hkv, D, layout, softmax_scale, B200ATTN_BWD_AUTO,
                             workspace, workspace_bytes, stream);
}

extern "C" int b200attn_bwd_mode(const void* q, const void* k, const void* v, const void* o, const float* lse,
                                 const void* dout, void* dq, void* dk, void* dv, int B, int T, int Hq, int Hkv, int D,
                                 int layout, float softmax_scale, int mode, void* workspace, size_t workspace_bytes,
                                 void* stream) {
    int rc = check_common(B, T, Hq, Hkv, D, layout);
    if (rc) return rc;
    if (!q || !k || !v || !o || !lse || !dout || !dq || !dk || !dv) return B200ATTN_ERR_INVALID_ARG;
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o) || !aligned16(dout) || !aligned16(dq) ||
        !aligned16(dk) || !aligned16(dv))
        return B200ATTN_ERR_ALIGNMENT;
    if (mode != B200ATTN_BWD_AUTO && mode != B200ATTN_BWD_TWO_PASS && mode != B200ATTN_BWD_ONE_PASS)
        return B200ATTN_ERR_INVALID_ARG;
    if (mode == B200ATTN_BWD_ONE_PASS && D != 64) return B200ATTN_ERR_UNSUPPORTED;
    const size_t two_pass_bytes = 2 * bwd_vec_elems(B, T, Hq) * sizeof(float);
    const size_t one_pass_bytes = bwd_vec_bytes_padded(B, T, Hq) + bwd_acc_bytes(B, T, Hq, D);
    if (!workspace || workspace_bytes < two_pass_bytes || (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0)
        return B200ATTN_ERR_WORKSPACE;
    // AUTO falls back to the two-pass kernels when the workspace only holds the row vectors
    const bool auto_mode = mode == B200ATTN_BWD_AUTO;
    mode = bwd_resolve_mode(mode, B, T, Hq, D);
    if (mode == B200ATTN_BWD_ONE_PASS && workspace_bytes < one_pass_bytes) {
        if (!auto_mode) return B200ATTN_ERR_WORKSPACE;
        mode = B200ATTN_BWD_TWO_PASS;
    }
    int* status = status_ptr(&rc);
    if (!status) return rc;
    const Strides sq = strides_for(layout, Hq, T, D), sk = strides_for(layout, Hkv, T, D);
    CUtensorMap tq, tk, tv, tk64, tv64, tdo, to, tdq, tdk, tdv;
    if (!make_tmap_bf16_4d(&tq, q, D, T, Hq, B, sq.t, sq.h, sq.b, 128) ||
        !make_tmap_bf16_4d(&tk, k, D, T, Hkv, B, sk.t, sk.h, sk.b, 128) ||
        !make_tmap_bf16_4d(&tv, v, D, T, Hkv, B, sk.t, sk.h, sk.b, 128) ||
        !make_tmap_bf16_4d(&tk64, k, D, T, Hkv, B, sk.t, sk.h, sk.b, 64) ||
        !make_tmap_bf16_4d(&tv64, v, D, T, Hkv, B, sk.t, sk.h, sk.b, 64) ||
        !make_tmap_bf16_4d(&tdo, dout, D, T, Hq, B, sq.t, sq.h, sq.b, 128) ||
        !make_tmap_bf16_4d(&to, o, D, T, Hq, B, sq.t, sq.h, sq.b, 128) ||
        !make_tmap_bf16_4d(&tdq, dq, D, T, Hq, B, sq.t, sq.h, sq.b, 128) ||
        !make_tmap_bf16_4d(&tdk, dk, D, T, Hkv, B, sk.t, sk.h, sk.b, 128) ||
        !make_tmap_bf16_4d(&tdv, dv, D, T, Hkv, B, sk.t, sk.h, sk.b, 128))
        return B200ATTN_ERR_TENSOR_MAP;
    float* ws = static_cast<float*>(workspace);
    const size_t nvec = bwd_vec_elems(B, T, Hq);
    BwdParams p;
    p.B = B;
    p.T = T;
    p.Tpad = (T + 127) / 128 * 128;
    p.Hq = Hq;
    p.Hkv = Hkv;
    p.group = Hq / Hkv;
    p.n_tiles = (T + 127) / 128;
    p.scale = softmax_scale > 0.f ? softmax_scale : 1.f / sqrtf((float)D);
    p.scale_log2 = p.scale * 1.4426950408889634f;
    p.lse2 = ws;
    p.dvec = ws + nvec;
    p.lse2_w = ws;
    p.dvec_w = ws + nvec;
    p.lse = lse;
    p.o = static_cast<const uint16_t*>(o);
    p.dout = static_cast<const uint16_t*>(dout);
    p.dq = static_cast<uint16_t*>(dq);
    p.q_st = sq.t;
    p.q_sh = sq.h;
    p.q_sb = sq.b;
    p.dk = static_cast<uint16_t*>(dk);
    p.dv = static_cast<uint16_t*>(dv);
    p.k_st = sk.t;
    p.k_sh = sk.h;
    p.k_sb = sk.b;
    p.status = status;
    p.sched = nullptr;
    p.sched2 = nullptr;
    p.div_bhq = fastdiv_make((unsigned)(B * Hq));
    p.div_hq = fastdiv_make((unsigned)Hq);
    p.div_bhkv = fastdiv_make((unsigned)(B * Hkv));
    p.div_hkv = fastdiv_make((unsigned)Hkv);
    p.div_group = fastdiv_make((unsigned)p.group);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (mode == B200ATTN_BWD_ONE_PASS) {
        float* dq_acc = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + bwd_vec_bytes_padded(B, T, Hq));
        return launch_bwd_onepass(tq, tk, tv, tdo, p, dq_acc, st);
    }
    return D == 64 ? launch_bwd<64>(tq, tk64, tv64, tk, tv, tdo, to, tdq, tdk, tdv, p, st)
                   : launch_bwd<128>(tq, tk64, tv64, tk, tv, tdo, to, tdq, tdk, tdv, p, st);
}

// ---------------------------------------------------------------------------------------
// Backward with its scratch in the library's own device image: no allocation anywhere.
// ---------------------------------------------------------------------------------------
namespace {

// Two FP32 vectors of B200ATTN_BWD_STATIC_MAX_ROWS rows (logsumexp * log2(e) and rowsum(O * dO)).
// In host code this name is only a handle for cudaGetSymbolAddress, never a device pointer.
static __device__ __align__(256) float g_bwd_static_scratch[2 * B200ATTN_BWD_STATIC_MAX_ROWS];

float* g_bwd_static_ptr[kMaxDevices] = {nullptr};

// Device address of the array on the current device, resolved once per device.
float* bwd_static_scratch(int* err) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        *err = B200ATTN_ERR_NO_DEVICE;
        return nullptr;
    }
    if (!g_bwd_static_ptr[dev]) {
        float* ptr = nullptr;
        if (cudaGetSymbolAddress((void**)&ptr, g_bwd_static_scratch) != cudaSuccess || ptr == nullptr) {
            cudaGetLastError();
            *err = B200ATTN_ERR_CUDA;
            return nullptr;
        }
        g_bwd_static_ptr[dev] = ptr;
    }
    return g_bwd_static_ptr[dev];
}

}  // namespace

extern "C" int b200attn_bwd_static(const void* q, const void* k, const void* v, const void* o, const float* lse,
                                   const void* dout, void* dq, void* dk, void* dv, int B, int T, int Hq, int Hkv, int D,
                                   int layout, float softmax_scale, void* stream) {
    int rc = check_common(B, T, Hq, Hkv, D, layout);
    if (rc) return rc;
    if (bwd_vec_elems(B, T, Hq) > (size_t)B200ATTN_BWD_STATIC_MAX_ROWS) return B200ATTN_ERR_TOO_LARGE;
    float* scratch = bwd_static_scratch(&rc);
    if (!scratch) return rc;
    // Same kernels as b200attn_bwd; the preprocess kernel rewrites every row (padding included) that
    // the two passes read, so stale contents of an earlier call are never seen.
    return b200attn_bwd_mode(q, k, v, o, lse, dout, dq, dk, dv, B, T, Hq, Hkv, D, layout, softmax_scale,
                             B200ATTN_BWD_TWO_PASS, scratch, 2 * sizeof(float) * (size_t)B200ATTN_BWD_STATIC_MAX_ROWS, stream);
}

namespace {

// Query heads served per decode CTA: the largest divisor of the group size that is <= 16
// (the row count of the kernel's MMA shape).
inline int decode_heads_per_cta(int group) {
    for (int g = 16; g >= 1; --g)
        if (group % g == 0) return g;
    return 1;
}

inline int decode_pick_splits(int B, int L, int Hq, int Hkv, int n_splits) {
    const int n_all = (L + 127) / 128;
    if (n_splits <= 0) {
        const int group = Hq / Hkv;
        const long long units = (long long)B * Hkv * (group / decode_heads_per_cta(group));
        // two CTAs fit on an SM: fill the 2 x 148 slots of the part once, and do not split further
        // (every extra split costs a partial write, a combine read and a shorter stream per CTA)
        long long want = (2 * 148) / units;
        n_splits = (int)(want < 1 ? 1 : want);
    }
    if (n_splits > n_all) n_splits = n_all;
    if (n_splits > 64) n_splits = 64;
    const int tps = (n_all + n_splits - 1) / n_splits;
    return (n_all + tps - 1) / tps;  // drop splits that would be empty
}

template <int D>
int launch_decode(const CUtensorMap& tk, const CUtensorMap& tv, const DecodeParams& p, cudaStream_t st) {
    using Cfg = DecodeCfg<D>;
    static bool set[kMaxDevices] = {false};
    int rc = set_smem_once(attn_decode_kernel<D>, Cfg::kSmemBytes, set);
    if (rc) return rc;
    if (launch_pdl(attn_decode_kernel<D>, dim3(p.n_splits, p.Hkv * p.n_chunks, p.B), 160, Cfg::kSmemBytes, st, tk, tv,
                   p) != cudaSuccess) {
        cudaGetLastError();
        return B200ATTN_ERR_CUDA;
    }
    return B200ATTN_OK;
}

}  // namespace

extern "C" int b200attn_decode_default_splits(int B, int L, int Hq, int Hkv, int D) {
    (void)D;
    if (B <= 0 || L <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv != 0) return 0;
    return decode_pick_splits(B, L, Hq, Hkv, 0);
}

extern "C" size_t b200attn_decode_workspace_bytes(int B, int L, int Hq, int Hkv, int D, int n_splits) {
    if (B <= 0 || L <= 0 || Hq <= 0 || Hkv <= 0 || D <= 0 || Hq % Hkv != 0) return 0;
    const int s = decode_pick_splits(B, L, Hq, Hkv, n_splits);
    return (size_t)B * Hq * s * (size_t)(D + 2) * sizeof(float);
}

extern "C" int b200attn_decode(const void* q, const void* kcache, const void* vcache, void* o, float* lse, int B, int L,
                               int Hq, int Hkv, int D, float softmax_scale, int n_splits, void* workspace,
                               size_t workspace_bytes, void* stream) {
    return b200attn_decode_cached(q, kcache, vcache, o, lse, B, L, L, Hq, Hkv, D, softmax_scale, n_splits, workspace,
                                  workspace_bytes, stream);
}

extern "C" int b200attn_decode_cached(const void* q, const void* kcache, const void* vcache, void* o, float* lse, int B,
                                      int L, int L_cap, int Hq, int Hkv, int D, float softmax_scale, int n_splits,
                                      void* workspace, size_t workspace_bytes, void* stream) {
    return b200attn_decode_ragged(q, kcache, vcache, o, lse, nullptr, B, L, L_cap, Hq, Hkv, D, softmax_scale, n_splits,
                                  workspace, workspace_bytes, stream);
}

extern "C" int b200attn_decode_ragged(const void* q, const void* kcache, const void* vcache, void* o, float* lse,
                                      const int* lens, int B, int L, int L_cap, int Hq, int Hkv, int D,
                                      float softmax_scale, int n_splits, void* workspace, size_t workspace_bytes,
                                      void* stream) {
    int rc = check_common(B, L, Hq, Hkv, D, B200ATTN_LAYOUT_BHTD);
    if (rc) return rc;
    if (L_cap < L) return B200ATTN_ERR_INVALID_ARG;
    if (!q || !kcache || !vcache || !o) return B200ATTN_ERR_INVALID_ARG;
    if (!aligned16(q) || !aligned16(kcache) || !aligned16(vcache) || !aligned16(o)) return B200ATTN_ERR_ALIGNMENT;
    if (!workspace || workspace_bytes < b200attn_decode_workspace_bytes(B, L, Hq, Hkv, D, n_splits) ||
        (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0)
        return B200ATTN_ERR_WORKSPACE;
    int* status = status_ptr(&rc);
    if (!status) return rc;
    // the maps end at row L of every (batch, head): rows of the cache beyond it are never read (TMA fills zeros)
    const Strides sk = strides_for(B200ATTN_LAYOUT_BHTD, Hkv, L_cap, D);
    CUtensorMap tk, tv;
    if (!make_tmap_bf16_4d(&tk, kcache, D, L, Hkv, B, sk.t, sk.h, sk.b, 128) ||
        !make_tmap_bf16_4d(&tv, vcache, D, L, Hkv, B, sk.t, sk.h, sk.b, 128))
        return B200ATTN_ERR_TENSOR_MAP;
    DecodeParams p;
    p.B = B;
    p.L = L;
    p.Hq = Hq;
    p.Hkv = Hkv;
    p.group = Hq / Hkv;
    p.G = decode_heads_per_cta(p.group);
    p.n_chunks = p.group / p.G;
    p.n_splits = decode_pick_splits(B, L, Hq, Hkv, n_splits);
    p.tiles_per_split = ((L + 127) / 128 + p.n_splits - 1) / p.n_splits;
    p.scale = softmax_scale > 0.f ? softmax_scale : 1.f / sqrtf((float)D);
    p.scale_log2 = p.scale * 1.4426950408889634f;
    p.q = static_cast<const uint16_t*>(q);
    p.lens = lens;
    float* ws = static_cast<float*>(workspace);
    const size_t rows = (size_t)B * Hq;
    p.part_o = ws;
    p.part_m = ws + rows * p.n_splits * D;
    p.part_l = p.part_m + rows * p.n_splits;
    p.status = status;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    rc = D == 64 ? launch_decode<64>(tk, tv, p, st) : launch_decode<128>(tk, tv, p, st);
    if (rc) return rc;
    const dim3 blocks((unsigned)((rows + 3) / 4), 1, 1);
    const float* po = p.part_o;
    const float* pm = p.part_m;
    const float* pl = p.part_l;
    uint16_t* o16 = static_cast<uint16_t*>(o);
    const cudaError_t e =
        D == 64 ? launch_pdl(attn_decode_combine_kernel<64>, blocks, 128, 0, st, po, pm, pl, o16, lse, (int)rows,
                             p.n_splits, p.scale, p.scale_log2)
                : launch_pdl(attn_decode_combine_kernel<128>, blocks, 128, 0, st, po, pm, pl, o16, lse, (int)rows,
                             p.n_splits, p.scale, p.scale_log2);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return B200ATTN_ERR_CUDA;
    }
    return B200ATTN_OK;
}

namespace {

template <int D, bool F32>
int launch_kv_append(const KvAppendParams& p, cudaStream_t st) {
    const long long rows = (long long)p.rows_q + 2LL * p.rows_kv;
    const long long rows_per_cta = (kKvAppendThreads / 32) * (256 / D);
    long long grid = (rows + rows_per_cta - 1) / rows_per_cta;
    const long long cap = 8LL * sm_count();  // 8 CTAs of 256 threads are resident per SM
    if (grid > cap) grid = cap;
    if (launch_pdl(kv_append_kernel<D, F32>, dim3((unsigned)grid, 1, 1), kKvAppendThreads, 0, st, p) != cudaSuccess) {
        cudaGetLastError();
        return B200ATTN_ERR_CUDA;
    }
    return B200ATTN_OK;
}

}  // namespace

namespace {
int kv_append_run(const void* xq, const void* xk, const void* xv, int x_dtype, void* q_out, void* kcache, void* vcache,
                  const float* gamma_q, const float* gamma_k, const float* cos_t, const float* sin_t, const int* pos,
                  int B, int n_new, int pos0, int L_cap, int Hq, int Hkv, int D, float eps, void* stream);
}

extern "C" int b200attn_kv_append(const void* xq, const void* xk, const void* xv, int x_dtype, void* q_out, void* kcache,
                                  void* vcache, const float* gamma_q, const float* gamma_k, const float* cos_t,
                                  const float* sin_t, int B, int n_new, int pos0, int L_cap, int Hq, int Hkv, int D,
                                  float eps, void* stream) {
    return kv_append_run(xq, xk, xv, x_dtype, q_out, kcache, vcache, gamma_q, gamma_k, cos_t, sin_t, nullptr, B, n_new, pos0,
                         L_cap, Hq, Hkv, D, eps, stream);
}

extern "C" int b200attn_kv_append_at(const void* xq, const void* xk, const void* xv, int x_dtype, void* q_out, void* kcache,
                                     void* vcache, const float* gamma_q, const float* gamma_k, const float* cos_t,
                                     const float* sin_t, const int* pos, int B, int n_new, int L_cap, int Hq, int Hkv,
                                     int D, float eps, void* stream) {
    if (!pos) return B200ATTN_ERR_INVALID_ARG;
    return kv_append_run(xq, xk, xv, x_dtype, q_out, kcache, vcache, gamma_q, gamma_k, cos_t, sin_t, pos, B, n_new, 0, L_cap,
                         Hq, Hkv, D, eps, stream);
}

namespace {
int kv_append_run(const void* xq, const void* xk, const void* xv, int x_dtype, void* q_out, void* kcache, void* vcache,
                  const float* gamma_q, const float* gamma_k, const float* cos_t, const float* sin_t, const int* pos,
                  int B, int n_new, int pos0, int L_cap, int Hq, int Hkv, int D, float eps, void* stream) {
    if (B <= 0 || n_new <= 0 || pos0 < 0 || L_cap <= 0 || Hq <= 0 || Hkv <= 0 || D <= 0) return B200ATTN_ERR_INVALID_ARG;
    if (Hq % Hkv != 0 || (long long)pos0 + n_new > L_cap) return B200ATTN_ERR_INVALID_ARG;
    if (x_dtype != B200ATTN_DTYPE_BF16 && x_dtype != B200ATTN_DTYPE_F32) return B200ATTN_ERR_INVALID_ARG;
    if (D != 64 && D != 128) return B200ATTN_ERR_UNSUPPORTED;
    if (!xq || !xk || !xv || !q_out || !kcache || !vcache || !gamma_q || !gamma_k || !cos_t || !sin_t)
        return B200ATTN_ERR_INVALID_ARG;
    if (!aligned16(xq) || !aligned16(xk) || !aligned16(xv) || !aligned16(q_out) || !aligned16(kcache) ||
        !aligned16(vcache) || !aligned16(gamma_q) || !aligned16(gamma_k) || !aligned16(cos_t) || !aligned16(sin_t))
        return B200ATTN_ERR_ALIGNMENT;
    const long long rows_q = (long long)B * n_new * Hq, rows_kv = (long long)B * n_new * Hkv;
    if (rows_q + 2 * rows_kv >= (1LL << 31)) return B200ATTN_ERR_TOO_LARGE;
    int rc = 0;
    int* status = status_ptr(&rc);
    if (!status) return rc;
    KvAppendParams p;
    p.pos = pos;
    p.status = status;
    p.xq = xq;
    p.xk = xk;
    p.xv = xv;
    p.q_out = static_cast<uint16_t*>(q_out);
    p.kcache = static_cast<uint16_t*>(kcache);
    p.vcache = static_cast<uint16_t*>(vcache);
    p.gamma_q = gamma_q;
    p.gamma_k = gamma_k;
    p.cos_t = cos_t;
    p.sin_t = sin_t;
    p.B = B;
    p.n_new = n_new;
    p.pos0 = pos0;
    p.L_cap = L_cap;
    p.Hq = Hq;
    p.Hkv = Hkv;
    p.rows_q = (unsigned)rows_q;
    p.rows_kv = (unsigned)rows_kv;
    p.div_hq = fastdiv_make((unsigned)Hq);
    p.div_hkv = fastdiv_make((unsigned)Hkv);
    p.div_n = fastdiv_make((unsigned)n_new);
    p.eps = eps;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool f32 = x_dtype == B200ATTN_DTYPE_F32;
    if (D == 64) return f32 ? launch_kv_append<64, true>(p, st) : launch_kv_append<64, false>(p, st);
    return f32 ? launch_kv_append<128, true>(p, st) : launch_kv_append<128, false>(p, st);
}
}  // namespace

extern "C" int b200attn_item_deal(int n_groups, int n_qtiles, int T, int n_ctas, int item_cost, unsigned short* ids,
                                  int* per_cta) {
    if (n_groups <= 0 || n_qtiles <= 0 || T <= 0 || n_ctas <= 0 || item_cost < 0 || !ids || !per_cta)
        return B200ATTN_ERR_INVALID_ARG;
    const ItemTable& tab = item_table_for((long long)n_groups * n_qtiles, (unsigned)n_ctas, n_groups, n_qtiles, T, item_cost);
    *per_cta = tab.per_cta;
    for (int i = 0; i < n_ctas * tab.per_cta; ++i) ids[i] = tab.ids[i];
    return B200ATTN_OK;
}

extern "C" int b200attn_last_device_status(void* stream) {
    int rc = 0;
    int* status = status_ptr(&rc);
    if (!status) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (cudaStreamSynchronize(st) != cudaSuccess) {
        cudaGetLastError();
        return B200ATTN_ERR_CUDA;
    }
    int host = 0;
    if (cudaMemcpy(&host, status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return B200ATTN_ERR_CUDA;
    if (host != 0) {
        // a kernel that gave up may have left its item counters behind: wait for everything else on the
        // device (kernels exit at once while the status word is set), then clear counters and status
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceSynchronize();
        cudaMemset(g_sched_ptr[dev], 0, sizeof(int) * 2 * kSchedSlots);
        cudaMemset(status, 0, sizeof(int));
        return host;
    }
    return B200ATTN_OK;
}

extern "C" const char* b200attn_strerror(int status) {
    switch (status) {
        case B200ATTN_OK: return "ok";
        case B200ATTN_ERR_INVALID_ARG: return "invalid argument (null pointer, non-positive size, Hq % Hkv != 0 or bad layout)";
        case B200ATTN_ERR_UNSUPPORTED: return "unsupported head dimension (only 64 and 128)";
        case B200ATTN_ERR_ALIGNMENT: return "a base pointer is not 16-byte aligned";
        case B200ATTN_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
        case B200ATTN_ERR_CUDA: return "a CUDA runtime call or kernel launch failed";
        case B200ATTN_ERR_TENSOR_MAP: return "the driver refused a TMA tensor map";
        case B200ATTN_ERR_DEVICE_WAIT: return "a kernel gave up on a bounded wait";
        case B200ATTN_ERR_NO_DEVICE: return "no usable CUDA device is current";
        case B200ATTN_ERR_TOO_LARGE:
            return "problem too large: beyond the fixed scratch of b200attn_bwd_static (B*Hq*ceil(T/128)*128 > 524288), or "
                   "2^31 or more rows in a RoPE / QK-Norm / KV-append call";
        case DEV_WAIT_TIMEOUT_LOAD: return "device: a TMA load barrier never completed";
        case DEV_WAIT_TIMEOUT_MMA: return "device: a tensor-core completion barrier never completed";
        case DEV_WAIT_TIMEOUT_SOFTMAX: return "device: a softmax hand-off barrier never completed";
        case DEV_WAIT_TIMEOUT_FREE: return "device: a buffer-free barrier never completed";
        case DEV_KV_CACHE_OVERFLOW: return "device: a KV-cache position plus the new tokens exceeds the cache capacity";
        default: return "unknown status";
    }
}

extern "C" int b200attn_version(void) { return 1; }

#ifdef B200ATTN_PROBE
// Tuning builds only: copies the phase timestamps of the last launch to the host.
extern "C" int b200attn_debug_read_probe(long long* host, int n) {
    if (n > 512) n = 512;
    return cudaMemcpyFromSymbol(host, b200attn::g_probe, sizeof(long long) * n) == cudaSuccess ? 0 : B200ATTN_ERR_CUDA;
}
extern "C" int b200attn_debug_read_trace(unsigned long long* host, int n_ctas) {
    if (n_ctas > 8192) n_ctas = 8192;
    return cudaMemcpyFromSymbol(host, b200attn::g_trace, sizeof(unsigned long long) * 3 * n_ctas) == cudaSuccess
               ? 0 : B200ATTN_ERR_CUDA;
}
extern "C" int b200attn_debug_read_trace_clk(long long* host, int n_ctas) {
    if (n_ctas > 8192) n_ctas = 8192;
    return cudaMemcpyFromSymbol(host, b200attn::g_trace_clk, sizeof(long long) * 2 * n_ctas) == cudaSuccess
               ? 0 : B200ATTN_ERR_CUDA;
}
#endif
