// See modernllm_shim.h.  Compiled inside the reference tree; links libb200attn.so.
#include "modernllm_shim.h"

#include <cuda_runtime.h>

#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

#include "b200attn.h"

namespace modernllm {
namespace b200 {

namespace {

void check(const Tensor& t, DType want, const char* fn, const char* name) {
    if (t.dtype() != want)
        throw std::invalid_argument(std::string(fn) + ": " + name + (want == DType::BF16 ? " must be BF16" : " must be FP32"));
}
void check_cuda(const Tensor& t, const char* fn, const char* name) {
    if (t.device() != Device::Cuda) throw std::invalid_argument(std::string(fn) + ": " + name + " must be CUDA");
}

void raise(int status, const char* fn) {
    if (status == B200ATTN_OK) return;
    std::string msg = std::string(fn) + ": " + b200attn_strerror(status);
    if (status == B200ATTN_ERR_INVALID_ARG || status == B200ATTN_ERR_UNSUPPORTED ||
        status == B200ATTN_ERR_ALIGNMENT || status == B200ATTN_ERR_WORKSPACE || status == B200ATTN_ERR_TOO_LARGE)
        throw std::invalid_argument(msg);
    throw std::runtime_error(msg);
}

// A private temporary that is kept between calls: one per (device, stream, operator), grown when a larger problem
// comes and never shrunk.  Growing frees the old buffer, and cudaFree waits for the work that still reads it.
enum WsKind { kWsBackward = 0, kWsDecode = 1, kWsRopeNorm = 2 };
struct WsEntry {
    int device;
    void* stream;
    int kind;
    Tensor buf;
};
void* cached_workspace(int kind, size_t bytes, void* stream) {
    static std::mutex mu;
    static std::vector<WsEntry> cache;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) throw std::runtime_error("cached_workspace: no current CUDA device");
    std::lock_guard<std::mutex> lock(mu);
    for (WsEntry& e : cache) {
        if (e.device == dev && e.stream == stream && e.kind == kind) {
            if (e.buf.bytes() < bytes) e.buf = Tensor({static_cast<std::int64_t>((bytes + 3) / 4)}, DType::FP32, Device::Cuda);
            return e.buf.data();
        }
    }
    cache.push_back(WsEntry{dev, stream, kind, Tensor({static_cast<std::int64_t>((bytes + 1023) / 4)}, DType::FP32, Device::Cuda)});
    return cache.back().buf.data();
}

}  // namespace

void flash_attn_forward_gqa(const Tensor& q, const Tensor& k, const Tensor& v, Tensor& ctx, Tensor& L, int B, int T,
                            int Hq, int Hkv, int D, Layout layout, void* stream) {
    const char* fn = "flash_attn_forward";
    check(q, DType::BF16, fn, "q"); check(k, DType::BF16, fn, "k"); check(v, DType::BF16, fn, "v");
    check(ctx, DType::BF16, fn, "ctx"); check(L, DType::FP32, fn, "L");
    check_cuda(q, fn, "q"); check_cuda(k, fn, "k"); check_cuda(v, fn, "v"); check_cuda(ctx, fn, "ctx");
    check_cuda(L, fn, "L");
    const long long nq = 1LL * B * Hq * T * D, nkv = 1LL * B * Hkv * T * D;
    if (q.numel() != nq || ctx.numel() != nq || k.numel() != nkv || v.numel() != nkv)
        throw std::invalid_argument("flash_attn_forward: shape mismatch (qkv/ctx)");
    if (L.numel() != 1LL * B * Hq * T) throw std::invalid_argument("flash_attn_forward: L must be [B, T]");
    raise(b200attn_fwd(q.data(), k.data(), v.data(), ctx.data(), L.data_as<float>(), B, T, Hq, Hkv, D,
                       static_cast<int>(layout), 0.f, stream),
          fn);
}

void flash_attn_backward_gqa(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& ctx, const Tensor& L,
                             const Tensor& d_ctx, Tensor& d_q, Tensor& d_k, Tensor& d_v, int B, int T, int Hq,
                             int Hkv, int D, Layout layout, void* stream) {
    const char* fn = "flash_attn_backward";
    const Tensor* bf[] = {&q, &k, &v, &ctx, &d_ctx, &d_q, &d_k, &d_v};
    const char* names[] = {"q", "k", "v", "ctx", "d_ctx", "d_q", "d_k", "d_v"};
    for (int i = 0; i < 8; ++i) {
        check(*bf[i], DType::BF16, fn, names[i]);
        check_cuda(*bf[i], fn, names[i]);
    }
    check(L, DType::FP32, fn, "L");
    check_cuda(L, fn, "L");
    const long long nq = 1LL * B * Hq * T * D, nkv = 1LL * B * Hkv * T * D;
    if (q.numel() != nq || ctx.numel() != nq || d_ctx.numel() != nq || d_q.numel() != nq || k.numel() != nkv ||
        v.numel() != nkv || d_k.numel() != nkv || d_v.numel() != nkv)
        throw std::invalid_argument("flash_attn_backward: shape mismatch");
    if (L.numel() != 1LL * B * Hq * T) throw std::invalid_argument("flash_attn_backward: L must be [B, T]");
    // Private temporary (the reference's Dh, llm/src/model/flash_attn.cu:463, is a cudaMalloc per call).  On the
    // legacy default stream - where the reference launches and where calls cannot overlap - the library's fixed
    // scratch serves every problem that fits it; otherwise a workspace kept for this (device, stream).
    const long long rows = 1LL * B * Hq * ((T + 127) / 128 * 128);
    if (stream == nullptr && rows <= B200ATTN_BWD_STATIC_MAX_ROWS) {
        raise(b200attn_bwd_static(q.data(), k.data(), v.data(), ctx.data(), L.data_as<float>(), d_ctx.data(), d_q.data(),
                                  d_k.data(), d_v.data(), B, T, Hq, Hkv, D, static_cast<int>(layout), 0.f, stream),
              fn);
        return;
    }
    const size_t ws_bytes = b200attn_bwd_workspace_bytes_mode(B, T, Hq, Hkv, D, B200ATTN_BWD_TWO_PASS);
    raise(b200attn_bwd_mode(q.data(), k.data(), v.data(), ctx.data(), L.data_as<float>(), d_ctx.data(), d_q.data(),
                            d_k.data(), d_v.data(), B, T, Hq, Hkv, D, static_cast<int>(layout), 0.f, B200ATTN_BWD_TWO_PASS,
                            cached_workspace(kWsBackward, ws_bytes, stream), ws_bytes, stream),
          fn);
}

void flash_attn_forward(const Tensor& q, const Tensor& k, const Tensor& v, Tensor& ctx, Tensor& L, int B, int T, int D,
                        int tile_kv, void* stream) {
    if (tile_kv <= 0) throw std::invalid_argument("flash_attn_forward: tile_kv must be > 0");
    flash_attn_forward_gqa(q, k, v, ctx, L, B, T, 1, 1, D, Layout::BHTD, stream);
}

void flash_attn_backward(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& ctx, const Tensor& L,
                         const Tensor& d_ctx, Tensor& d_q, Tensor& d_k, Tensor& d_v, int B, int T, int D, int tile,
                         void* stream) {
    if (tile <= 0) throw std::invalid_argument("flash_attn_backward: tile must be > 0");
    flash_attn_backward_gqa(q, k, v, ctx, L, d_ctx, d_q, d_k, d_v, B, T, 1, 1, D, Layout::BHTD, stream);
}

void flash_attn_decode(const Tensor& q, const Tensor& kcache, const Tensor& vcache, Tensor& o, int B, int Lcache,
                       int Hq, int Hkv, int D, void* stream) {
    const char* fn = "flash_attn_decode";
    check(q, DType::BF16, fn, "q"); check(kcache, DType::BF16, fn, "kcache"); check(vcache, DType::BF16, fn, "vcache");
    check(o, DType::BF16, fn, "o");
    check_cuda(q, fn, "q"); check_cuda(kcache, fn, "kcache"); check_cuda(vcache, fn, "vcache"); check_cuda(o, fn, "o");
    if (q.numel() != 1LL * B * Hq * D || o.numel() != q.numel() || kcache.numel() != 1LL * B * Hkv * Lcache * D ||
        vcache.numel() != kcache.numel())
        throw std::invalid_argument("flash_attn_decode: shape mismatch");
    const size_t ws_bytes = b200attn_decode_workspace_bytes(B, Lcache, Hq, Hkv, D, 0);
    raise(b200attn_decode(q.data(), kcache.data(), vcache.data(), o.data(), nullptr, B, Lcache, Hq, Hkv, D, 0.f, 0,
                          cached_workspace(kWsDecode, ws_bytes, stream), ws_bytes, stream),
          fn);
}

namespace {
int x_dtype_of(const Tensor& x, const char* fn) {
    if (x.dtype() == DType::BF16) return B200ATTN_DTYPE_BF16;
    if (x.dtype() == DType::FP32) return B200ATTN_DTYPE_F32;
    throw std::invalid_argument(std::string(fn) + ": x must be FP32 or BF16");
}
}  // namespace

void rope_qknorm_forward(const Tensor& x, const Tensor& cos, const Tensor& sin, const Tensor& gamma, float eps, Tensor& y,
                         Tensor& rstd, int B, int T, int H, int d_h, Layout x_layout, Layout y_layout, void* stream) {
    const char* fn = "rope_qknorm_forward";
    const int xd = x_dtype_of(x, fn);
    check(y, DType::BF16, fn, "y"); check(cos, DType::FP32, fn, "cos"); check(sin, DType::FP32, fn, "sin");
    check(gamma, DType::FP32, fn, "gamma"); check(rstd, DType::FP32, fn, "rstd");
    check_cuda(x, fn, "x"); check_cuda(y, fn, "y"); check_cuda(cos, fn, "cos"); check_cuda(sin, fn, "sin");
    check_cuda(gamma, fn, "gamma"); check_cuda(rstd, fn, "rstd");
    if (d_h % 2 != 0) throw std::invalid_argument("rope: d_h must be even");
    if (x.numel() != 1LL * B * T * H * d_h || y.numel() != x.numel()) throw std::invalid_argument("rope: x numel mismatch");
    if (gamma.numel() != d_h || rstd.numel() != 1LL * B * H * T || cos.numel() < 1LL * T * (d_h / 2) ||
        sin.numel() < 1LL * T * (d_h / 2))
        throw std::invalid_argument("rope_qknorm_forward: shape mismatch (gamma/rstd/cos/sin)");
    raise(b200attn_rope_norm_fwd(x.data(), xd, static_cast<int>(x_layout), y.data(), static_cast<int>(y_layout),
                                 static_cast<float*>(rstd.data()), static_cast<const float*>(gamma.data()),
                                 static_cast<const float*>(cos.data()), static_cast<const float*>(sin.data()), B, T, H, d_h,
                                 eps, stream),
          fn);
}

void rope_qknorm_backward(const Tensor& d_y, const Tensor& x, const Tensor& cos, const Tensor& sin, const Tensor& gamma,
                          const Tensor& rstd, Tensor& d_x, Tensor& d_gamma, int B, int T, int H, int d_h, Layout x_layout,
                          Layout y_layout, void* stream) {
    const char* fn = "rope_qknorm_backward";
    const int xd = x_dtype_of(x, fn);
    check(d_y, DType::BF16, fn, "d_y"); check(d_x, x.dtype(), fn, "d_x"); check(cos, DType::FP32, fn, "cos");
    check(sin, DType::FP32, fn, "sin"); check(gamma, DType::FP32, fn, "gamma"); check(rstd, DType::FP32, fn, "rstd");
    check(d_gamma, DType::FP32, fn, "d_gamma");
    check_cuda(d_y, fn, "d_y"); check_cuda(x, fn, "x"); check_cuda(d_x, fn, "d_x"); check_cuda(cos, fn, "cos");
    check_cuda(sin, fn, "sin"); check_cuda(gamma, fn, "gamma"); check_cuda(rstd, fn, "rstd"); check_cuda(d_gamma, fn, "d_gamma");
    if (d_h % 2 != 0) throw std::invalid_argument("rope: d_h must be even");
    if (x.numel() != 1LL * B * T * H * d_h || d_y.numel() != x.numel() || d_x.numel() != x.numel())
        throw std::invalid_argument("rope: x numel mismatch");
    if (gamma.numel() != d_h || d_gamma.numel() != d_h || rstd.numel() != 1LL * B * H * T)
        throw std::invalid_argument("rope_qknorm_backward: shape mismatch (gamma/d_gamma/rstd)");
    const size_t ws_bytes = b200attn_rope_norm_bwd_workspace_bytes(d_h);
    raise(b200attn_rope_norm_bwd(d_y.data(), static_cast<int>(y_layout), x.data(), xd, static_cast<int>(x_layout),
                                 static_cast<const float*>(rstd.data()), static_cast<const float*>(gamma.data()),
                                 static_cast<const float*>(cos.data()), static_cast<const float*>(sin.data()), d_x.data(),
                                 static_cast<float*>(d_gamma.data()), B, T, H, d_h,
                                 cached_workspace(kWsRopeNorm, ws_bytes, stream), ws_bytes, stream),
          fn);
}

void kv_cache_append(const Tensor& q_proj, const Tensor& k_proj, const Tensor& v_proj, const Tensor& cos, const Tensor& sin,
                     const Tensor& gamma_q, const Tensor& gamma_k, float eps, Tensor& q_out, Tensor& kcache, Tensor& vcache,
                     int B, int n_new, int pos0, int L_cap, int Hq, int Hkv, int d_h, void* stream) {
    const char* fn = "kv_cache_append";
    const int xd = x_dtype_of(q_proj, fn);
    check(k_proj, q_proj.dtype(), fn, "k_proj"); check(v_proj, q_proj.dtype(), fn, "v_proj");
    check(q_out, DType::BF16, fn, "q_out"); check(kcache, DType::BF16, fn, "kcache"); check(vcache, DType::BF16, fn, "vcache");
    check(cos, DType::FP32, fn, "cos"); check(sin, DType::FP32, fn, "sin");
    check(gamma_q, DType::FP32, fn, "gamma_q"); check(gamma_k, DType::FP32, fn, "gamma_k");
    check_cuda(q_proj, fn, "q_proj"); check_cuda(k_proj, fn, "k_proj"); check_cuda(v_proj, fn, "v_proj");
    check_cuda(q_out, fn, "q_out"); check_cuda(kcache, fn, "kcache"); check_cuda(vcache, fn, "vcache");
    check_cuda(cos, fn, "cos"); check_cuda(sin, fn, "sin"); check_cuda(gamma_q, fn, "gamma_q"); check_cuda(gamma_k, fn, "gamma_k");
    if (q_proj.numel() != 1LL * B * n_new * Hq * d_h || q_out.numel() != q_proj.numel() ||
        k_proj.numel() != 1LL * B * n_new * Hkv * d_h || v_proj.numel() != k_proj.numel())
        throw std::invalid_argument("kv_cache_append: shape mismatch (q/k/v)");
    if (kcache.numel() != 1LL * B * Hkv * L_cap * d_h || vcache.numel() != kcache.numel())
        throw std::invalid_argument("kv_cache_append: shape mismatch (caches)");
    if (gamma_q.numel() != d_h || gamma_k.numel() != d_h || cos.numel() < 1LL * (pos0 + n_new) * (d_h / 2) ||
        sin.numel() < 1LL * (pos0 + n_new) * (d_h / 2))
        throw std::invalid_argument("kv_cache_append: shape mismatch (gamma/cos/sin)");
    raise(b200attn_kv_append(q_proj.data(), k_proj.data(), v_proj.data(), xd, q_out.data(), kcache.data(), vcache.data(),
                             static_cast<const float*>(gamma_q.data()), static_cast<const float*>(gamma_k.data()),
                             static_cast<const float*>(cos.data()), static_cast<const float*>(sin.data()), B, n_new, pos0,
                             L_cap, Hq, Hkv, d_h, eps, stream),
          fn);
}

void flash_attn_decode_cached(const Tensor& q, const Tensor& kcache, const Tensor& vcache, Tensor& o, int B, int L, int L_cap,
                              int Hq, int Hkv, int D, void* stream) {
    const char* fn = "flash_attn_decode_cached";
    check(q, DType::BF16, fn, "q"); check(kcache, DType::BF16, fn, "kcache"); check(vcache, DType::BF16, fn, "vcache");
    check(o, DType::BF16, fn, "o");
    check_cuda(q, fn, "q"); check_cuda(kcache, fn, "kcache"); check_cuda(vcache, fn, "vcache"); check_cuda(o, fn, "o");
    if (q.numel() != 1LL * B * Hq * D || o.numel() != q.numel() || kcache.numel() != 1LL * B * Hkv * L_cap * D ||
        vcache.numel() != kcache.numel())
        throw std::invalid_argument("flash_attn_decode_cached: shape mismatch");
    const size_t ws_bytes = b200attn_decode_workspace_bytes(B, L, Hq, Hkv, D, 0);
    raise(b200attn_decode_cached(q.data(), kcache.data(), vcache.data(), o.data(), nullptr, B, L, L_cap, Hq, Hkv, D, 0.f, 0,
                                 cached_workspace(kWsDecode, ws_bytes, stream), ws_bytes, stream),
          fn);
}

void flash_attn_forward_kvcache(const Tensor& q, const Tensor& kcache, const Tensor& vcache, Tensor& ctx, Tensor& L, int B,
                                int T, int L_cap, int Hq, int Hkv, int D, void* stream) {
    const char* fn = "flash_attn_forward_kvcache";
    check(q, DType::BF16, fn, "q"); check(kcache, DType::BF16, fn, "kcache"); check(vcache, DType::BF16, fn, "vcache");
    check(ctx, DType::BF16, fn, "ctx"); check(L, DType::FP32, fn, "L");
    check_cuda(q, fn, "q"); check_cuda(kcache, fn, "kcache"); check_cuda(vcache, fn, "vcache"); check_cuda(ctx, fn, "ctx");
    check_cuda(L, fn, "L");
    if (q.numel() != 1LL * B * Hq * T * D || ctx.numel() != q.numel() || L.numel() != 1LL * B * Hq * T ||
        kcache.numel() != 1LL * B * Hkv * L_cap * D || vcache.numel() != kcache.numel())
        throw std::invalid_argument("flash_attn_forward_kvcache: shape mismatch");
    raise(b200attn_fwd_kvcache(q.data(), kcache.data(), vcache.data(), ctx.data(), static_cast<float*>(L.data()), B, T, L_cap,
                               Hq, Hkv, D, B200ATTN_LAYOUT_BHTD, 0.f, stream),
          fn);
}

}  // namespace b200
}  // namespace modernllm
