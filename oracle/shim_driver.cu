// Checker-side glue, built only where the reference tree is present: a C ABI over the C++ shim
// (modern-llm-v1_b200/csrc/modernllm_shim.{h,cc}), which offers the reference's own flash-attention signatures
// (llm/src/model/flash_attn.h:25-28,47-52) over the reference's Tensor (llm/src/core/tensor.h:25-97) on top of
// libb200attn.so.  It lets the GPU tests call the boundary exactly as a C++ caller inside the reference tree would:
// reference Tensors in, reference exception types out.  Test infrastructure only; compiled against the reference
// sources where they lie, output under oracle/_ref/.
#include <cuda_runtime.h>

#include <stdexcept>
#include <string>

#include "core/tensor.h"
#include "modernllm_shim.h"

using modernllm::Device;
using modernllm::DType;
using modernllm::Tensor;
namespace shim = modernllm::b200;

namespace {
std::string g_error;

// dtype_code: 0 = BF16 (what the shim takes), 1 = FP32 (what the reference's kernels take: the shim must refuse it)
Tensor blob(const void* p, std::vector<std::int64_t> shape, int dtype_code) {
    return Tensor::from_blob(const_cast<void*>(p), std::move(shape), dtype_code == 0 ? DType::BF16 : DType::FP32, Device::Cuda);
}
Tensor blob_f32(const void* p, std::vector<std::int64_t> shape) {
    return Tensor::from_blob(const_cast<void*>(p), std::move(shape), DType::FP32, Device::Cuda);
}

// 0 = returned normally, 1 = std::invalid_argument, 2 = std::runtime_error, 3 = anything else
template <typename F>
int guarded(F&& f) {
    try {
        f();
        return 0;
    } catch (const std::invalid_argument& e) {
        g_error = e.what();
        return 1;
    } catch (const std::runtime_error& e) {
        g_error = e.what();
        return 2;
    } catch (...) {
        g_error = "unknown exception";
        return 3;
    }
}
}  // namespace

extern "C" const char* shim_last_error() { return g_error.c_str(); }

// The reference-shaped entry points: [B, T, D] with B = batch x heads.
extern "C" int shim_flash_attn_forward(const void* q, const void* k, const void* v, void* ctx, float* L, int B, int T, int D,
                                       int tile_kv, int dtype_code, void* stream) {
    return guarded([&] {
        Tensor tq = blob(q, {B, T, D}, dtype_code), tk = blob(k, {B, T, D}, dtype_code), tv = blob(v, {B, T, D}, dtype_code);
        Tensor tc = blob(ctx, {B, T, D}, dtype_code), tl = blob_f32(L, {B, T});
        shim::flash_attn_forward(tq, tk, tv, tc, tl, B, T, D, tile_kv, stream);
    });
}

extern "C" int shim_flash_attn_backward(const void* q, const void* k, const void* v, const void* ctx, const float* L,
                                        const void* d_ctx, void* d_q, void* d_k, void* d_v, int B, int T, int D, int tile,
                                        int dtype_code, void* stream) {
    return guarded([&] {
        Tensor tq = blob(q, {B, T, D}, dtype_code), tk = blob(k, {B, T, D}, dtype_code), tv = blob(v, {B, T, D}, dtype_code);
        Tensor tc = blob(ctx, {B, T, D}, dtype_code), tl = blob_f32(L, {B, T}), tdc = blob(d_ctx, {B, T, D}, dtype_code);
        Tensor tdq = blob(d_q, {B, T, D}, dtype_code), tdk = blob(d_k, {B, T, D}, dtype_code), tdv = blob(d_v, {B, T, D}, dtype_code);
        shim::flash_attn_backward(tq, tk, tv, tc, tl, tdc, tdq, tdk, tdv, B, T, D, tile, stream);
    });
}

// The GQA overloads: q, ctx, d_* of Hq heads; k, v, d_k, d_v of Hkv heads; layout 0 = BHTD, 1 = BTHD.
extern "C" int shim_flash_attn_forward_gqa(const void* q, const void* k, const void* v, void* ctx, float* L, int B, int T,
                                           int Hq, int Hkv, int D, int layout, void* stream) {
    return guarded([&] {
        Tensor tq = blob(q, {B * Hq, T, D}, 0), tk = blob(k, {B * Hkv, T, D}, 0), tv = blob(v, {B * Hkv, T, D}, 0);
        Tensor tc = blob(ctx, {B * Hq, T, D}, 0), tl = blob_f32(L, {B * Hq, T});
        shim::flash_attn_forward_gqa(tq, tk, tv, tc, tl, B, T, Hq, Hkv, D, static_cast<shim::Layout>(layout), stream);
    });
}

extern "C" int shim_flash_attn_backward_gqa(const void* q, const void* k, const void* v, const void* ctx, const float* L,
                                            const void* d_ctx, void* d_q, void* d_k, void* d_v, int B, int T, int Hq, int Hkv,
                                            int D, int layout, void* stream) {
    return guarded([&] {
        Tensor tq = blob(q, {B * Hq, T, D}, 0), tk = blob(k, {B * Hkv, T, D}, 0), tv = blob(v, {B * Hkv, T, D}, 0);
        Tensor tc = blob(ctx, {B * Hq, T, D}, 0), tl = blob_f32(L, {B * Hq, T}), tdc = blob(d_ctx, {B * Hq, T, D}, 0);
        Tensor tdq = blob(d_q, {B * Hq, T, D}, 0), tdk = blob(d_k, {B * Hkv, T, D}, 0), tdv = blob(d_v, {B * Hkv, T, D}, 0);
        shim::flash_attn_backward_gqa(tq, tk, tv, tc, tl, tdc, tdq, tdk, tdv, B, T, Hq, Hkv, D, static_cast<shim::Layout>(layout),
                                      stream);
    });
}

extern "C" int shim_flash_attn_decode(const void* q, const void* kcache, const void* vcache, void* o, int B, int Lcache, int Hq,
                                      int Hkv, int D, void* stream) {
    return guarded([&] {
        Tensor tq = blob(q, {B, Hq, D}, 0), tk = blob(kcache, {B * Hkv, Lcache, D}, 0), tv = blob(vcache, {B * Hkv, Lcache, D}, 0);
        Tensor to = blob(o, {B, Hq, D}, 0);
        shim::flash_attn_decode(tq, tk, tv, to, B, Lcache, Hq, Hkv, D, stream);
    });
}
