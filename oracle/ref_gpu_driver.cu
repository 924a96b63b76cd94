// Checker-side glue, built only where the reference tree is present: a C ABI
// over the reference's own GPU attention so that GPU tests and the benchmark's
// side table can run "the reference's attention on identical inputs".  Test
// infrastructure only; compiled against the reference sources where they lie,
// output under oracle/_ref/.  All pointers are FP32 device pointers in the
// reference's split layout [B*H, T, D] (llm/src/model/attention.h:22-61,
// llm/src/model/flash_attn.h:25-52).
//
// GQA is done the reference's way (llm/src/model/modern_gpt.cu:372-376,
// 513-522): repeat_kv_heads -> attention -> accumulate_kv_grads.
#include <cuda_runtime.h>

#include <exception>

#include "core/gemm.h"
#include "core/tensor.h"
#include "model/attention.h"
#include "model/flash_attn.h"

using modernllm::Device;
using modernllm::DType;
using modernllm::Tensor;

namespace {
Tensor blob(const void* p, std::vector<std::int64_t> shape) {
    return Tensor::from_blob(const_cast<void*>(p), std::move(shape), DType::FP32, Device::Cuda);
}
}  // namespace

// which: 0 = flash_attn_* (per-row kernels), 1 = scaled_dot_attention_* (cuBLAS SGEMM path).
// q,dout,o,dq: [B*Hq,T,D]; k,v,dk,dv: [B*Hkv,T,D]; lse: [B*Hq,T] (written only by which == 0).
// dout == nullptr skips the backward.  Returns 0, or 1 when the reference threw.
extern "C" int ref_gpu_attention(int which, const float* q, const float* k, const float* v, const float* dout,
                                 float* o, float* lse, float* dq, float* dk, float* dv, int B, int T, int Hq,
                                 int Hkv, int D) {
    try {
        const int BH = B * Hq;
        Tensor tq = blob(q, {BH, T, D});
        Tensor tk = blob(k, {B * Hkv, T, D});
        Tensor tv = blob(v, {B * Hkv, T, D});
        Tensor to = blob(o, {BH, T, D});
        Tensor kfull({BH, T, D}, DType::FP32, Device::Cuda);
        Tensor vfull({BH, T, D}, DType::FP32, Device::Cuda);
        modernllm::repeat_kv_heads(tk, kfull, B, Hkv, Hq, T, D);
        modernllm::repeat_kv_heads(tv, vfull, B, Hkv, Hq, T, D);
        Tensor dkfull, dvfull;
        if (dout) {
            dkfull = Tensor({BH, T, D}, DType::FP32, Device::Cuda);
            dvfull = Tensor({BH, T, D}, DType::FP32, Device::Cuda);
        }
        if (which == 0) {
            Tensor tl = blob(lse, {BH, T});
            modernllm::flash_attn_forward(tq, kfull, vfull, to, tl, BH, T, D);
            if (dout) {
                Tensor tdo = blob(dout, {BH, T, D});
                Tensor tdq = blob(dq, {BH, T, D});
                modernllm::flash_attn_backward(tq, kfull, vfull, to, tl, tdo, tdq, dkfull, dvfull, BH, T, D);
            }
        } else {
            modernllm::CublasHandle handle;
            Tensor probs({BH, T, T}, DType::FP32, Device::Cuda);
            modernllm::scaled_dot_attention_forward(handle, tq, kfull, vfull, to, probs, BH, T, D);
            if (dout) {
                Tensor tdo = blob(dout, {BH, T, D});
                Tensor tdq = blob(dq, {BH, T, D});
                modernllm::scaled_dot_attention_backward(handle, tdo, tq, kfull, vfull, probs, tdq, dkfull, dvfull,
                                                         BH, T, D);
            }
            cudaDeviceSynchronize();
        }
        if (dout) {
            Tensor tdk = blob(dk, {B * Hkv, T, D});
            Tensor tdv = blob(dv, {B * Hkv, T, D});
            tdk.zero();
            tdv.zero();
            modernllm::accumulate_kv_grads(dkfull, tdk, B, Hkv, Hq, T, D);
            modernllm::accumulate_kv_grads(dvfull, tdv, B, Hkv, Hq, T, D);
        }
        return cudaDeviceSynchronize() == cudaSuccess ? 0 : 1;
    } catch (const std::exception&) {
        return 1;
    }
}
