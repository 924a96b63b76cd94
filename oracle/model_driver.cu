// Checker-side glue, built only where the reference tree is present: a C ABI over the reference's ModernGPT
// (llm/src/model/modern_gpt.h:57-177), so that a GPU test can run one forward + backward of the model as the
// reference builds it ("stock") and of the same model with its attention chain on the b200attn engine (the
// generated oracle/_ref/modern_gpt_engine*.cu), compare the loss and every gradient, and time a step both ways.
// The same file is compiled into each variant's library.  Test infrastructure only; output under oracle/_ref/.
#include <cuda_runtime.h>

#include <chrono>
#include <string>
#include <vector>

#include "core/gemm.h"
#include "core/tensor.h"
#include "model/modern_gpt.h"

using modernllm::Device;
using modernllm::DType;
using modernllm::ModernGPT;
using modernllm::Tensor;

namespace {
struct Model {
    ModernGPT gpt;
    modernllm::CublasHandle handle;
    Tensor ids, targets;
    std::vector<modernllm::NamedParam> params;
    size_t free_before = 0;
};
std::string g_error;

void upload(Model& m, const int* ids, const int* targets) {
    const size_t n = static_cast<size_t>(m.gpt.B()) * m.gpt.T() * sizeof(int);
    cudaMemcpy(m.ids.data(), ids, n, cudaMemcpyHostToDevice);
    cudaMemcpy(m.targets.data(), targets, n, cudaMemcpyHostToDevice);
}
float step(Model& m) {
    for (auto& p : m.params) p.grad->zero();
    const float loss = m.gpt.forward(m.ids, &m.targets, m.handle.get());
    m.gpt.backward(m.ids, m.handle.get());
    return loss;
}
}  // namespace

extern "C" const char* model_last_error() { return g_error.c_str(); }

extern "C" void* model_create(int B, int T, int V, int D, int H, int n_kv, int Dff, int n_layers, unsigned long long seed,
                              int use_bf16) {
    try {
        size_t free_b = 0, total_b = 0;
        cudaMemGetInfo(&free_b, &total_b);
        Model* m = new Model();
        m->free_before = free_b;
        ModernGPT::Config cfg;
        cfg.B = B, cfg.T = T, cfg.V = V, cfg.D = D, cfg.H = H, cfg.n_kv_heads = n_kv, cfg.Dff = Dff, cfg.n_layers = n_layers;
        m->gpt.set_use_bf16(use_bf16 != 0);
        m->gpt.allocate(cfg);
        m->gpt.init_random(seed);
        m->ids = Tensor({1LL * B * T}, DType::INT32, Device::Cuda);
        m->targets = Tensor({1LL * B * T}, DType::INT32, Device::Cuda);
        m->params = m->gpt.named_params();
        return m;
    } catch (const std::exception& e) {
        g_error = e.what();
        return nullptr;
    }
}

// One forward + backward on the given token ids / targets (host, B*T int32 each); gradients start from zero.
// Returns the mean loss, or -1 after an exception.
extern "C" float model_step(void* handle, const int* ids, const int* targets) {
    Model& m = *static_cast<Model*>(handle);
    try {
        upload(m, ids, targets);
        const float loss = step(m);
        if (cudaDeviceSynchronize() != cudaSuccess) throw std::runtime_error(cudaGetErrorString(cudaGetLastError()));
        return loss;
    } catch (const std::exception& e) {
        g_error = e.what();
        return -1.f;
    }
}

// Wall time in ms of one forward + backward, averaged over `iters` steps after one untimed step (the reference times
// its steps with the host clock around a synchronise too, llm/apps/train_modern_gpt.cu:259,295-298).
extern "C" double model_time_ms(void* handle, const int* ids, const int* targets, int iters) {
    Model& m = *static_cast<Model*>(handle);
    try {
        upload(m, ids, targets);
        step(m);
        cudaDeviceSynchronize();
        const auto t0 = std::chrono::steady_clock::now();
        for (int i = 0; i < iters; ++i) step(m);
        cudaDeviceSynchronize();
        return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count() / iters;
    } catch (const std::exception& e) {
        g_error = e.what();
        return -1.0;
    }
}

// Device memory this model holds: what the device had free before it was created minus what it has free now.
extern "C" long long model_device_bytes(void* handle) {
    Model& m = *static_cast<Model*>(handle);
    size_t free_b = 0, total_b = 0;
    cudaDeviceSynchronize();
    cudaMemGetInfo(&free_b, &total_b);
    return static_cast<long long>(m.free_before) - static_cast<long long>(free_b);
}

extern "C" int model_n_params(void* handle) { return static_cast<int>(static_cast<Model*>(handle)->params.size()); }
extern "C" const char* model_param_name(void* handle, int i) { return static_cast<Model*>(handle)->params[i].name.c_str(); }
extern "C" long long model_param_numel(void* handle, int i) { return static_cast<Model*>(handle)->params[i].grad->numel(); }
extern "C" int model_copy_grad(void* handle, int i, float* host) {
    Tensor* g = static_cast<Model*>(handle)->params[i].grad;
    return cudaMemcpy(host, g->data(), g->bytes(), cudaMemcpyDeviceToHost) == cudaSuccess ? 0 : 1;
}
extern "C" void model_destroy(void* handle) { delete static_cast<Model*>(handle); }
