// Checker-side glue, built only where the reference tree is present: pulls the
// reference's own host functions (which live in anonymous namespaces of its
// test translation units) into a shared library with a C ABI, so that the
// oracle can be pinned against them.  Test infrastructure only; compiled from
// the reference sources where they lie, output under oracle/_ref/.
//
//   REF_TU == 1: attn_host     llm/tests/test_attention.cu:21-75
//   REF_TU == 2: mha_host      llm/tests/test_mha.cu:24-72
//   REF_TU == 3: rope_host     llm/tests/test_rope.cu:18-38
//   REF_TU == 4: rmsnorm_host  llm/tests/test_rmsnorm.cu:16-27
#if REF_TU == 1
#define main modernllm_ref_test_attention_main
#include "tests/test_attention.cu"
#undef main
#include "core/dtype.h"
// BF16 round-to-nearest-even of the reference, llm/src/core/dtype.h:34-49
extern "C" void ref_f32_to_bf16(const float* x, unsigned short* y, long long n) {
    for (long long i = 0; i < n; ++i) y[i] = modernllm::f32_to_bf16(x[i]);
}
extern "C" void ref_bf16_to_f32(const unsigned short* x, float* y, long long n) {
    for (long long i = 0; i < n; ++i) y[i] = modernllm::bf16_to_f32(x[i]);
}
extern "C" void ref_attn_host(const float* q, const float* k, const float* v, int B, int T, int D, float* ctx,
                              float* probs) {
    attn_host(q, k, v, B, T, D, ctx, probs);
}
#elif REF_TU == 2
#define main modernllm_ref_test_mha_main
#include "tests/test_mha.cu"
#undef main
extern "C" void ref_mha_host(const float* q, const float* k, const float* v, int B, int T, int H, int d_h,
                             float* ctx) {
    mha_host(q, k, v, B, T, H, d_h, ctx);
}
#elif REF_TU == 3
#define main modernllm_ref_test_rope_main
#include "tests/test_rope.cu"
#undef main
extern "C" void ref_rope_host(const float* in, float* out, int N, int T, int d_h, float base) {
    rope_host(in, out, N, T, d_h, base);
}
#elif REF_TU == 4
#define main modernllm_ref_test_rmsnorm_main
#include "tests/test_rmsnorm.cu"
#undef main
extern "C" void ref_rmsnorm_host(const float* x, const float* gamma, float* y, int N, int D, float eps) {
    rmsnorm_host(x, gamma, y, N, D, eps);
}
#else
#error "REF_TU must be 1..4"
#endif
