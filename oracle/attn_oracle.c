/*
 * CPU oracle for causal grouped-query attention.  TEST INFRASTRUCTURE ONLY:
 * it is the checker for the CUDA kernels and the timed CPU baseline of the
 * benchmark; no product code path may call into it.
 *
 * It restates, in plain C with double accumulation, the algorithm of
 * AlsoTheZv3n/modern-llm-v1 (paths are relative to that project's root):
 *   - forward softmax(scale * Q K^T, causal) V:
 *       host reference attn_host, llm/tests/test_attention.cu:21-75
 *       (double dot products :36-41, float row max :45-48, double row sum
 *       :49-52, double P.V accumulation :64-72);
 *   - logsumexp L = row_max + log(row_sum) of the SCALED scores, natural log:
 *       llm/src/model/flash_attn.cu:124-130, host loop
 *       llm/tests/test_flash_attn.cu:104-129;
 *   - backward  P = exp(s - L), dP = dO V^T, D = sum_j P dP (= O . dO),
 *       dS = P (dP - D), dQ = scale dS K, dK = scale dS^T Q, dV = P^T dO:
 *       llm/src/model/flash_attn.cu:137-146 and the softmax backward of
 *       llm/src/model/attention.cu:66-108, GEMM orientation :199-257;
 *   - grouped-query mapping h_kv = h_q / (Hq / Hkv) and the sum of the
 *       per-query-head dK/dV over the group:
 *       llm/src/model/attention.cu:393-429 (repeat_kv_heads_kernel,
 *       accumulate_kv_grads_kernel);
 *   - softmax scale 1/sqrt(D): llm/src/model/flash_attn.cu:418;
 *   - BF16 round-to-nearest-even: llm/src/core/dtype.h:34-49;
 *   - RoPE (interleaved pairs, theta_i = base^(-2i/d) in float):
 *       llm/src/model/rope.cu:25-44,112-128, host form llm/tests/test_rope.cu:18-38;
 *   - RMSNorm rows (rsqrt(mean(x^2)+eps), gamma = 1):
 *       llm/src/model/rmsnorm.cu:24-53, host form llm/tests/test_rmsnorm.cu:16-27.
 *
 * Pinned against the reference's own host code (attn_host, mha_host,
 * rope_host, rmsnorm_host compiled from the reference tree) through the
 * committed fixtures under tests/golden/.
 *
 * Layout of every tensor: element (b, h, t, d) at b*sb + h*sh + t*st + d
 * (unit stride on d), so both [B,H,T,D] and [B,T,H,D] are expressible.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef struct {
    long long sb, sh, st; /* element strides of batch, head, token */
} oracle_strides;

int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void oracle_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* llm/src/core/dtype.h:34-42 */
static inline uint16_t f32_to_bf16_bits(float f) {
    uint32_t bits;
    memcpy(&bits, &f, 4);
    uint32_t lsb = (bits >> 16) & 1u;
    bits += 0x7fffu + lsb;
    return (uint16_t)(bits >> 16);
}
static inline float bf16_bits_to_f32(uint16_t h) {
    uint32_t bits = (uint32_t)h << 16;
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

void oracle_round_bf16(float* x, long long n) {
    for (long long i = 0; i < n; ++i) x[i] = bf16_bits_to_f32(f32_to_bf16_bits(x[i]));
}
void oracle_f32_to_bf16(const float* x, uint16_t* y, long long n) {
    for (long long i = 0; i < n; ++i) y[i] = f32_to_bf16_bits(x[i]);
}
void oracle_bf16_to_f32(const uint16_t* x, float* y, long long n) {
    for (long long i = 0; i < n; ++i) y[i] = bf16_bits_to_f32(x[i]);
}

/* RoPE in place over rows [n_rows_outer, T, D]; token t gets position pos0 + t.
 * llm/src/model/rope.cu:112-128 (table) and :25-44 (rotation). */
void oracle_rope_inplace(float* x, long long n_outer, int T, int D, float base, int pos0) {
    int half = D / 2;
#pragma omp parallel for schedule(static)
    for (long long n = 0; n < n_outer; ++n) {
        for (int t = 0; t < T; ++t) {
            float* row = x + (n * T + t) * (long long)D;
            for (int i = 0; i < half; ++i) {
                float theta = powf(base, -(float)(2 * i) / (float)D);
                float angle = (float)(pos0 + t) * theta;
                float c = cosf(angle), s = sinf(angle);
                float x0 = row[2 * i], x1 = row[2 * i + 1];
                row[2 * i] = x0 * c - x1 * s;
                row[2 * i + 1] = x0 * s + x1 * c;
            }
        }
    }
}

/* RMSNorm with gamma = 1 over rows of length D.  llm/src/model/rmsnorm.cu:24-53
 * (float sum of squares, rsqrtf(ms + eps)). */
void oracle_rmsnorm_rows(float* x, long long rows, int D, float eps) {
#pragma omp parallel for schedule(static)
    for (long long n = 0; n < rows; ++n) {
        float* row = x + n * (long long)D;
        double sq = 0.0;
        for (int d = 0; d < D; ++d) sq += (double)row[d] * (double)row[d];
        float ms = (float)(sq / D);
        float rstd = 1.f / sqrtf(ms + eps);
        for (int d = 0; d < D; ++d) row[d] = row[d] * rstd;
    }
}

/* Fused RoPE + RMSNorm with gamma over x [n_outer, T, D] (row (n, t) is token t): the chain
 * rope_apply_inplace -> rmsnorm_forward of llm/src/model/modern_gpt.cu:358-370.
 * Rotation and table: llm/src/model/rope.cu:25-44,112-128; norm: llm/src/model/rmsnorm.cu:24-53
 * (rstd = rsqrt(mean r^2 + eps), y = r rstd gamma).  Sums in double. */
void oracle_rope_norm_fwd_at(const float* x, const float* gamma, float* y, float* rstd, long long n_outer, int T,
                             int D, float base, float eps, int pos0);
void oracle_rope_norm_fwd(const float* x, const float* gamma, float* y, float* rstd, long long n_outer, int T, int D,
                          float base, float eps) {
    oracle_rope_norm_fwd_at(x, gamma, y, rstd, n_outer, T, D, base, eps, 0);
}
/* The same with row (n, t) at position pos0 + t: what a KV cache needs for the newest tokens of a sequence
 * (the reference's rope_apply_inplace takes the position from the row index, llm/src/model/rope.cu:25-44, and
 * its sampler has no cache, llm/apps/infer_modern_gpt.cu:13). */
void oracle_rope_norm_fwd_at(const float* x, const float* gamma, float* y, float* rstd, long long n_outer, int T,
                             int D, float base, float eps, int pos0) {
    int half = D / 2;
#pragma omp parallel for schedule(static)
    for (long long n = 0; n < n_outer; ++n) {
        for (int t = 0; t < T; ++t) {
            const float* xr = x + (n * T + t) * (long long)D;
            float* yr = y + (n * T + t) * (long long)D;
            float r[512];
            double sq = 0.0;
            for (int i = 0; i < half; ++i) {
                float theta = powf(base, -(float)(2 * i) / (float)D);
                float angle = (float)(pos0 + t) * theta;
                float c = cosf(angle), s = sinf(angle);
                r[2 * i] = xr[2 * i] * c - xr[2 * i + 1] * s;
                r[2 * i + 1] = xr[2 * i] * s + xr[2 * i + 1] * c;
                sq += (double)r[2 * i] * r[2 * i] + (double)r[2 * i + 1] * r[2 * i + 1];
            }
            float rs = (float)(1.0 / sqrt(sq / D + (double)eps));
            rstd[n * T + t] = rs;
            for (int d = 0; d < D; ++d) yr[d] = r[d] * rs * gamma[d];
        }
    }
}

/* Backward of the chain above: rmsnorm_backward (llm/src/model/rmsnorm.cu:55-101:
 * g = dy gamma, s = sum g r, dr = rstd g - rstd^3 / D s r, d_gamma += dy r rstd) followed by
 * rope_apply_backward_inplace (llm/src/model/rope.cu:46-65: the inverse rotation).
 * d_gamma [D] is accumulated into (llm/src/model/rmsnorm.h:17).  Sums in double; single thread
 * over rows for d_gamma so that the result does not depend on the thread count. */
void oracle_rope_norm_bwd(const float* dy, const float* x, const float* gamma, const float* rstd, float* dx,
                          float* d_gamma, long long n_outer, int T, int D, float base) {
    int half = D / 2;
    double dg[512];
    for (int d = 0; d < D; ++d) dg[d] = 0.0;
    for (long long n = 0; n < n_outer; ++n) {
        for (int t = 0; t < T; ++t) {
            const float* xr = x + (n * T + t) * (long long)D;
            const float* dyr = dy + (n * T + t) * (long long)D;
            float* dxr = dx + (n * T + t) * (long long)D;
            double rs = rstd[n * T + t];
            double r[512], c[256], s[256], dr[512];
            double sum = 0.0;
            for (int i = 0; i < half; ++i) {
                float theta = powf(base, -(float)(2 * i) / (float)D);
                float angle = (float)t * theta;
                c[i] = cosf(angle), s[i] = sinf(angle);
                r[2 * i] = xr[2 * i] * c[i] - xr[2 * i + 1] * s[i];
                r[2 * i + 1] = xr[2 * i] * s[i] + xr[2 * i + 1] * c[i];
            }
            for (int d = 0; d < D; ++d) {
                sum += (double)dyr[d] * gamma[d] * r[d];
                dg[d] += (double)dyr[d] * r[d] * rs;
            }
            double coeff = rs * rs * rs / D * sum;
            for (int d = 0; d < D; ++d) dr[d] = rs * dyr[d] * gamma[d] - coeff * r[d];
            for (int i = 0; i < half; ++i) {
                dxr[2 * i] = (float)(dr[2 * i] * c[i] + dr[2 * i + 1] * s[i]);
                dxr[2 * i + 1] = (float)(-dr[2 * i] * s[i] + dr[2 * i + 1] * c[i]);
            }
        }
    }
    for (int d = 0; d < D; ++d) d_gamma[d] += (float)dg[d];
}

/* One query head (b, hq): forward and, when dout != NULL, backward.
 * dk_acc/dv_acc are [T, D] double accumulators private to this query head
 * (the per-query-head dK/dV that the reference produces before
 * accumulate_kv_grads sums them over the group). */
static void head_fwd_bwd(const float* q, const float* k, const float* v, const float* dout, long long qst,
                         long long kst, int T, int D, float scale, float* o, long long ost, float* lse,
                         float* dq, long long dqst, double* dk_acc, double* dv_acc, double* p, double* ds) {
    for (int i = 0; i < T; ++i) {
        const float* qi = q + i * qst;
        /* scores: double dot, times scale, stored as float (test_attention.cu:36-41) */
        float row_max = -INFINITY;
        for (int j = 0; j <= i; ++j) {
            const float* kj = k + j * kst;
            double s = 0.0;
            for (int d = 0; d < D; ++d) s += (double)qi[d] * (double)kj[d];
            float sf = (float)(s * scale);
            p[j] = sf;
            row_max = fmaxf(row_max, sf);
        }
        double sum = 0.0;
        for (int j = 0; j <= i; ++j) {
            p[j] = exp(p[j] - (double)row_max);
            sum += p[j];
        }
        double inv = 1.0 / sum;
        for (int j = 0; j <= i; ++j) p[j] *= inv;
        if (lse) lse[i] = (float)((double)row_max + log(sum));
        if (o) {
            float* oi = o + i * ost;
            for (int d = 0; d < D; ++d) {
                double acc = 0.0;
                for (int j = 0; j <= i; ++j) acc += p[j] * (double)v[j * kst + d];
                oi[d] = (float)acc;
            }
        }
        if (!dout) continue;
        const float* doi = dout + i * qst;
        /* dP_j = dO_i . V_j ; D_i = sum_j P_ij dP_ij (attention.cu:86-100) */
        double Di = 0.0;
        for (int j = 0; j <= i; ++j) {
            const float* vj = v + j * kst;
            double dp = 0.0;
            for (int d = 0; d < D; ++d) dp += (double)doi[d] * (double)vj[d];
            ds[j] = dp;
            Di += p[j] * dp;
        }
        for (int j = 0; j <= i; ++j) ds[j] = p[j] * (ds[j] - Di);
        float* dqi = dq + i * dqst;
        for (int d = 0; d < D; ++d) {
            double acc = 0.0;
            for (int j = 0; j <= i; ++j) acc += ds[j] * (double)k[j * kst + d];
            dqi[d] = (float)((double)scale * acc);
        }
        for (int j = 0; j <= i; ++j) {
            double dsj = ds[j] * (double)scale, pj = p[j];
            double* dkj = dk_acc + (long long)j * D;
            double* dvj = dv_acc + (long long)j * D;
            for (int d = 0; d < D; ++d) {
                dkj[d] += dsj * (double)qi[d];
                dvj[d] += pj * (double)doi[d];
            }
        }
    }
}

/* Forward: o [B,Hq,T,D] (strides so), lse [B,Hq,T] contiguous (may be NULL). */
void oracle_attn_fwd(const float* q, const float* k, const float* v, float* o, float* lse, int B, int T, int Hq,
                     int Hkv, int D, float scale, const oracle_strides* sq, const oracle_strides* skv,
                     const oracle_strides* so) {
    int group = Hq / Hkv;
#pragma omp parallel
    {
        double* p = (double*)malloc(sizeof(double) * (size_t)T);
#pragma omp for schedule(dynamic, 1) collapse(2)
        for (int b = 0; b < B; ++b)
            for (int h = 0; h < Hq; ++h) {
                int hk = h / group; /* attention.cu:406 */
                head_fwd_bwd(q + b * sq->sb + h * sq->sh, k + b * skv->sb + hk * skv->sh,
                             v + b * skv->sb + hk * skv->sh, NULL, sq->st, skv->st, T, D, scale,
                             o + b * so->sb + h * so->sh, so->st, lse ? lse + ((long long)b * Hq + h) * T : NULL,
                             NULL, 0, NULL, NULL, p, NULL);
            }
        free(p);
    }
}

/* Forward + backward.  Outputs o, lse, dq as in forward layouts; dk, dv in the
 * K/V layout (strides skv), summed over the query heads of each group in
 * ascending head order.  Any of o, lse may be NULL. */
void oracle_attn_fwd_bwd(const float* q, const float* k, const float* v, const float* dout, float* o, float* lse,
                         float* dq, float* dk, float* dv, int B, int T, int Hq, int Hkv, int D, float scale,
                         const oracle_strides* sq, const oracle_strides* skv, const oracle_strides* so) {
    int group = Hq / Hkv;
    size_t per_head = (size_t)T * D;
    /* per-query-head dK/dV, like the reference's n_q-wide buffers before accumulate_kv_grads */
    double* dkh = (double*)calloc((size_t)B * Hq * per_head, sizeof(double));
    double* dvh = (double*)calloc((size_t)B * Hq * per_head, sizeof(double));
#pragma omp parallel
    {
        double* p = (double*)malloc(sizeof(double) * (size_t)T);
        double* ds = (double*)malloc(sizeof(double) * (size_t)T);
#pragma omp for schedule(dynamic, 1) collapse(2)
        for (int b = 0; b < B; ++b)
            for (int h = 0; h < Hq; ++h) {
                int hk = h / group;
                size_t hh = ((size_t)b * Hq + h) * per_head;
                /* dO shares q's layout; dq shares q's layout */
                head_fwd_bwd(q + b * sq->sb + h * sq->sh, k + b * skv->sb + hk * skv->sh,
                             v + b * skv->sb + hk * skv->sh, dout + b * sq->sb + h * sq->sh, sq->st, skv->st, T, D,
                             scale, o ? o + b * so->sb + h * so->sh : NULL, so->st,
                             lse ? lse + ((long long)b * Hq + h) * T : NULL, dq + b * sq->sb + h * sq->sh, sq->st,
                             dkh + hh, dvh + hh, p, ds);
            }
        free(p);
        free(ds);
        /* group sum: attention.cu:412-429 (there with atomics; here in head order) */
#pragma omp for schedule(static) collapse(2)
        for (int b = 0; b < B; ++b)
            for (int hk = 0; hk < Hkv; ++hk)
                for (int t = 0; t < T; ++t)
                    for (int d = 0; d < D; ++d) {
                        double sk = 0.0, sv = 0.0;
                        for (int g = 0; g < group; ++g) {
                            size_t hh = ((size_t)b * Hq + hk * group + g) * per_head + (size_t)t * D + d;
                            sk += dkh[hh];
                            sv += dvh[hh];
                        }
                        long long off = b * skv->sb + hk * skv->sh + t * skv->st + d;
                        dk[off] = (float)sk;
                        dv[off] = (float)sv;
                    }
    }
    free(dkh);
    free(dvh);
}

/* Decode: one query token per sequence against a cache of L keys.  Equals row
 * L-1 of the causal forward with T = L (the cache already holds the current
 * token).  q,o: [B,Hq,D] contiguous; kc,vc: [B,Hkv,L,D] via strides skv;
 * lse [B,Hq] (may be NULL). */
void oracle_decode(const float* q, const float* kc, const float* vc, float* o, float* lse, int B, int L, int Hq,
                   int Hkv, int D, float scale, const oracle_strides* skv) {
    int group = Hq / Hkv;
#pragma omp parallel
    {
        double* p = (double*)malloc(sizeof(double) * (size_t)L);
#pragma omp for schedule(dynamic, 1) collapse(2)
        for (int b = 0; b < B; ++b)
            for (int h = 0; h < Hq; ++h) {
                int hk = h / group;
                const float* qi = q + ((long long)b * Hq + h) * D;
                const float* k = kc + b * skv->sb + hk * skv->sh;
                const float* v = vc + b * skv->sb + hk * skv->sh;
                float row_max = -INFINITY;
                for (int j = 0; j < L; ++j) {
                    double s = 0.0;
                    for (int d = 0; d < D; ++d) s += (double)qi[d] * (double)k[j * skv->st + d];
                    float sf = (float)(s * scale);
                    p[j] = sf;
                    row_max = fmaxf(row_max, sf);
                }
                double sum = 0.0;
                for (int j = 0; j < L; ++j) {
                    p[j] = exp(p[j] - (double)row_max);
                    sum += p[j];
                }
                float* oi = o + ((long long)b * Hq + h) * D;
                for (int d = 0; d < D; ++d) {
                    double acc = 0.0;
                    for (int j = 0; j < L; ++j) acc += p[j] * (double)v[j * skv->st + d];
                    oi[d] = (float)(acc / sum);
                }
                if (lse) lse[(long long)b * Hq + h] = (float)((double)row_max + log(sum));
            }
        free(p);
    }
}
