/*
 * Oracle (test infrastructure only): token-sequential gated delta rule in plain C, float32.
 * Restates the recurrence of the reference's CUDA kernel (src/kernels/qwen35.cu:64-96) and of its in-test
 * scalar loop (src/archs/qwen35_text.rs:1419-1438):
 *     S *= exp(g_t);  r = S^T k_t;  delta = (v_t - r) * beta_t;  S += k_t delta^T;  o_t = S^T q_t,  S0 = 0.
 * Layout: q, k [B, H, L, Dk]; v [B, H, L, Dv]; g, beta [B, H, L]; out [B, L, H, Dv].
 * Also a plain f32 `x W^T` used as the single-threaded CPU GEMM baseline.
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>

void oracle_delta_rule_seq(const float* q, const float* k, const float* v, const float* g, const float* beta,
                           float* out, int B, int H, int L, int Dk, int Dv) {
    for (int b = 0; b < B; ++b) {
        for (int h = 0; h < H; ++h) {
            float* S = (float*)calloc((size_t)Dk * Dv, sizeof(float));
            const size_t bh = (size_t)b * H + h;
            for (int t = 0; t < L; ++t) {
                const float* qt = q + (bh * L + t) * Dk;
                const float* kt = k + (bh * L + t) * Dk;
                const float* vt = v + (bh * L + t) * Dv;
                const float decay = expf(g[bh * L + t]);
                const float bt = beta[bh * L + t];
                float* ot = out + (((size_t)b * L + t) * H + h) * Dv;
                for (size_t i = 0; i < (size_t)Dk * Dv; ++i) S[i] *= decay;
                for (int c = 0; c < Dv; ++c) {
                    float r = 0.f;
                    for (int d = 0; d < Dk; ++d) r += kt[d] * S[(size_t)d * Dv + c];
                    const float delta = (vt[c] - r) * bt;
                    float o = 0.f;
                    for (int d = 0; d < Dk; ++d) {
                        S[(size_t)d * Dv + c] += kt[d] * delta;
                        o += qt[d] * S[(size_t)d * Dv + c];
                    }
                    ot[c] = o;
                }
            }
            free(S);
        }
    }
}

/* y[T, N] = x[T, K] w[N, K]^T, f32, row-major. */
void oracle_linear_f32(const float* x, const float* w, float* y, int T, int N, int K) {
    for (int t = 0; t < T; ++t) {
        for (int n = 0; n < N; ++n) {
            float acc = 0.f;
            const float* xr = x + (size_t)t * K;
            const float* wr = w + (size_t)n * K;
            for (int kk = 0; kk < K; ++kk) acc += xr[kk] * wr[kk];
            y[(size_t)t * N + n] = acc;
        }
    }
}
