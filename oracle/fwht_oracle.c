/*
 * CPU oracle in plain C for the Walsh-Hadamard hot path.  TEST INFRASTRUCTURE
 * ONLY: it is built into oracle/liboracle.so and loaded by tests/, by
 * __graft_entry__.smoke() and by the CPU-baseline legs of bench.py.  Nothing in
 * the product links or calls it.
 *
 * Each function restates one routine of the reference (paths relative to the
 * reference project) as scalar host code:
 *   oracle_fwht_f32 / _f64      fused_ht/fusion_pipelined.cu:117-129 (hadamard_1d)
 *   oracle_fused_gemm_f32/_f64  fused_ht/fusion_pipelined.cu:148-185 + 201-221
 *   oracle_fused_gemv_f32/_f64  fused_ht/fwht_gemv_fusion.cu:98-159
 * The f32 variants keep the reference's fp32 arithmetic and summation order;
 * the f64 variants carry the same algorithm in double so fp32 rounding of the
 * f32 variants is visible.  Parity is pinned by tests/test_oracle.py against
 * the golden vectors made from the reference's bench/bench.py hadamard_ref.
 */
#include <stddef.h>
#include <stdlib.h>
#include <string.h>

/* In-place butterfly, strides 1,2,4,...  (hadamard_1d).  Unscaled. */
void oracle_fwht_f32(float *v, size_t rows, size_t n, float scale)
{
    for (size_t r = 0; r < rows; ++r) {
        float *p = v + r * n;
        for (size_t h = 1; h < n; h <<= 1)
            for (size_t i = 0; i < n; i += (h << 1))
                for (size_t j = i; j < i + h; ++j) {
                    float x = p[j], y = p[j + h];
                    p[j] = x + y;
                    p[j + h] = x - y;
                }
        if (scale != 1.0f)
            for (size_t j = 0; j < n; ++j) p[j] *= scale;
    }
}

void oracle_fwht_f64(double *v, size_t rows, size_t n, double scale)
{
    for (size_t r = 0; r < rows; ++r) {
        double *p = v + r * n;
        for (size_t h = 1; h < n; h <<= 1)
            for (size_t i = 0; i < n; i += (h << 1))
                for (size_t j = i; j < i + h; ++j) {
                    double x = p[j], y = p[j + h];
                    p[j] = x + y;
                    p[j + h] = x - y;
                }
        if (scale != 1.0)
            for (size_t j = 0; j < n; ++j) p[j] *= scale;
    }
}

/* C[m*N+n] = sum_k W[m*K+k] * (scale * H x_n)[k];  X is N x K token-major. */
int oracle_fused_gemm_f32(const float *X, const float *W, float *C,
                          size_t M, size_t N, size_t K, float scale)
{
    float *Y = (float *)malloc(N * K * sizeof(float));
    if (!Y) return -1;
    memcpy(Y, X, N * K * sizeof(float));
    oracle_fwht_f32(Y, N, K, scale);
    for (size_t m = 0; m < M; ++m)
        for (size_t n = 0; n < N; ++n) {
            float acc = 0.f;
            for (size_t k = 0; k < K; ++k) acc += W[m * K + k] * Y[n * K + k];
            C[m * N + n] = acc;
        }
    free(Y);
    return 0;
}

int oracle_fused_gemm_f64(const double *X, const double *W, double *C,
                          size_t M, size_t N, size_t K, double scale)
{
    double *Y = (double *)malloc(N * K * sizeof(double));
    if (!Y) return -1;
    memcpy(Y, X, N * K * sizeof(double));
    oracle_fwht_f64(Y, N, K, scale);
    for (size_t m = 0; m < M; ++m)
        for (size_t n = 0; n < N; ++n) {
            double acc = 0.0;
            for (size_t k = 0; k < K; ++k) acc += W[m * K + k] * Y[n * K + k];
            C[m * N + n] = acc;
        }
    free(Y);
    return 0;
}

/* Y[m*B+b] = sum_k W[m*N+k] * (scale * H x_b)[k];  X[i*B+b], b fastest. */
int oracle_fused_gemv_f32(const float *W, const float *X, float *Y,
                          size_t M, size_t N, size_t B, float scale)
{
    float *col = (float *)malloc(N * sizeof(float));
    if (!col) return -1;
    for (size_t b = 0; b < B; ++b) {
        for (size_t i = 0; i < N; ++i) col[i] = X[i * B + b];
        oracle_fwht_f32(col, 1, N, scale);
        for (size_t m = 0; m < M; ++m) {
            float acc = 0.f;
            for (size_t k = 0; k < N; ++k) acc += W[m * N + k] * col[k];
            Y[m * B + b] = acc;
        }
    }
    free(col);
    return 0;
}

int oracle_fused_gemv_f64(const double *W, const double *X, double *Y,
                          size_t M, size_t N, size_t B, double scale)
{
    double *col = (double *)malloc(N * sizeof(double));
    if (!col) return -1;
    for (size_t b = 0; b < B; ++b) {
        for (size_t i = 0; i < N; ++i) col[i] = X[i * B + b];
        oracle_fwht_f64(col, 1, N, scale);
        for (size_t m = 0; m < M; ++m) {
            double acc = 0.0;
            for (size_t k = 0; k < N; ++k) acc += W[m * N + k] * col[k];
            Y[m * B + b] = acc;
        }
    }
    free(col);
    return 0;
}
