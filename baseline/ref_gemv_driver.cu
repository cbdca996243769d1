// Same-box GPU comparator driver (not product code, not an oracle): launches the reference's fused GEMV kernels
//   fused_hadamard_gemv_kernel / fused_hadamard_gemv_kernel_vec <<<B, 256, N*4>>>(W, X, Y, M, N, B)
// (fused_ht/fwht_gemv_fusion.cu:98-244, launch configuration of :383-400), compiled unmodified from a checkout of
// the reference, on the small-batch shape: W 4096 x 4096, B = 1, 4, 16 (fp32, the only type they take; unscaled
// transform).  16 copies of W are rotated so that W is not L2-resident.  The reference file's own main() is
// renamed out of the way; everything below the include is this repository's code.
#define main reference_main
#include "fwht_gemv_fusion.cu"   // -I <ref>/fused_ht
#undef main

#include <cmath>
#include <vector>

int main()
{
    const int M = 4096, N = 4096, NW = 16;
    std::vector<float> hW((size_t)M * N), hX((size_t)N * 16);
    uint32_t s = 7u;
    auto rnd = [&]() { s = s * 1664525u + 1013904223u; return ((int)(s >> 8) % 2001 - 1000) / 1000.0f; };
    for (auto &v : hW) v = rnd() / 64.0f;
    for (auto &v : hX) v = rnd();
    std::vector<float *> dW(NW);
    for (auto &p : dW) {
        CUDA_CHECK(cudaMalloc(&p, hW.size() * 4));
        CUDA_CHECK(cudaMemcpy(p, hW.data(), hW.size() * 4, cudaMemcpyHostToDevice));
    }
    float *dX, *dY;
    CUDA_CHECK(cudaMalloc(&dX, hX.size() * 4));
    CUDA_CHECK(cudaMalloc(&dY, (size_t)M * 16 * 4));
    cudaEvent_t e0, e1;
    CUDA_CHECK(cudaEventCreate(&e0));
    CUDA_CHECK(cudaEventCreate(&e1));
    for (int B : {1, 4, 16}) {
        // X as N x B, b fastest: take the first B columns of the 16-column host array
        std::vector<float> hXb((size_t)N * B);
        for (int i = 0; i < N; ++i)
            for (int b = 0; b < B; ++b) hXb[(size_t)i * B + b] = hX[(size_t)i * 16 + b];
        CUDA_CHECK(cudaMemcpy(dX, hXb.data(), hXb.size() * 4, cudaMemcpyHostToDevice));
        for (int vec = 0; vec < 2; ++vec) {
            auto launch = [&](float *W) {
                if (vec) fused_hadamard_gemv_kernel_vec<<<B, 256, N * sizeof(float)>>>(W, dX, dY, M, N, B);
                else fused_hadamard_gemv_kernel<<<B, 256, N * sizeof(float)>>>(W, dX, dY, M, N, B);
            };
            for (int i = 0; i < 3; ++i) launch(dW[i]);
            CUDA_CHECK(cudaDeviceSynchronize());
            const int reps = 3;
            CUDA_CHECK(cudaEventRecord(e0));
            for (int r = 0; r < reps; ++r)
                for (int i = 0; i < NW; ++i) launch(dW[i]);
            CUDA_CHECK(cudaEventRecord(e1));
            CUDA_CHECK(cudaEventSynchronize(e1));
            float ms;
            CUDA_CHECK(cudaEventElapsedTime(&ms, e0, e1));
            ms /= reps * NW;
            // check 4 rows of column 0 against a host computation (double)
            std::vector<float> hY((size_t)M * B);
            CUDA_CHECK(cudaMemcpy(hY.data(), dY, hY.size() * 4, cudaMemcpyDeviceToHost));
            std::vector<double> v(N);
            for (int i = 0; i < N; ++i) v[i] = hXb[(size_t)i * B];
            for (int st = 1; st < N; st <<= 1)
                for (int i = 0; i < N; i += 2 * st)
                    for (int j = i; j < i + st; ++j) { double a = v[j], b = v[j + st]; v[j] = a + b; v[j + st] = a - b; }
            double maxrel = 0;
            for (int row : {0, 1, 2047, 4095}) {
                double acc = 0;
                for (int k = 0; k < N; ++k) acc += (double)hW[(size_t)row * N + k] * v[k];
                maxrel = fmax(maxrel, fabs(acc - hY[(size_t)row * B]) / fmax(1e-9, fabs(acc)));
            }
            printf("RESULT case=%s shape=gemv m=%d n=%d batch=%d dtype=float32 runs=%d per_iter_ms=%.6f total_ms=%.4f max_rel_err=%.2e\n",
                   vec ? "fused_hadamard_gemv_kernel_vec" : "fused_hadamard_gemv_kernel", M, N, B, reps * NW, ms,
                   ms * reps * NW, maxrel);
        }
    }
    return 0;
}
