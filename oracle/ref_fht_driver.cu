// Same-box GPU comparator driver (test infrastructure, run by hand): times the reference's standalone transform
// launcher  template <DType> void run_fht(void* a, void* out, uint32_t numel, uint32_t had_size, cudaStream_t)
// (csrc/main.cuh:5-6), compiled unmodified from a checkout of the reference, on the shapes of the transform sweep:
// (16384, n) bf16, n = 2^8 .. 2^15, buffers rotated so that at least 512 MB pass between reuses.  The first rows of
// each result are checked against a plain butterfly on the host.  This file is the only code here; the kernels
// are the reference's.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <vector>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "main.cuh"   // from the reference checkout (-I <ref>/csrc)

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { printf("CUDA error %s at %d\n", cudaGetErrorString(e_), __LINE__); return 1; } } while (0)

int main()
{
    const uint32_t rows = 16384;
    for (int logn = 8; logn <= 15; ++logn) {
        const uint32_t n = 1u << logn;
        const size_t numel = (size_t)rows * n, bytes = numel * 2;
        size_t nbuf = ((512ull << 20) + bytes - 1) / bytes;
        if (nbuf < 2) nbuf = 2;
        std::vector<__nv_bfloat16> h(numel);
        uint32_t s = 12345u + logn;
        for (size_t i = 0; i < numel; ++i) {
            s = s * 1664525u + 1013904223u;
            h[i] = __float2bfloat16(((int)(s >> 8) % 2001 - 1000) / 500.0f);
        }
        std::vector<void *> in(nbuf);
        void *out;
        for (auto &p : in) { CK(cudaMalloc(&p, bytes)); CK(cudaMemcpy(p, h.data(), bytes, cudaMemcpyHostToDevice)); }
        CK(cudaMalloc(&out, bytes));
        for (size_t i = 0; i < nbuf && i < 3; ++i) run_fht<DType::BFloat16>(in[i], out, (uint32_t)numel, n, 0);
        CK(cudaDeviceSynchronize());
        cudaEvent_t e0, e1;
        CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1));
        const int reps = 10;
        CK(cudaEventRecord(e0));
        for (int r = 0; r < reps; ++r)
            for (size_t i = 0; i < nbuf; ++i) run_fht<DType::BFloat16>(in[i], out, (uint32_t)numel, n, 0);
        CK(cudaEventRecord(e1));
        CK(cudaEventSynchronize(e1));
        float ms;
        CK(cudaEventElapsedTime(&ms, e0, e1));
        ms /= (float)(reps * nbuf);
        // check 4 rows against a host butterfly (scale 1/sqrt(n))
        std::vector<__nv_bfloat16> got((size_t)4 * n);
        CK(cudaMemcpy(got.data(), out, got.size() * 2, cudaMemcpyDeviceToHost));
        double maxerr = 0;
        std::vector<double> v(n);
        for (int r = 0; r < 4; ++r) {
            for (uint32_t i = 0; i < n; ++i) v[i] = __bfloat162float(h[(size_t)r * n + i]);
            for (uint32_t st = 1; st < n; st <<= 1)
                for (uint32_t i = 0; i < n; i += 2 * st)
                    for (uint32_t j = i; j < i + st; ++j) { double a = v[j], b = v[j + st]; v[j] = a + b; v[j + st] = a - b; }
            for (uint32_t i = 0; i < n; ++i) {
                double e = fabs(v[i] / sqrt((double)n) - __bfloat162float(got[(size_t)r * n + i]));
                if (e > maxerr) maxerr = e;
            }
        }
        printf("n=%6u  %8.2f us  %7.1f GB/s  max|err|=%.3e (4 rows vs host butterfly)\n", n, ms * 1000.0, bytes * 2.0 / ms / 1e6, maxerr);
        for (auto &p : in) cudaFree(p);
        cudaFree(out);
    }
    return 0;
}
