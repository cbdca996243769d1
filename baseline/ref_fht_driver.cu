// Same-box GPU comparator driver (not product code, not an oracle): times the reference's two standalone transform
// launchers, compiled unmodified from a checkout of the reference, and prints one RESULT line per shape.
//   default        template <DType> void run_fht(void*, void*, uint32_t numel, uint32_t had_size, cudaStream_t)
//                  of csrc/main.cu (declared in csrc/main.cuh:5-6)
//   -DUSE_HADACORE template <torch::ScalarType> void run_fht(...) of HadaCore/hadamard_transform_cuda.cu:699-746
// Shapes (bf16, n = 2^8 .. 2^15):
//   rot   (16384, n), in place on rotating buffers of at least 512 MB (the shape of this repository's transform sweep)
//   2p30  2^30 elements per n, in place on one buffer (the reference's own benchmark shape, bench/bench.py:138, 268-276)
// The first rows of a result are checked against a plain butterfly on the host (out of place, once per n).
// Everything in this file is this repository's code; the kernels are the reference's.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#ifdef USE_HADACORE
#include <c10/core/ScalarType.h>
template <c10::ScalarType dtype>
void run_fht(void *a, void *out, uint32_t numel, uint32_t had_size, cudaStream_t stream);
#define RUN_FHT run_fht<c10::ScalarType::BFloat16>
#define CASE_NAME "HadaCore"
#else
#include "main.cuh"   // from the reference checkout (-I <ref>/csrc)
#define RUN_FHT run_fht<DType::BFloat16>
#define CASE_NAME "Ours(reference csrc)"
#endif

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { printf("CUDA error %s at %d\n", cudaGetErrorString(e_), __LINE__); return 1; } } while (0)

int main(int argc, char **argv)
{
    const bool only_rot = argc > 1 && !strcmp(argv[1], "rot");
    const bool only_2p30 = argc > 1 && !strcmp(argv[1], "2p30");
    cudaEvent_t e0, e1;
    CK(cudaEventCreate(&e0));
    CK(cudaEventCreate(&e1));
    for (int logn = 8; logn <= 15; ++logn) {
        const uint32_t n = 1u << logn;
        // ---- check: 4 rows, out of place, against a host butterfly (scale 1/sqrt(n))
        {
            const uint32_t rows = 256;
            std::vector<__nv_bfloat16> h((size_t)rows * n), got((size_t)4 * n);
            uint32_t s = 12345u + logn;
            for (auto &v : h) { s = s * 1664525u + 1013904223u; v = __float2bfloat16(((int)(s >> 8) % 2001 - 1000) / 500.0f); }
            void *din, *dout;
            CK(cudaMalloc(&din, h.size() * 2));
            CK(cudaMalloc(&dout, h.size() * 2));
            CK(cudaMemcpy(din, h.data(), h.size() * 2, cudaMemcpyHostToDevice));
            RUN_FHT(din, dout, rows * n, n, 0);
            CK(cudaDeviceSynchronize());
            CK(cudaMemcpy(got.data(), dout, got.size() * 2, cudaMemcpyDeviceToHost));
            double maxerr = 0;
            std::vector<double> v(n);
            for (int r = 0; r < 4; ++r) {
                for (uint32_t i = 0; i < n; ++i) v[i] = __bfloat162float(h[(size_t)r * n + i]);
                for (uint32_t st = 1; st < n; st <<= 1)
                    for (uint32_t i = 0; i < n; i += 2 * st)
                        for (uint32_t j = i; j < i + st; ++j) { double a = v[j], b = v[j + st]; v[j] = a + b; v[j + st] = a - b; }
                for (uint32_t i = 0; i < n; ++i)
                    maxerr = fmax(maxerr, fabs(v[i] / sqrt((double)n) - __bfloat162float(got[(size_t)r * n + i])));
            }
            printf("CHECK case=%s n=%u max_abs_err=%.3e\n", CASE_NAME, n, maxerr);
            cudaFree(din);
            cudaFree(dout);
        }
        for (int shape = 0; shape < 2; ++shape) {
            if ((shape == 0 && only_2p30) || (shape == 1 && only_rot)) continue;
            const uint64_t rows = shape == 0 ? 16384 : ((1ull << 30) >> logn);
            const size_t numel = (size_t)rows * n, bytes = numel * 2;
            size_t nbuf = shape == 0 ? ((512ull << 20) + bytes - 1) / bytes : 1;
            if (shape == 0 && nbuf < 2) nbuf = 2;
            std::vector<void *> buf(nbuf);
            for (auto &p : buf) { CK(cudaMalloc(&p, bytes)); CK(cudaMemset(p, 0x3c, bytes)); }   // 0x3c3c: a small bf16
            const int reps = shape == 0 ? 10 : 10;
            for (size_t i = 0; i < nbuf; ++i) RUN_FHT(buf[i], buf[i], (uint32_t)numel, n, 0);
            CK(cudaDeviceSynchronize());
            CK(cudaEventRecord(e0));
            for (int r = 0; r < reps; ++r)
                for (size_t i = 0; i < nbuf; ++i) RUN_FHT(buf[i], buf[i], (uint32_t)numel, n, 0);
            CK(cudaEventRecord(e1));
            CK(cudaEventSynchronize(e1));
            float ms;
            CK(cudaEventElapsedTime(&ms, e0, e1));
            printf("RESULT case=%s shape=%s m=%u n=%llu dtype=bfloat16 runs=%d per_iter_ms=%.6f total_ms=%.4f\n", CASE_NAME,
                   shape == 0 ? "rot" : "2p30", n, (unsigned long long)rows, (int)(reps * nbuf), ms / (reps * nbuf), ms);
            for (auto &p : buf) cudaFree(p);
        }
    }
    return 0;
}
