// fp32 butterfly transform of a slab held in shared memory.  Used by the exact
// fp32 paths (standalone fp32 transform, fp32 fused GEMM, fp32 fused GEMV).
#pragma once
#include "common.cuh"

namespace b200ht {

// One pass over index bits [b, b+G): every thread takes groups of 2^G elements
// that differ only in those bits, runs the butterflies in registers, writes back.
template <int G>
__device__ __forceinline__ void radix_pass(float *s, int total, int b, int tid, int nthr)
{
    constexpr int R = 1 << G;
    const int items = total >> G;
    const int lowmask = (1 << b) - 1;
    for (int i = tid; i < items; i += nthr) {
        const int base = ((i >> b) << (b + G)) | (i & lowmask);
        float v[R];
#pragma unroll
        for (int t = 0; t < R; ++t) v[t] = s[base + (t << b)];
#pragma unroll
        for (int h = 1; h < R; h <<= 1) {
#pragma unroll
            for (int t = 0; t < R; ++t) {
                if (!(t & h)) {
                    const float x = v[t], y = v[t | h];
                    v[t] = x + y;
                    v[t | h] = x - y;
                }
            }
        }
#pragma unroll
        for (int t = 0; t < R; ++t) s[base + (t << b)] = v[t];
    }
    __syncthreads();
}

// In-place unscaled transform of total / 2^logn contiguous rows of length 2^logn
// in shared memory.  Called by all threads of the block; the data must be
// visible (a __syncthreads() before the call) and is visible on return.
__device__ __forceinline__ void slab_fwht_f32(float *s, int total, int logn, int tid, int nthr)
{
    int b = 0;
    while (b < logn) {
        const int g = (logn - b) >= 3 ? 3 : (logn - b);
        if (g == 3) radix_pass<3>(s, total, b, tid, nthr);
        else if (g == 2) radix_pass<2>(s, total, b, tid, nthr);
        else radix_pass<1>(s, total, b, tid, nthr);
        b += g;
    }
}

}  // namespace b200ht
