// Small-batch fused Y = W . H(X).  Replaces fused_hadamard_gemv_kernel(_vec)
// (fused_ht/fwht_gemv_fusion.cu:98-244).
//
// The reference launches one block per column of X, so W is streamed B times.
// Here the grid runs over ROWS of W: every CTA transforms the (tiny) X once
// into shared memory, then streams its rows of W exactly once with 16-byte
// loads and multiplies them against all B columns at the same time.  Bound:
// HBM traffic of W (M*N*2 bytes for bf16).
//
//   bf16: H(X) is kept in shared memory as bf16 (rounded once, after an fp32
//         transform); products run on mma.sync m16n8k16 with fp32 accumulators.
//         A lane loads 8 consecutive k of one W row (16 bytes); the same 8 k of
//         H(X) are read from shared memory for the B operand, so the two mma of
//         a 32-wide k block see one consistent permutation of k.
//   fp32: exact FFMA path (correctness cases), one warp per row.
#include "common.cuh"
#include "fwht_f32.cuh"

namespace b200ht {

__device__ __forceinline__ uint4 ld_nc16(const void *p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ void store_out(void *Y, size_t idx, float v, int out_dtype)
{
    if (out_dtype == B200HT_F32) ((float *)Y)[idx] = v;
    else ((__nv_bfloat16 *)Y)[idx] = __float2bfloat16_rn(v);
}

// ---------------------------------------------------------------------------
// bf16
// ---------------------------------------------------------------------------
template <int NT>
__global__ void __launch_bounds__(256, 1)
gemv_bf16_kernel(const __nv_bfloat16 *W, const __nv_bfloat16 *X, void *Y, int M, int N, int logn, int B,
                 int b0, int Bg, int gc, int out_dtype, float scale)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int hstride = N + 32;  // bf16 elements per H(X) row: 64 bytes of padding
    __nv_bfloat16 *hx = (__nv_bfloat16 *)smem_raw;
    float *scratch = (float *)(smem_raw + (size_t)Bg * hstride * 2);
    float *red = scratch + (size_t)gc * N;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;

    // H(X) for the columns of this group, gc columns at a time through fp32 scratch
    for (int c0 = 0; c0 < Bg; c0 += gc) {
        const int cols = (Bg - c0) < gc ? (Bg - c0) : gc;
        for (int idx = tid; idx < cols * N; idx += 256) {
            const int i = idx / cols, c = idx - i * cols;
            scratch[c * N + i] = __bfloat162float(X[(size_t)i * B + b0 + c0 + c]);
        }
        __syncthreads();
        slab_fwht_f32(scratch, cols * N, logn, tid, 256);
        for (int idx = tid; idx < cols * N; idx += 256) {
            const int c = idx >> logn, i = idx & (N - 1);
            hx[(size_t)(c0 + c) * hstride + i] = __float2bfloat16_rn(scratch[idx] * scale);
        }
        __syncthreads();
    }

    const int ntiles = (M + 15) >> 4;
    const int kblocks = N >> 5;
    for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        float acc[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
        const int r0 = tile * 16 + g, r1 = r0 + 8;
        const __nv_bfloat16 *w0 = W + (size_t)r0 * N + 8 * t;
        const __nv_bfloat16 *w1 = W + (size_t)r1 * N + 8 * t;
        constexpr int U = 4;
        for (int kb0 = warp; kb0 < kblocks; kb0 += 8 * U) {
            uint4 wa[U], wb[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int kb = kb0 + 8 * u;
                wa[u] = (kb < kblocks && r0 < M) ? ld_nc16(w0 + kb * 32) : make_uint4(0, 0, 0, 0);
                wb[u] = (kb < kblocks && r1 < M) ? ld_nc16(w1 + kb * 32) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int kb = kb0 + 8 * u;
                if (kb < kblocks) {
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        int col = nt * 8 + g;
                        col = col < Bg ? col : Bg - 1;
                        const uint4 h = *(const uint4 *)(hx + (size_t)col * hstride + kb * 32 + 8 * t);
                        mma16816_bf16_acc(acc[nt], wa[u].x, wb[u].x, wa[u].y, wb[u].y, h.x, h.y);
                        mma16816_bf16_acc(acc[nt], wa[u].z, wb[u].z, wa[u].w, wb[u].w, h.z, h.w);
                    }
                }
            }
        }
        // cross-warp reduction: red[warp][row 0..15][col 0..NT*8-1]
        constexpr int RC = NT * 8;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            float *p = red + ((size_t)warp * 16 + g) * RC + nt * 8 + 2 * t;
            p[0] = acc[nt][0];
            p[1] = acc[nt][1];
            p[8 * RC] = acc[nt][2];
            p[8 * RC + 1] = acc[nt][3];
        }
        __syncthreads();
        for (int idx = tid; idx < 16 * Bg; idx += 256) {
            const int r = idx / Bg, c = idx - r * Bg;
            float s = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) s += red[((size_t)w * 16 + r) * RC + c];
            const int row = tile * 16 + r;
            if (row < M) store_out(Y, (size_t)row * B + b0 + c, s, out_dtype);
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------
// fp32 (exact): H(X) in shared memory as fp32, one warp per row of W
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
gemv_f32_kernel(const float *W, const float *X, void *Y, int M, int N, int logn, int B, int b0, int Bg,
                int out_dtype, float scale)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float *hx = (float *)smem_raw;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int idx = tid; idx < Bg * N; idx += 256) {
        const int i = idx / Bg, c = idx - i * Bg;
        hx[c * N + i] = X[(size_t)i * B + b0 + c];
    }
    __syncthreads();
    slab_fwht_f32(hx, Bg * N, logn, tid, 256);
    for (int idx = tid; idx < Bg * N; idx += 256) hx[idx] *= scale;
    __syncthreads();
    for (int row = blockIdx.x * 8 + warp; row < M; row += gridDim.x * 8) {
        const float *w = W + (size_t)row * N;
        for (int c0 = 0; c0 < Bg; c0 += 4) {
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            for (int k = lane; k < N; k += 32) {
                const float wv = w[k];
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (c0 + j < Bg) acc[j] = fmaf(wv, hx[(c0 + j) * N + k], acc[j]);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float s = acc[j];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                if (lane == 0 && c0 + j < Bg) store_out(Y, (size_t)row * B + b0 + c0 + j, s, out_dtype);
            }
        }
    }
}

static int sm_count()
{
    int dev = 0, n = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    return n;
}

template <int NT>
static int launch_bf16_nt(const void *W, const void *X, void *Y, int M, int N, int logn, int B, int b0,
                          int Bg, int gc, int out_dtype, float scale, size_t smem, cudaStream_t st)
{
    cudaError_t e =
        cudaFuncSetAttribute(gemv_bf16_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    const int tiles = (M + 15) / 16;
    const int grid = tiles < sm_count() ? tiles : sm_count();
    gemv_bf16_kernel<NT><<<grid, 256, smem, st>>>((const __nv_bfloat16 *)W, (const __nv_bfloat16 *)X, Y, M,
                                                  N, logn, B, b0, Bg, gc, out_dtype, scale);
    return (int)cudaGetLastError();
}

static size_t bf16_smem(int N, int Bg, int gc)
{
    int nt = (Bg + 7) / 8;
    if (nt > 4) nt = 8;  // the kernel is instantiated for 1, 2, 3, 4 and 8 column tiles
    return (size_t)Bg * (N + 32) * 2 + (size_t)gc * N * 4 + (size_t)8 * 16 * nt * 8 * 4;
}

int launch_gemv(const void *W, const void *X, void *Y, int M, int N, int B, int in_dtype, int out_dtype,
                float scale, cudaStream_t st)
{
    const int logn = ilog2((uint32_t)N);
    constexpr size_t kBudget = 200 * 1024;
    if (in_dtype == B200HT_F32 || N < 32) {
        if (in_dtype != B200HT_F32) return B200HT_ERR_SIZE;  // bf16 path needs N >= 32
        int bg_max = (int)(kBudget / ((size_t)N * 4));
        if (bg_max < 1) bg_max = 1;
        for (int b0 = 0; b0 < B; b0 += bg_max) {
            const int Bg = (B - b0) < bg_max ? (B - b0) : bg_max;
            const size_t smem = (size_t)Bg * N * 4;
            cudaError_t e = cudaFuncSetAttribute(gemv_f32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)smem);
            if (e != cudaSuccess) return (int)e;
            int grid = (M + 7) / 8;
            const int cap = sm_count() * 2;
            grid = grid < cap ? grid : cap;
            gemv_f32_kernel<<<grid, 256, smem, st>>>((const float *)W, (const float *)X, Y, M, N, logn, B, b0,
                                                     Bg, out_dtype, scale);
            e = cudaGetLastError();
            if (e != cudaSuccess) return (int)e;
        }
        return 0;
    }
    // bf16: largest column group whose H(X) fits in shared memory
    int gc = 16384 / N;
    gc = gc < 1 ? 1 : (gc > 4 ? 4 : gc);
    int bg_max = B < 64 ? B : 64;
    while (bg_max > 1 && bf16_smem(N, bg_max, gc < bg_max ? gc : bg_max) > kBudget) --bg_max;
    for (int b0 = 0; b0 < B; b0 += bg_max) {
        const int Bg = (B - b0) < bg_max ? (B - b0) : bg_max;
        const int g = gc < Bg ? gc : Bg;
        const size_t smem = bf16_smem(N, Bg, g);
        const int nt = (Bg + 7) / 8;
        int rc;
        switch (nt) {
        case 1: rc = launch_bf16_nt<1>(W, X, Y, M, N, logn, B, b0, Bg, g, out_dtype, scale, smem, st); break;
        case 2: rc = launch_bf16_nt<2>(W, X, Y, M, N, logn, B, b0, Bg, g, out_dtype, scale, smem, st); break;
        case 3: rc = launch_bf16_nt<3>(W, X, Y, M, N, logn, B, b0, Bg, g, out_dtype, scale, smem, st); break;
        case 4: rc = launch_bf16_nt<4>(W, X, Y, M, N, logn, B, b0, Bg, g, out_dtype, scale, smem, st); break;
        default: rc = launch_bf16_nt<8>(W, X, Y, M, N, logn, B, b0, Bg, g, out_dtype, scale, smem, st); break;
        }
        if (rc) return rc;
    }
    return 0;
}

}  // namespace b200ht

extern "C" int b200ht_fused_gemv(const void *W, const void *X, void *Y, int M, int N, int B, int in_dtype,
                                 int out_dtype, float scale, void *stream)
{
    using namespace b200ht;
    if (in_dtype != B200HT_F32 && in_dtype != B200HT_BF16) return B200HT_ERR_DTYPE;
    if (out_dtype != B200HT_F32 && out_dtype != B200HT_BF16) return B200HT_ERR_DTYPE;
    if (N < 2 || N > (1 << kMaxLogN) || !is_pow2((uint64_t)N)) return B200HT_ERR_SIZE;
    if (M < 0 || B < 1 || B > 64) return B200HT_ERR_SIZE;
    if (in_dtype == B200HT_BF16 && N < 32) return B200HT_ERR_SIZE;
    if (M == 0) return 0;
    if (!W || !X || !Y) return B200HT_ERR_NULL;
    if (!aligned16(W) || !aligned16(X) || !aligned16(Y)) return B200HT_ERR_ALIGN;
    int rc = check_device();
    if (rc) return rc;
    return launch_gemv(W, X, Y, M, N, B, in_dtype, out_dtype, scale, (cudaStream_t)stream);
}
