// Fused C = W . H(X).  Replaces fused_ht_gemm_pipelined
// (fused_ht/fusion_pipelined.cu:306-563).
//
// One call = transform of the token rows of X into a workspace that is sized to
// stay L2-resident, followed on the same stream by the contraction against W.
//   fp32 inputs: exact fp32 butterflies + FFMA GEMM (sgemm_nt_kernel, this file)
//   bf16 inputs: 16-bit transform (fwht.cu) + tcgen05 GEMM (gemm_tcgen05.cu)
#include <cstdlib>
#include <mutex>

#include "common.cuh"

namespace b200ht {

int launch_fwht_f32_split(const float *in, __nv_bfloat16 *split, uint64_t rows, uint32_t n, float scale, cudaStream_t st);
int launch_fwht(const void *in, void *out, uint64_t rows, uint32_t n, int dtype, float scale, const void *signs,
                cudaStream_t st, int keep_out = 0);
int launch_gemm_bf16_tcgen05(const void *Y, const void *W, void *C, int M, int N, int K, int out_dtype,
                             int out_layout, cudaStream_t st, const float *row_scale = nullptr,
                             const float *tok_scale = nullptr, size_t ldc = 0);

// ---------------------------------------------------------------------------
// C[m, n] = sum_k A[m, k] * Bm[n, k]   (both operands K-contiguous), fp32 FFMA.
// 128 x 128 x 16 tiles, 256 threads, 8 x 8 outputs per thread, register-staged
// double buffering.
// ---------------------------------------------------------------------------
constexpr int SG_BM = 128, SG_BN = 128, SG_BK = 16, SG_PAD = 4;

__device__ __forceinline__ float4 sg_load4(const float *base, int row, int nrows, int k, int K, bool vec)
{
    float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
    if (row < nrows) {
        const float *p = base + (size_t)row * K + k;
        if (vec && k + 3 < K) {
            r = *(const float4 *)p;
        } else {
            if (k < K) r.x = p[0];
            if (k + 1 < K) r.y = p[1];
            if (k + 2 < K) r.z = p[2];
            if (k + 3 < K) r.w = p[3];
        }
    }
    return r;
}

template <int OUT_DT, int LAYOUT>
__global__ void __launch_bounds__(256)
sgemm_nt_kernel(const float *A, const float *Bm, void *C, int M, int N, int K, int vec, const float *row_scale,
                const float *tok_scale)
{
    __shared__ __align__(16) float As[2][SG_BK][SG_BM + SG_PAD];
    __shared__ __align__(16) float Bs[2][SG_BK][SG_BN + SG_PAD];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * SG_BM, n0 = blockIdx.x * SG_BN;
    float4 ra[2], rb[2];
    const int lrow = tid >> 2, lk = (tid & 3) * 4;  // second half: row + 64

    auto gload = [&](int kt) {
        const int k = kt * SG_BK + lk;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            ra[i] = sg_load4(A, m0 + lrow + 64 * i, M, k, K, vec != 0);
            rb[i] = sg_load4(Bm, n0 + lrow + 64 * i, N, k, K, vec != 0);
        }
    };
    auto sstore = [&](int buf) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int r = lrow + 64 * i;
            As[buf][lk + 0][r] = ra[i].x; As[buf][lk + 1][r] = ra[i].y;
            As[buf][lk + 2][r] = ra[i].z; As[buf][lk + 3][r] = ra[i].w;
            Bs[buf][lk + 0][r] = rb[i].x; Bs[buf][lk + 1][r] = rb[i].y;
            Bs[buf][lk + 2][r] = rb[i].z; Bs[buf][lk + 3][r] = rb[i].w;
        }
    };

    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

    const int ktiles = (K + SG_BK - 1) / SG_BK;
    gload(0);
    sstore(0);
    __syncthreads();
    for (int kt = 0; kt < ktiles; ++kt) {
        const int buf = kt & 1;
        if (kt + 1 < ktiles) gload(kt + 1);
#pragma unroll
        for (int k = 0; k < SG_BK; ++k) {
            const float4 a0 = *(const float4 *)&As[buf][k][ty * 4];
            const float4 a1 = *(const float4 *)&As[buf][k][64 + ty * 4];
            const float4 b0 = *(const float4 *)&Bs[buf][k][tx * 4];
            const float4 b1 = *(const float4 *)&Bs[buf][k][64 + tx * 4];
            const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        if (kt + 1 < ktiles) sstore(buf ^ 1);
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int m = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
        if (m >= M) continue;
        // optional epilogue scales, applied to the fp32 sums before the one rounding of the store
        if (row_scale || tok_scale) {
            const float rs = row_scale ? row_scale[m] : 1.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int n = n0 + (j >> 2) * 64 + tx * 4 + (j & 3);
                acc[i][j] *= rs * (tok_scale && n < N ? tok_scale[n] : 1.f);
            }
        }
#pragma unroll
        for (int jh = 0; jh < 2; ++jh) {
            const int n = n0 + jh * 64 + tx * 4;
            if (LAYOUT == B200HT_OUT_MN && OUT_DT == B200HT_F32 && (N & 3) == 0 && n + 3 < N) {
                *(float4 *)((float *)C + (size_t)m * N + n) =
                    make_float4(acc[i][jh * 4], acc[i][jh * 4 + 1], acc[i][jh * 4 + 2], acc[i][jh * 4 + 3]);
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (n + j < N) {
                        const size_t idx = LAYOUT == B200HT_OUT_MN ? (size_t)m * N + n + j : (size_t)(n + j) * M + m;
                        if (OUT_DT == B200HT_F32) ((float *)C)[idx] = acc[i][jh * 4 + j];
                        else ((__nv_bfloat16 *)C)[idx] = __float2bfloat16_rn(acc[i][jh * 4 + j]);
                    }
                }
            }
        }
    }
}

static int launch_sgemm(const float *A, const float *Bm, void *C, int M, int N, int K, int out_dtype,
                        int out_layout, cudaStream_t st, const float *row_scale, const float *tok_scale)
{
    dim3 grid((N + SG_BN - 1) / SG_BN, (M + SG_BM - 1) / SG_BM);
    const int vec = ((K & 3) == 0 && aligned16(A) && aligned16(Bm)) ? 1 : 0;
    note_launch();
    if (out_dtype == B200HT_F32) {
        if (out_layout == B200HT_OUT_MN)
            sgemm_nt_kernel<B200HT_F32, B200HT_OUT_MN><<<grid, 256, 0, st>>>(A, Bm, C, M, N, K, vec, row_scale, tok_scale);
        else
            sgemm_nt_kernel<B200HT_F32, B200HT_OUT_NM><<<grid, 256, 0, st>>>(A, Bm, C, M, N, K, vec, row_scale, tok_scale);
    } else {
        if (out_layout == B200HT_OUT_MN)
            sgemm_nt_kernel<B200HT_BF16, B200HT_OUT_MN><<<grid, 256, 0, st>>>(A, Bm, C, M, N, K, vec, row_scale, tok_scale);
        else
            sgemm_nt_kernel<B200HT_BF16, B200HT_OUT_NM><<<grid, 256, 0, st>>>(A, Bm, C, M, N, K, vec, row_scale, tok_scale);
    }
    return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------
// fp32 on the tensor cores: every fp32 operand is the exact sum of three bf16
// terms (8 + 8 + 8 significant bits), a = a1 + a2 + a3.  Of the nine cross
// products the six with weight >= 2^-16 are kept,
//   a.b ~ a1.b3 + a3.b1 + a2.b2 + a1.b2 + a2.b1 + a1.b1      (dropped: ~3 * 2^-24 |a.b|),
// every bf16 x bf16 product is exact in the fp32 accumulator, and the six
// partial contractions are one bf16 GEMM over a K axis six times as long:
// row m of W becomes [w1 w3 w2 w1 w2 w1] and token row n of H(X) becomes
// [y3 y1 y2 y2 y1 y1] (six blocks of K), smallest terms first.  The contraction
// then runs on the tcgen05 kernel at bf16 rate / 6 instead of the FFMA rate.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) split3_kernel(const float4 *src, __nv_bfloat16 *dst, size_t nvec, int K,
                                                     int is_w)
{
    const int kv = K >> 2;   // float4 per row
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) {
        const float4 v = src[i];
        const size_t row = i / kv;
        const int k = (int)(i - row * kv) * 4;
        const float a[4] = {v.x, v.y, v.z, v.w};
        uint2 t[3];
        uint32_t h[3][4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float r = a[e];
#pragma unroll
            for (int j = 0; j < 3; ++j) {
                const __nv_bfloat16 b = __float2bfloat16_rn(r);
                h[j][e] = (uint32_t)__bfloat16_as_ushort(b);
                r -= __bfloat162float(b);   // exact
            }
        }
#pragma unroll
        for (int j = 0; j < 3; ++j) t[j] = make_uint2(h[j][0] | (h[j][1] << 16), h[j][2] | (h[j][3] << 16));
        __nv_bfloat16 *o = dst + row * (size_t)(6 * K) + k;
        // block order (smallest products first): W: 1 3 2 1 2 1 ; H(X): 3 1 2 2 1 1
        const int pw[6] = {0, 2, 1, 0, 1, 0}, py[6] = {2, 0, 1, 1, 0, 0};
#pragma unroll
        for (int b = 0; b < 6; ++b) *(uint2 *)(o + (size_t)b * K) = t[is_w ? pw[b] : py[b]];
    }
}

static size_t fp32_tc_workspace_bytes(int M, int N, int K)
{
    const size_t a = (((size_t)N * K * 4) + 255) & ~(size_t)255;
    const size_t b = (((size_t)M * K * 12) + 255) & ~(size_t)255;
    const size_t c = (((size_t)N * K * 12) + 255) & ~(size_t)255;
    return a + b + c;
}
// Shapes that take the split path: rows long enough for the tcgen05 kernel, enough work to hide the two extra
// passes over the operands, and K <= 4096.  The tensor core adds into its fp32 accumulator with truncation, so the
// error of a contraction grows with its length: measured relative error (Frobenius) 1.0e-6 at K = 1024, 4.4e-6 at
// K = 4096, 9.1e-6 at K = 8192 (FFMA kernel: 0.6e-6, 1.2e-6, 1.6e-6); beyond 4096 the margin to 1e-5 is gone.
static bool fp32_tc_shape(int M, int N, int K) { return K >= 32 && K <= 4096 && (double)M * N * K >= 5e8; }

// X (fp32, untransformed) and W (fp32) -> C through the split contraction; `ws` is the part of the workspace behind
// the fp32 H(X) area (which this path leaves unused: the transform kernel writes the split rows directly).
static int launch_fp32_tc(const float *X, const float *W, void *C, int M, int N, int K, float scale, int out_dtype,
                          int out_layout, unsigned char *ws, cudaStream_t st, const float *row_scale,
                          const float *tok_scale)
{
    __nv_bfloat16 *Ws = (__nv_bfloat16 *)ws;
    __nv_bfloat16 *Ys = (__nv_bfloat16 *)(ws + ((((size_t)M * K * 12) + 255) & ~(size_t)255));
    int rc = launch_fwht_f32_split(X, Ys, (uint64_t)N, (uint32_t)K, scale, st);
    if (rc) return rc;
    const size_t wv = (size_t)M * K / 4;
    const int cap = 148 * 16;
    note_launch();
    split3_kernel<<<(unsigned)((wv + 255) / 256 < (size_t)cap ? (wv + 255) / 256 : cap), 256, 0, st>>>(
        (const float4 *)W, Ws, wv, K, 1);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    return launch_gemm_bf16_tcgen05(Ys, Ws, C, M, N, 6 * K, out_dtype, out_layout, st, row_scale, tok_scale);
}

}  // namespace b200ht

extern "C" size_t b200ht_fused_gemm_tc_workspace_bytes(int M, int N, int K, int in_dtype)
{
    using namespace b200ht;
    if (N <= 0 || K <= 0 || M <= 0) return 0;
    if (in_dtype != B200HT_F32 || !fp32_tc_shape(M, N, K)) return b200ht_fused_gemm_workspace_bytes(M, N, K, in_dtype);
    return fp32_tc_workspace_bytes(M, N, K);
}

extern "C" size_t b200ht_fused_gemm_workspace_bytes(int M, int N, int K, int in_dtype)
{
    (void)M;
    if (N <= 0 || K <= 0) return 0;
    const size_t esz = in_dtype == B200HT_F32 ? 4 : 2;
    size_t bytes = (size_t)N * (size_t)K * esz;
    return (bytes + 255) & ~(size_t)255;
}

static int fused_gemm_entry(const void *X, const void *W, void *C, int M, int N, int K, int in_dtype, int out_dtype,
                            int out_layout, float scale, const void *signs, void *workspace, size_t workspace_bytes,
                            void *stream, const float *row_scale = nullptr, const float *tok_scale = nullptr)
{
    using namespace b200ht;
    if (in_dtype != B200HT_F32 && in_dtype != B200HT_BF16) return B200HT_ERR_DTYPE;
    if (out_dtype != B200HT_F32 && out_dtype != B200HT_BF16) return B200HT_ERR_DTYPE;
    if (signs && in_dtype != B200HT_BF16) return B200HT_ERR_DTYPE;
    if (out_layout != B200HT_OUT_MN && out_layout != B200HT_OUT_NM) return B200HT_ERR_SIZE;
    if (K < 2 || K > (1 << kMaxLogN) || !is_pow2((uint64_t)K)) return B200HT_ERR_SIZE;
    if (M < 0 || N < 0) return B200HT_ERR_SIZE;
    if (M == 0 || N == 0) return 0;
    if (!X || !W || !C) return B200HT_ERR_NULL;
    if (!aligned16(X) || !aligned16(W) || !aligned16(C) || (signs && !aligned16(signs))) return B200HT_ERR_ALIGN;
    const size_t need = b200ht_fused_gemm_workspace_bytes(M, N, K, in_dtype);
    if (!workspace || workspace_bytes < need) return B200HT_ERR_WORKSPACE;
    if (((uintptr_t)workspace & 255u) != 0) return B200HT_ERR_ALIGN;
    int rc = check_device();
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    // fp32: a workspace of the larger size (b200ht_fused_gemm_tc_workspace_bytes) selects the split-bf16 tensor-core
    // contraction, the minimal one the exact FFMA kernel
    if (in_dtype == B200HT_F32 && fp32_tc_shape(M, N, K) && workspace_bytes >= fp32_tc_workspace_bytes(M, N, K))
        return launch_fp32_tc((const float *)X, (const float *)W, C, M, N, K, scale, out_dtype, out_layout,
                              (unsigned char *)workspace + ((((size_t)N * K * 4) + 255) & ~(size_t)255), st, row_scale,
                              tok_scale);
    if (in_dtype == B200HT_F32) {
        rc = launch_fwht(X, workspace, (uint64_t)N, (uint32_t)K, in_dtype, scale, signs, st);
        if (rc) return rc;
        return launch_sgemm((const float *)W, (const float *)workspace, C, M, N, K, out_dtype, out_layout, st, row_scale,
                            tok_scale);
    }
    // bf16.  A token range whose transformed rows would not stay in the 126 MB L2 is processed in chunks: transform
    // of a chunk into the (one) chunk-sized head of the workspace, contraction of that chunk against all of W, next
    // chunk.  Every kernel of the chain waits for its predecessor, so the chunk is written, read while it is still in
    // L2, and overwritten by the next chunk before its lines are evicted: the transformed tokens do not travel to HBM
    // and back.  B200HT_GEMM_CHUNK_MB=<MB> sets the chunk size (0: one chunk; tuning knob).
    static const size_t chunk_bytes = [] {
        size_t mb = 32;
        if (const char *e = std::getenv("B200HT_GEMM_CHUNK_MB")) mb = (size_t)std::atol(e);
        return mb << 20;
    }();
    const size_t row_bytes = (size_t)K * 2;
    if (chunk_bytes == 0 || K < 64 || (size_t)N * row_bytes <= chunk_bytes + chunk_bytes / 2) {
        rc = launch_fwht(X, workspace, (uint64_t)N, (uint32_t)K, in_dtype, scale, signs, st, 1);
        if (rc) return rc;
        return launch_gemm_bf16_tcgen05(workspace, W, C, M, N, K, out_dtype, out_layout, st, row_scale, tok_scale);
    }
    long per = (long)(chunk_bytes / row_bytes) & ~255L;       // tokens per chunk: whole 256-token tiles
    if (per < 256) per = 256;
    const long nchunks = (N + per - 1) / per;
    per = (((N + nchunks - 1) / nchunks) + 255) & ~255L;      // balanced
    const size_t out_esz = out_dtype == B200HT_F32 ? 4 : 2;
    for (long t0 = 0; t0 < N; t0 += per) {
        const int nt = (int)((N - t0) < per ? (N - t0) : per);
        rc = launch_fwht((const unsigned char *)X + (size_t)t0 * row_bytes, workspace, (uint64_t)nt, (uint32_t)K, in_dtype,
                         scale, signs, st, 1);
        if (rc) return rc;
        unsigned char *Cc = (unsigned char *)C + (out_layout == B200HT_OUT_MN ? (size_t)t0 : (size_t)t0 * M) * out_esz;
        rc = launch_gemm_bf16_tcgen05(workspace, W, Cc, M, nt, K, out_dtype, out_layout, st, row_scale,
                                      tok_scale ? tok_scale + t0 : nullptr,
                                      out_layout == B200HT_OUT_MN ? (size_t)N : (size_t)M);
        if (rc) return rc;
    }
    return 0;
}

extern "C" int b200ht_fused_gemm(const void *X, const void *W, void *C, int M, int N, int K, int in_dtype,
                                 int out_dtype, int out_layout, float scale, void *workspace,
                                 size_t workspace_bytes, void *stream)
{
    return fused_gemm_entry(X, W, C, M, N, K, in_dtype, out_dtype, out_layout, scale, nullptr, workspace,
                            workspace_bytes, stream);
}

extern "C" int b200ht_fused_gemm_signed(const void *X, const void *W, void *C, int M, int N, int K, int in_dtype,
                                        int out_dtype, int out_layout, float scale, const void *signs,
                                        void *workspace, size_t workspace_bytes, void *stream)
{
    if (!signs) return B200HT_ERR_NULL;
    return fused_gemm_entry(X, W, C, M, N, K, in_dtype, out_dtype, out_layout, scale, signs, workspace,
                            workspace_bytes, stream);
}

extern "C" int b200ht_fused_gemm_scaled(const void *X, const void *W, void *C, int M, int N, int K, int in_dtype,
                                        int out_dtype, int out_layout, float scale, const void *signs,
                                        const float *row_scale, const float *tok_scale, void *workspace,
                                        size_t workspace_bytes, void *stream)
{
    if ((row_scale && ((uintptr_t)row_scale & 3u)) || (tok_scale && ((uintptr_t)tok_scale & 3u))) return B200HT_ERR_ALIGN;
    return fused_gemm_entry(X, W, C, M, N, K, in_dtype, out_dtype, out_layout, scale, signs, workspace,
                            workspace_bytes, stream, row_scale, tok_scale);
}

// ---------------------------------------------------------------------------
// Allocation-free variant of b200ht_fused_gemm.
//
// Some callers cannot hand this library a workspace because they cannot
// allocate one at the point of the call: a serving process whose own pool took
// all device memory at start-up, a plugin whose enqueue hook is forbidden to
// allocate, a latency-critical loop that must not take the driver's allocation
// lock (cudaMalloc may also synchronise the device).  For them the transformed
// tokens go into a fixed array that is part of the library image.
//
// g_static_scratch is a __device__ array: in host code its name is only a
// handle for the runtime, not a device address.  The address the kernels and
// the TMA descriptor need is resolved with cudaGetSymbolAddress, once per
// device, while that device is current.
// ---------------------------------------------------------------------------
namespace b200ht {

static __device__ __align__(256) unsigned char g_static_scratch[B200HT_STATIC_SCRATCH_BYTES];

static int static_scratch_address(void **out)
{
    static std::mutex mu;
    static void *addr[64] = {nullptr};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return B200HT_ERR_DEVICE;
    std::lock_guard<std::mutex> lk(mu);
    if (!addr[dev]) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) return (int)e;
        if (!p) return B200HT_ERR_NULL;
        addr[dev] = p;
    }
    *out = addr[dev];
    return 0;
}

}  // namespace b200ht

extern "C" int b200ht_fused_gemm_static(const void *X, const void *W, void *C, int M, int N, int K, int in_dtype,
                                        int out_dtype, int out_layout, float scale, void *stream)
{
    using namespace b200ht;
    if (in_dtype != B200HT_F32 && in_dtype != B200HT_BF16) return B200HT_ERR_DTYPE;
    if (M < 0 || N < 0 || K < 2 || K > (1 << kMaxLogN) || !is_pow2((uint64_t)K)) return B200HT_ERR_SIZE;
    // Reject before anything is enqueued: the transformed tokens must fit the built-in array.
    const size_t need = b200ht_fused_gemm_workspace_bytes(M, N, K, in_dtype);
    if (need > (size_t)B200HT_STATIC_SCRATCH_BYTES) return B200HT_ERR_STATIC_SCRATCH;
    int rc = check_device();
    if (rc) return rc;
    void *scratch = nullptr;
    rc = static_scratch_address(&scratch);
    if (rc) return rc;
    // Same two phases as b200ht_fused_gemm, on the resolved device address.  Every row of the
    // scratch that the contraction reads is written by the transform phase of this same call,
    // so nothing has to be cleared between calls.
    return b200ht_fused_gemm(X, W, C, M, N, K, in_dtype, out_dtype, out_layout, scale, scratch, need, stream);
}
