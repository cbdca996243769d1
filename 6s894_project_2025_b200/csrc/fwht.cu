// Standalone Walsh-Hadamard transform along the last dimension of a row-major
// (rows x n) array.  Replaces the reference's hadamard_transform_ker and its
// RowHandler strategies (csrc/main.cu:12-40, csrc/hada_handler.cuh:78-219).
//
// HBM-bound: 2 B read + 2 B written per element, ~15 butterfly stages of
// arithmetic per element at n = 2^15.  The 16x16 Hadamard blocks run on the
// tensor cores (mma.sync m16n8k16, fp32 accumulate) so the arithmetic stays far
// below the memory time; data moves with 16-byte, fully coalesced accesses.
//
//   n = 8 .. 2048   fwht_reg_kernel : a warp keeps whole rows in registers
//   n = 4096..16384 fwht_smem_kernel: a slab of 32 or 64 chunks (two rows of 4096, one row
//                     of 8192 or 16384) in padded shared memory; low 8 index bits in pass
//                     1, the rest in pass 2, both through rot8
//   n = 32768       fwht_tc_kernel (fwht_tcgen05.cu): tcgen05 + TMEM; falls back to
//                     fwht_smem_kernel for buffers that are not 128-byte aligned
//   n = 2, 4        fwht_tiny_kernel : one thread per row
//   fp32            fwht_f32_kernel  : exact fp32 butterflies in shared memory
#include "common.cuh"
#include "fwht_f32.cuh"

#include <cstdlib>

namespace b200ht {

int launch_fwht_tc(const void *in, void *out, uint64_t rows, int logn, int dtype, float scale, cudaStream_t st);

// Optional +-1 diagonal in front of the transform (randomised Hadamard transform): `signs` holds one 16-bit word
// per column, 0x8000 where the column is negated, and is applied by flipping the sign bits of the loaded vector.
// The kernels take it as a template flag: in the unsigned instantiation the loads of a batch stay back to back,
// which a run-time test between them would prevent.
__device__ __forceinline__ void flip_signs(uint4 &v, const uint4 *signs, uint32_t vec_in_row)
{
    const uint4 m = __ldg(signs + vec_in_row);
    v.x ^= m.x; v.y ^= m.y; v.z ^= m.z; v.w ^= m.w;
}
// Smallest log2(n) sent to the tcgen05 kernel; B200HT_FWHT_TC_MIN=<log2 n> overrides it (tuning knob).
static int tc_min_logn()
{
    const char *e = std::getenv("B200HT_FWHT_TC_MIN");
    if (e && e[0] >= '0' && e[0] <= '9') return std::atoi(e);
    return 15;
}

// ---------------------------------------------------------------------------
// n <= 2048, 16-bit: rows live in one warp's registers.
// A warp owns GRP consecutive 256-element chunks (GRP*32 16-byte vectors).
// ---------------------------------------------------------------------------
template <int DT, int LOGN, bool SG>
__global__ void __launch_bounds__(256) fwht_reg_kernel(const uint4 *in, uint4 *out, uint64_t total_vec,
                                                       float mult, const uint4 *signs, int keep)
{
    constexpr int P = LOGN < 8 ? LOGN : 8;
    constexpr int CPR = LOGN > 8 ? (1 << (LOGN - 8)) : 1;  // chunks per row
    constexpr int GRP = CPR > 4 ? CPR : 4;
    // Programmatic dependent launch: let the next kernel of the stream be scheduled while this one
    // drains, and wait here until everything before this kernel has completed and is visible.
    pdl_launch_dependents();
    pdl_wait();
    const uint64_t keep_policy = keep ? l2_policy_evict_last() : 0;   // 0: streaming stores
    const int lane = threadIdx.x & 31;
    const uint64_t warp = (uint64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const uint64_t first = warp * (uint64_t)(GRP * 32);
    if (first >= total_vec) return;

    constexpr unsigned M1 = rot8_mask1(P), M2 = rot8_mask2(P);
    uint32_t A1[4], A2[4];
    make_hfrag<DT>(A1, lane, M1, hfrag_c(popc4(M1)));
    make_hfrag<DT>(A2, lane, M2, hfrag_c(popc4(M2)));

    uint4 v[GRP];
#pragma unroll
    for (int g = 0; g < GRP; ++g) {
        const uint64_t idx = first + (uint64_t)g * 32 + lane;
        v[g] = idx < total_vec ? ld_stream(in + idx) : make_uint4(0, 0, 0, 0);
    }
    if constexpr (SG) {
#pragma unroll
        for (int g = 0; g < GRP; ++g) {
            const uint64_t idx = first + (uint64_t)g * 32 + lane;
            flip_signs(v[g], signs, (uint32_t)idx & ((1u << (LOGN - 3)) - 1u));
        }
    }
    float o[GRP][8];
    rot8x<DT, GRP>(v, o, A1, A2);
    // index bits 8.. : butterflies across the chunks of a row, fp32
#pragma unroll
    for (int s = 1; s < CPR; s <<= 1) {
#pragma unroll
        for (int g = 0; g < GRP; ++g) {
            if (!(g & s)) {
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float x = o[g][e], y = o[g | s][e];
                    o[g][e] = x + y;
                    o[g | s][e] = x - y;
                }
            }
        }
    }
#pragma unroll
    for (int g = 0; g < GRP; ++g) {
        const uint64_t idx = first + (uint64_t)g * 32 + lane;
        if (idx < total_vec) {
            uint4 r;
            r.x = pack2<DT>(o[g][0] * mult, o[g][1] * mult);
            r.y = pack2<DT>(o[g][2] * mult, o[g][3] * mult);
            r.z = pack2<DT>(o[g][4] * mult, o[g][5] * mult);
            r.w = pack2<DT>(o[g][6] * mult, o[g][7] * mult);
            st_out(out + idx, r, keep_policy);
        }
    }
}

// ---------------------------------------------------------------------------
// n = 4096, 8192, 16384 (and 32768 for unaligned buffers or with a sign diagonal), 16-bit: a CTA of 4 warps (8 at
// n = 32768) holds a slab of 32 chunks or more in shared memory: two rows of 4096, one row otherwise.  Chunk c (256
// elements = 32 vectors) sits at vector offset 33*c so that both the contiguous accesses of pass 1 and the
// chunk-strided accesses of pass 2 are bank-conflict free.
//   pass 1: every chunk: index bits 0..7, eight 16-byte loads in flight per lane, result rounded to 16 bit into smem
//   pass 2: index bits 8..LOGN-1: the lanes carry five chunk-index bits and go through rot8 with identity on the
//           in-lane bits (and, at n = 4096, on the lane bit that selects the row); further bits are fp32 register
//           butterflies.  With 4 warps a warp owns 8 consecutive vectors of every chunk.
//   pass 3: copy-out, 128 contiguous bytes per chunk and warp, by the warp that wrote them (no CTA barrier); with 8
//           warps a CTA barrier and whole chunks
// ---------------------------------------------------------------------------
template <int LOGN>
struct SmemCfg {
    static constexpr int Q = LOGN - 8;
    static constexpr int SLAB_ROWS = LOGN >= 13 ? 1 : (1 << (13 - LOGN));
    static constexpr int CPR = 1 << Q;
    static constexpr int NCHUNK = SLAB_ROWS * CPR;
    static constexpr int SMEM_BYTES = NCHUNK * 33 * 16;
    static constexpr int NW = LOGN <= 14 ? 4 : 8;   // warps per CTA
};

template <int DT, int LOGN, bool SG>
__global__ void __launch_bounds__(SmemCfg<LOGN>::NW * 32) fwht_smem_kernel(const uint4 *in, uint4 *out, uint64_t rows,
                                                        float mult, const uint4 *signs, int keep)
{
    using Cfg = SmemCfg<LOGN>;
    constexpr int Q = Cfg::Q, CPR = Cfg::CPR, NW = Cfg::NW;
    extern __shared__ uint4 sm[];
    pdl_launch_dependents();
    pdl_wait();
    const uint64_t keep_policy = keep ? l2_policy_evict_last() : 0;   // 0: streaming stores
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const uint64_t row0 = (uint64_t)blockIdx.x * Cfg::SLAB_ROWS;
    const int rows_here = (int)((rows - row0) < (uint64_t)Cfg::SLAB_ROWS ? (rows - row0)
                                                                          : (uint64_t)Cfg::SLAB_ROWS);
    const int chunks_here = rows_here * CPR;
    const uint4 *gin = in + row0 * (uint64_t)(CPR * 32);
    uint4 *gout = out + row0 * (uint64_t)(CPR * 32);

    uint32_t A1[4], A2[4];
    make_hfrag<DT>(A1, lane, 15u, 0.25f);
    make_hfrag<DT>(A2, lane, 15u, 0.25f);

    constexpr int U = 8;   // chunks (16-byte loads per lane) in flight per warp: 8 is 3-5 % faster than 4
    // Chunks of a missing second row (n = 4096, odd row count) are zeroed: pass 2 multiplies them by the zero entries
    // of its constant, and 0 * (stale NaN) would poison row one.  (A separate loop: with a compile-time bound on the
    // main loop the compiler gives up the stage-wise order of rot8x and the kernel loses a fifth of its speed.)
    for (int c = chunks_here + warp; c < Cfg::NCHUNK; c += NW) sm[c * 33 + lane] = make_uint4(0, 0, 0, 0);
    for (int c0 = warp; c0 < chunks_here; c0 += NW * U) {
        uint4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int c = c0 + NW * u;
            v[u] = c < chunks_here ? ld_stream(gin + c * 32 + lane) : make_uint4(0, 0, 0, 0);
        }
        if constexpr (SG) {
#pragma unroll
            for (int u = 0; u < U; ++u) flip_signs(v[u], signs, (uint32_t)(((c0 + NW * u) & (CPR - 1)) * 32 + lane));
        }
        float o[U][8];
        rot8x<DT, U>(v, o, A1, A2);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int c = c0 + NW * u;
            if (c < chunks_here) {
                uint4 r;
                r.x = pack2<DT>(o[u][0], o[u][1]);
                r.y = pack2<DT>(o[u][2], o[u][3]);
                r.z = pack2<DT>(o[u][4], o[u][5]);
                r.w = pack2<DT>(o[u][6], o[u][7]);
                sm[c * 33 + lane] = r;
            }
        }
    }
    __syncthreads();

    // pass 2: lanes <-> chunk-index bits 0..4 of the row (element bits 8..12)
    // A slab always holds at least 32 chunks: for n = 4096 these are two rows, and the lane bit that selects the row
    // is left alone (identity in the second constant), so the slab goes through the same code as one row of 8192.
    static_assert(Q >= 4, "the slab kernel is written for n >= 4096");
    constexpr unsigned M2 = Q >= 5 ? 7u : 3u;
    make_hfrag<DT>(A1, lane, 6u, 0.5f);
    make_hfrag<DT>(A2, lane, M2, 0.5f);
    constexpr int J = Q > 5 ? (1 << (Q - 5)) : 1;
    const int nitems = 32;
    // n = 8192, 16384 (one row per CTA, 4 warps): a warp takes SPW = 8 consecutive slots, so that it alone writes, and afterwards reads,
    // SPW*16 contiguous bytes of every chunk and no CTA-wide barrier is needed before the copy-out
    constexpr int SPW = 32 / NW;
    constexpr bool LOCAL_OUT = NW == 4;   // n = 8192, 16384: one row per CTA, SPW = 8
    for (int it = 0; it < (LOCAL_OUT ? SPW : (nitems - warp + NW - 1) / NW); ++it) {
        const int item = LOCAL_OUT ? warp * SPW + it : warp + it * NW;
        const int slot = item & 31;
        const int chunk0 = lane;
        float o[J][8];
        uint4 tv[J];
#pragma unroll
        for (int j = 0; j < J; ++j) tv[j] = sm[(chunk0 + 32 * j) * 33 + slot];
        rot8x<DT, J>(tv, o, A1, A2);
#pragma unroll
        for (int s = 1; s < J; s <<= 1) {
#pragma unroll
            for (int j = 0; j < J; ++j) {
                if (!(j & s)) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const float x = o[j][e], y = o[j | s][e];
                        o[j][e] = x + y;
                        o[j | s][e] = x - y;
                    }
                }
            }
        }
#pragma unroll
        for (int j = 0; j < J; ++j) {
            uint4 r;
            r.x = pack2<DT>(o[j][0] * mult, o[j][1] * mult);
            r.y = pack2<DT>(o[j][2] * mult, o[j][3] * mult);
            r.z = pack2<DT>(o[j][4] * mult, o[j][5] * mult);
            r.w = pack2<DT>(o[j][6] * mult, o[j][7] * mult);
            sm[(chunk0 + 32 * j) * 33 + slot] = r;
        }
    }
    if constexpr (LOCAL_OUT) {
        __syncwarp();
        // pass 3, warp-local: 32/SPW chunks x SPW slots per instruction, four instructions in flight
        constexpr int CPI = 32 / SPW;
        const int sub = lane % SPW, cl = lane / SPW;
        const int v0 = warp * SPW + sub;
        for (int c0 = 0; c0 < chunks_here; c0 += 4 * CPI) {
            uint4 r[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int c = c0 + u * CPI + cl;
                if (c < chunks_here) r[u] = sm[c * 33 + v0];
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int c = c0 + u * CPI + cl;
                if (c < chunks_here) st_out(gout + c * 32 + v0, r[u], keep_policy);
            }
        }
    } else {
        __syncthreads();
        for (int c = warp; c < chunks_here; c += NW) st_out(gout + c * 32 + lane, sm[c * 33 + lane], keep_policy);
    }
}

// ---------------------------------------------------------------------------
// n = 2, 4 (16-bit): one thread per row.
// ---------------------------------------------------------------------------
template <int DT>
__global__ void fwht_tiny_kernel(const uint16_t *in, uint16_t *out, uint64_t rows, int n, float scale,
                                 const uint16_t *signs)
{
    const uint64_t r = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    float v[4];
    for (int i = 0; i < n; ++i) {
        const uint32_t u = in[r * n + i] ^ (signs ? (uint32_t)signs[i] : 0u);
        v[i] = unpack2<DT>(u).x;
    }
    if (n == 2) {
        const float a = v[0], b = v[1];
        v[0] = a + b; v[1] = a - b;
    } else {
        const float a = v[0] + v[1], b = v[0] - v[1], c = v[2] + v[3], d = v[2] - v[3];
        v[0] = a + c; v[1] = b + d; v[2] = a - c; v[3] = b - d;
    }
    for (int i = 0; i < n; ++i) out[r * n + i] = to_b16<DT>(v[i] * scale);
}

// ---------------------------------------------------------------------------
// fp32: exact butterflies on a slab of max(n, 2048) floats in shared memory.
// ---------------------------------------------------------------------------
// With `split` set the result is not stored as fp32 but as the six-block bf16 row of the tensor-core contraction of
// fused_gemm.cu: every value y = y1 + y2 + y3 (three bf16 terms, exact), row layout [y3 y1 y2 y2 y1 y1], each block
// n elements long.
__global__ void __launch_bounds__(256) fwht_f32_kernel(const float *in, float *out, uint64_t rows,
                                                       int logn, int slab_rows, float scale, __nv_bfloat16 *split)
{
    extern __shared__ float sf[];
    const int n = 1 << logn;
    const uint64_t row0 = (uint64_t)blockIdx.x * slab_rows;
    const int rows_here = (int)((rows - row0) < (uint64_t)slab_rows ? (rows - row0) : (uint64_t)slab_rows);
    const int total = rows_here * n;
    const float *gin = in + row0 * n;
    float *gout = out + row0 * n;
    for (int i = threadIdx.x; i < total; i += blockDim.x) sf[i] = gin[i];
    __syncthreads();
    slab_fwht_f32(sf, total, logn, threadIdx.x, blockDim.x);
    if (!split) {
        for (int i = threadIdx.x; i < total; i += blockDim.x) gout[i] = sf[i] * scale;
        return;
    }
    __syncthreads();
    for (int i4 = threadIdx.x; i4 < total / 4; i4 += blockDim.x) {   // n >= 32 on this path: rows are multiples of 4
        const float4 v = ((const float4 *)sf)[i4];
        const float a[4] = {v.x * scale, v.y * scale, v.z * scale, v.w * scale};
        uint32_t h[3][4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float r = a[e];
#pragma unroll
            for (int j = 0; j < 3; ++j) {
                const __nv_bfloat16 b = __float2bfloat16_rn(r);
                h[j][e] = (uint32_t)__bfloat16_as_ushort(b);
                r -= __bfloat162float(b);
            }
        }
        uint2 t[3];
#pragma unroll
        for (int j = 0; j < 3; ++j) t[j] = make_uint2(h[j][0] | (h[j][1] << 16), h[j][2] | (h[j][3] << 16));
        const int idx = i4 * 4, row = idx >> logn, k = idx & (n - 1);
        __nv_bfloat16 *o = split + (row0 + row) * (uint64_t)(6 * n) + k;
        const int py[6] = {2, 0, 1, 1, 0, 0};
#pragma unroll
        for (int b = 0; b < 6; ++b) *(uint2 *)(o + (size_t)b * n) = t[py[b]];
    }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
template <int DT, int LOGN>
static int launch_reg(const void *in, void *out, uint64_t rows, float scale, const void *signs, cudaStream_t st, int keep)
{
    constexpr int P = LOGN < 8 ? LOGN : 8;
    constexpr int CPR = LOGN > 8 ? (1 << (LOGN - 8)) : 1;
    constexpr int GRP = CPR > 4 ? CPR : 4;
    const uint64_t total_vec = (rows << LOGN) >> 3;
    const uint64_t warps = (total_vec + GRP * 32 - 1) / (GRP * 32);
    const uint64_t blocks = (warps + 7) / 8;
    if (blocks > 0x7fffffffull) return B200HT_ERR_SIZE;
    const float f = hfrag_c(popc4(rot8_mask1(P))) * hfrag_c(popc4(rot8_mask2(P)));
    // programmatic dependent launch: the small sizes are bound by launch latency, and this lets the scheduling
    // of back-to-back launches overlap (the kernel itself waits for its predecessors before touching memory)
    if (signs)
        return launch_pdl(fwht_reg_kernel<DT, LOGN, true>, dim3((unsigned)blocks), dim3(256), 0, st,
                          (const uint4 *)in, (uint4 *)out, total_vec, scale / f, (const uint4 *)signs, keep);
    return launch_pdl(fwht_reg_kernel<DT, LOGN, false>, dim3((unsigned)blocks), dim3(256), 0, st, (const uint4 *)in,
                      (uint4 *)out, total_vec, scale / f, (const uint4 *)nullptr, keep);
}

template <int DT, int LOGN>
static int launch_smem(const void *in, void *out, uint64_t rows, float scale, const void *signs, cudaStream_t st, int keep)
{
    using Cfg = SmemCfg<LOGN>;
    const uint64_t blocks = (rows + Cfg::SLAB_ROWS - 1) / Cfg::SLAB_ROWS;
    if (blocks > 0x7fffffffull) return B200HT_ERR_SIZE;
    auto go = [&](auto kernel) -> int {
        const int rc = ensure_dyn_smem((const void *)kernel, Cfg::SMEM_BYTES);
        if (rc) return rc;
        return launch_pdl(kernel, dim3((unsigned)blocks), dim3(Cfg::NW * 32), (size_t)Cfg::SMEM_BYTES, st,
                          (const uint4 *)in, (uint4 *)out, rows, scale * 64.0f, (const uint4 *)signs, keep);
    };
    return signs ? go(fwht_smem_kernel<DT, LOGN, true>) : go(fwht_smem_kernel<DT, LOGN, false>);
}

template <int DT>
static int launch_b16(const void *in, void *out, uint64_t rows, int logn, float scale, const void *signs, int keep,
                      cudaStream_t st)
{
    switch (logn) {
    case 1:
    case 2: {
        const uint64_t blocks = (rows + 255) / 256;
        if (blocks > 0x7fffffffull) return B200HT_ERR_SIZE;
        note_launch();
        fwht_tiny_kernel<DT><<<(unsigned)blocks, 256, 0, st>>>((const uint16_t *)in, (uint16_t *)out, rows,
                                                              1 << logn, scale, (const uint16_t *)signs);
        return (int)cudaGetLastError();
    }
    case 3: return launch_reg<DT, 3>(in, out, rows, scale, signs, st, keep);
    case 4: return launch_reg<DT, 4>(in, out, rows, scale, signs, st, keep);
    case 5: return launch_reg<DT, 5>(in, out, rows, scale, signs, st, keep);
    case 6: return launch_reg<DT, 6>(in, out, rows, scale, signs, st, keep);
    case 7: return launch_reg<DT, 7>(in, out, rows, scale, signs, st, keep);
    case 8: return launch_reg<DT, 8>(in, out, rows, scale, signs, st, keep);
    case 9: return launch_reg<DT, 9>(in, out, rows, scale, signs, st, keep);
    case 10: return launch_reg<DT, 10>(in, out, rows, scale, signs, st, keep);
    case 11: return launch_reg<DT, 11>(in, out, rows, scale, signs, st, keep);
    case 12: return launch_smem<DT, 12>(in, out, rows, scale, signs, st, keep);
    case 13: return launch_smem<DT, 13>(in, out, rows, scale, signs, st, keep);
    case 14: return launch_smem<DT, 14>(in, out, rows, scale, signs, st, keep);
    case 15: return launch_smem<DT, 15>(in, out, rows, scale, signs, st, keep);
    }
    return B200HT_ERR_SIZE;
}

int launch_fwht_f32(const float *in, float *out, uint64_t rows, int logn, float scale, cudaStream_t st,
                    __nv_bfloat16 *split = nullptr)
{
    const int n = 1 << logn;
    const int slab = n >= 2048 ? n : 2048;
    const int slab_rows = slab / n;
    const uint64_t blocks = (rows + slab_rows - 1) / slab_rows;
    if (blocks > 0x7fffffffull) return B200HT_ERR_SIZE;
    const int smem = slab * 4;
    const int rc = ensure_dyn_smem((const void *)fwht_f32_kernel, smem);
    if (rc) return rc;
    note_launch();
    fwht_f32_kernel<<<(unsigned)blocks, 256, smem, st>>>(in, out, rows, logn, slab_rows, scale, split);
    return (int)cudaGetLastError();
}

// fp32 transform whose result goes straight into the split bf16 operand of the tensor-core contraction
int launch_fwht_f32_split(const float *in, __nv_bfloat16 *split, uint64_t rows, uint32_t n, float scale, cudaStream_t st)
{
    return launch_fwht_f32(in, nullptr, rows, ilog2(n), scale, st, split);
}

// keep_out != 0: the result is about to be read again (by the contraction of the fused GEMM): store it with the L2
// eviction priority `evict_last` instead of as a stream.
int launch_fwht(const void *in, void *out, uint64_t rows, uint32_t n, int dtype, float scale, const void *signs,
                cudaStream_t st, int keep_out)
{
    const int logn = ilog2(n);
    if (dtype == B200HT_F32 && signs) return B200HT_ERR_DTYPE;  // the +-1 diagonal is implemented for 16-bit data
    if (dtype == B200HT_F32) return launch_fwht_f32((const float *)in, (float *)out, rows, logn, scale, st);
    // n = 32768: tcgen05 kernel (fwht_tcgen05.cu; needs 128-byte aligned pointers for TMA).  It is correct for
    // every n >= 256; B200HT_FWHT_TC_MIN=<log2 n> lowers the threshold, B200HT_FWHT_MMA_SYNC=1 disables it.
    static const int kTcMinLogN = tc_min_logn();
    static const bool use_mma_sync = [] {
        const char *e = std::getenv("B200HT_FWHT_MMA_SYNC");
        return e && e[0] == '1';
    }();
    if (logn >= kTcMinLogN && !use_mma_sync && !signs && ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 127u) == 0)
        return launch_fwht_tc(in, out, rows, logn, dtype, scale, st);
    if (dtype == B200HT_BF16) return launch_b16<B200HT_BF16>(in, out, rows, logn, scale, signs, keep_out, st);
    return launch_b16<B200HT_F16>(in, out, rows, logn, scale, signs, keep_out, st);
}

}  // namespace b200ht

static int fwht_entry(const void *in, void *out, uint64_t rows, uint32_t n, int dtype, float scale, const void *signs,
                      void *stream)
{
    using namespace b200ht;
    if (dtype != B200HT_F16 && dtype != B200HT_BF16 && dtype != B200HT_F32) return B200HT_ERR_DTYPE;
    if (signs && dtype == B200HT_F32) return B200HT_ERR_DTYPE;
    if (!is_pow2(n) || n < 2 || n > (1u << kMaxLogN)) return B200HT_ERR_SIZE;
    if (rows == 0) return 0;
    if (!in || !out) return B200HT_ERR_NULL;
    if (!aligned16(in) || !aligned16(out) || (signs && !aligned16(signs))) return B200HT_ERR_ALIGN;
    const uint64_t esz = dtype == B200HT_F32 ? 4 : 2;
    if (rows > (~0ull) / ((uint64_t)n * esz)) return B200HT_ERR_SIZE;
    const uint64_t bytes = rows * n * esz;
    if (in != out) {
        const uintptr_t a = (uintptr_t)in, b = (uintptr_t)out;
        if (a < b + bytes && b < a + bytes) return B200HT_ERR_OVERLAP;
    }
    int rc = check_device();
    if (rc) return rc;
    return launch_fwht(in, out, rows, n, dtype, scale, signs, (cudaStream_t)stream, 0);
}

extern "C" int b200ht_fwht(const void *in, void *out, uint64_t rows, uint32_t n, int dtype, float scale,
                           void *stream)
{
    return fwht_entry(in, out, rows, n, dtype, scale, nullptr, stream);
}

extern "C" int b200ht_fwht_signed(const void *in, void *out, uint64_t rows, uint32_t n, int dtype, float scale,
                                  const void *signs, void *stream)
{
    if (!signs) return B200HT_ERR_NULL;
    return fwht_entry(in, out, rows, n, dtype, scale, signs, stream);
}
