// Shared device/host helpers of the b200ht library (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b200ht.h"

#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ < 1000)
#error "b200ht is written for sm_100a only"
#endif

namespace b200ht {

constexpr int kMaxLogN = 15;

__host__ __device__ constexpr bool is_pow2(uint64_t x) { return x && !(x & (x - 1)); }

inline int ilog2(uint32_t x)
{
    int l = 0;
    while ((1u << l) < x) ++l;
    return l;
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Device status word: 0 or a B200HT_ERR_* code written by a kernel whose bounded
// wait expired.  One per device context that loaded the library.  Kernels get
// its device address as an argument (the variable lives in api.cu).
int *status_word_ptr();  // device address of the status word on the current device

// Checks (once per device) that the current device is compute capability 10.x.
int check_device();
// Number of SMs of the current device (cached per device).
int sm_count();
// Raises the dynamic shared-memory limit of `func` to `bytes` on the current device; the runtime is asked only when
// the cached limit is lower.
int ensure_dyn_smem(const void *func, int bytes);

// Launch with programmatic stream serialization (programmatic dependent launch): the
// kernel may be scheduled while its predecessor in the stream is still draining.  Every
// kernel launched this way executes pdl_wait() before it touches global memory, which
// blocks until all earlier work of the stream has completed and is visible, and
// pdl_launch_dependents() as early as it likes.
// Every kernel launch of the library is counted (b200ht_launch_count reports the total).
void note_launch();

template <typename... KArgs, typename... Args>
inline int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args)
{
    note_launch();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
#endif

// ---------------------------------------------------------------------------
// 16-bit packing
// ---------------------------------------------------------------------------
template <int DT>
__device__ __forceinline__ uint32_t pack2(float lo, float hi)
{
    if constexpr (DT == B200HT_BF16) {
        __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t *>(&v);
    } else {
        __half2 v = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t *>(&v);
    }
}

template <int DT>
__device__ __forceinline__ float2 unpack2(uint32_t u)
{
    if constexpr (DT == B200HT_BF16) {
        return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162 *>(&u));
    } else {
        return __half22float2(*reinterpret_cast<__half2 *>(&u));
    }
}

template <int DT>
__device__ __forceinline__ uint16_t to_b16(float x)
{
    if constexpr (DT == B200HT_BF16) {
        __nv_bfloat16 v = __float2bfloat16_rn(x);
        return *reinterpret_cast<uint16_t *>(&v);
    } else {
        __half v = __float2half_rn(x);
        return *reinterpret_cast<uint16_t *>(&v);
    }
}

// ---------------------------------------------------------------------------
// mma.sync m16n8k16 (fp32 accumulate) and constant Hadamard A-fragments.
// Fragment ownership for lane = 4*g + t (PTX ISA, m16n8k16 .f16/.bf16):
//   A (16x16, row): a0 = (g, 2t..2t+1)  a1 = (g+8, 2t..)  a2 = (g, 2t+8..)  a3 = (g+8, 2t+8..)
//   B (16x8,  col): b0 = (k 2t..2t+1, n g)              b1 = (k 2t+8..2t+9, n g)
//   D (16x8)      : d0,d1 = (g, 2t..2t+1)               d2,d3 = (g+8, 2t..2t+1)
// ---------------------------------------------------------------------------
template <int DT>
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1)
{
    if constexpr (DT == B200HT_BF16) {
        asm(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
            "{%8,%9}, {%10,%10,%10,%10};\n"
            : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
    } else {
        asm(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
            "{%8,%9}, {%10,%10,%10,%10};\n"
            : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
    }
}

// d += a . b, bf16 operands, fp32 accumulators.
__device__ __forceinline__ void mma16816_bf16_acc(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                  uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Entry (m, k) of the 16x16 matrix  (x)_{bit i}  [ H_2 if hmask bit i else I_2 ],
// times c:  +-c where the Hadamard bits decide the sign, 0 where an identity bit
// of m and k differs.
__device__ __forceinline__ float hmat_entry(int m, int k, unsigned hmask, float c)
{
    unsigned diff = (unsigned)(m ^ k) & ~hmask & 15u;
    if (diff) return 0.f;
    unsigned sgn = __popc((unsigned)(m & k) & hmask) & 1u;
    return sgn ? -c : c;
}

template <int DT>
__device__ __forceinline__ void make_hfrag(uint32_t (&a)[4], int lane, unsigned hmask, float c)
{
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int m = g + ((r & 1) ? 8 : 0);
        const int k = 2 * t + ((r & 2) ? 8 : 0);
        a[r] = pack2<DT>(hmat_entry(m, k, hmask, c), hmat_entry(m, k + 1, hmask, c));
    }
}

// 256-point transform step on a warp-resident chunk.  Each lane holds 8
// consecutive 16-bit elements of a 256-element chunk (lane l owns elements
// 8l..8l+7) packed in v[0..3].  With element index bits m0..m7 (m0..m2 inside
// the lane, m3..m7 = lane bits), the first pair of mma contracts the index bits
// (m0, m3, m4, m1) and the second pair (m5, m6, m7, m2); the data never leaves
// the lane layout it was loaded in, so o[0..7] are the same 8 element positions.
// A1/A2 choose which of those bits get a Hadamard factor and which pass through.
template <int DT>
__device__ __forceinline__ void rot8(const uint32_t (&v)[4], float (&o)[8], const uint32_t (&A1)[4],
                                     const uint32_t (&A2)[4])
{
    float c0[4], c1[4], d0[4], d1[4];
    mma16816<DT>(c0, A1, v[0], v[1]);
    mma16816<DT>(c1, A1, v[2], v[3]);
    const uint32_t p00 = pack2<DT>(c0[0], c0[1]), p01 = pack2<DT>(c0[2], c0[3]);
    const uint32_t p10 = pack2<DT>(c1[0], c1[1]), p11 = pack2<DT>(c1[2], c1[3]);
    mma16816<DT>(d0, A2, p00, p10);
    mma16816<DT>(d1, A2, p01, p11);
    o[0] = d0[0]; o[1] = d0[1]; o[2] = d1[0]; o[3] = d1[1];
    o[4] = d0[2]; o[5] = d0[3]; o[6] = d1[2]; o[7] = d1[3];
}

// rot8 on CNT independent chunks at once, written stage by stage so that the
// 2*CNT mma of a stage are independent and their latencies overlap.
template <int DT, int CNT>
__device__ __forceinline__ void rot8x(const uint4 (&v)[CNT], float (&o)[CNT][8], const uint32_t (&A1)[4],
                                      const uint32_t (&A2)[4])
{
    float c[CNT][2][4];
#pragma unroll
    for (int i = 0; i < CNT; ++i) {
        mma16816<DT>(c[i][0], A1, v[i].x, v[i].y);
        mma16816<DT>(c[i][1], A1, v[i].z, v[i].w);
    }
    uint32_t p[CNT][4];
#pragma unroll
    for (int i = 0; i < CNT; ++i) {
        p[i][0] = pack2<DT>(c[i][0][0], c[i][0][1]);
        p[i][1] = pack2<DT>(c[i][0][2], c[i][0][3]);
        p[i][2] = pack2<DT>(c[i][1][0], c[i][1][1]);
        p[i][3] = pack2<DT>(c[i][1][2], c[i][1][3]);
    }
    float d[CNT][2][4];
#pragma unroll
    for (int i = 0; i < CNT; ++i) {
        mma16816<DT>(d[i][0], A2, p[i][0], p[i][2]);
        mma16816<DT>(d[i][1], A2, p[i][1], p[i][3]);
    }
#pragma unroll
    for (int i = 0; i < CNT; ++i) {
        o[i][0] = d[i][0][0]; o[i][1] = d[i][0][1]; o[i][2] = d[i][1][0]; o[i][3] = d[i][1][1];
        o[i][4] = d[i][0][2]; o[i][5] = d[i][0][3]; o[i][6] = d[i][1][2]; o[i][7] = d[i][1][3];
    }
}

// Hadamard masks of rot8 for a transform over the low `p` (<= 8) index bits.
__host__ __device__ constexpr unsigned rot8_mask1(int p)
{
    return (0 < p ? 1u : 0u) | (3 < p ? 2u : 0u) | (4 < p ? 4u : 0u) | (1 < p ? 8u : 0u);
}
__host__ __device__ constexpr unsigned rot8_mask2(int p)
{
    return (5 < p ? 1u : 0u) | (6 < p ? 2u : 0u) | (7 < p ? 4u : 0u) | (2 < p ? 8u : 0u);
}
__host__ __device__ constexpr int popc4(unsigned m) { return (m & 1) + ((m >> 1) & 1) + ((m >> 2) & 1) + ((m >> 3) & 1); }
// Power-of-two magnitude stored in an A-fragment with h Hadamard bits: 2^-(h/2).
__host__ __device__ constexpr float hfrag_c(int h) { return h >= 4 ? 0.25f : (h >= 2 ? 0.5f : 1.0f); }

__device__ __forceinline__ uint4 ld_stream(const uint4 *p)
{
    uint4 v;
    asm volatile("ld.global.cs.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ void st_stream(uint4 *p, const uint4 &v)
{
    asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
                 "r"(v.w)
                 : "memory");
}

// L2 eviction-priority policies for accesses that carry a cache hint: `evict_first` for data that streams through
// once, `evict_last` for data that should stay resident.
__device__ __forceinline__ uint64_t l2_policy_evict_first()
{
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;\n" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last()
{
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;\n" : "=l"(p));
    return p;
}
// 16-byte result store: as a stream (policy 0), or with the given L2 policy.
__device__ __forceinline__ void st_out(uint4 *p, const uint4 &v, uint64_t policy)
{
    if (policy == 0) {
        st_stream(p, v);
    } else {
        asm volatile("st.global.L2::cache_hint.v4.u32 [%0], {%1,%2,%3,%4}, %5;\n" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
                     "r"(v.w), "l"(policy)
                     : "memory");
    }
}

}  // namespace b200ht
