// Small-batch fused Y = W . H(X).  Replaces fused_hadamard_gemv_kernel(_vec)
// (fused_ht/fwht_gemv_fusion.cu:98-244).
//
// The reference launches one block per column of X, so W is streamed B times.
// Here the grid runs over ROWS of W: every CTA transforms the (tiny) X once
// into shared memory, then streams its rows of W exactly once with 16-byte
// loads and multiplies them against all B columns at the same time.  Bound:
// HBM traffic of W (M*N*2 bytes for bf16).
//
//   bf16, 256 <= N <= 8192: gemv_bf16_stream_kernel (the fast path, below).
//   bf16, other N: gemv_bf16_kernel: H(X) in shared memory as bf16 after an fp32
//         transform; a lane loads 8 consecutive k of one W row (16 bytes) and
//         the same 8 k of H(X) for the B operand of mma.sync, so the two mma of
//         a 32-wide k block see one consistent permutation of k.
//   fp32: exact FFMA path (correctness cases), one warp per row.
#include <cstdlib>
#include <cstring>

#include "tc_common.cuh"
#include "fwht_f32.cuh"

namespace b200ht {

int gemv_tc_cols_max(int N, int B);
int launch_gemv_tc(const void *W, const void *X, void *Y, int M, int N, int logn, int B, int b0, int Bg, int out_dtype,
                   float scale, cudaStream_t st);

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
// bf16, 256 <= N <= 8192: the fast path.  16 warps per CTA, one CTA per SM,
// every CTA owns a contiguous, balanced range of rows of W.
//
//  * As soon as every warp has issued its loads of X (requests of one SM are
//    served in order, and X must not queue behind W) the CTA streams its rows
//    of W into a shared-memory ring with TMA tile loads, the first sixteen
//    issued by sixteen lanes at once (cp.async.bulk.tensor.3d over a [64 k][rows][N/64]
//    view of W: one op brings all rows of a row group x 256..1024 k as
//    consecutive 128-byte-swizzled K-major tiles; completion is counted on an
//    mbarrier per stage).  The copies hold no registers and no LSU slots, so HBM
//    traffic runs underneath the transform of X and only pauses when the ring
//    is full.
//  * Meanwhile the warps transpose X (N x B, b fastest) into shared memory as
//    one row of N bf16 per column (row pitch N*2+16 bytes) and transform the
//    rows there, so the cost of the transform follows the number of columns:
//    pass A sends the low eight index bits of each 256-element chunk through
//    rot8 (tensor cores) and up to two more through fp32 register butterflies;
//    pass B finishes the remaining (at most three) bits with fp32 butterflies
//    over 16-byte vectors.
//  * Then the warps consume the ring in four groups of four warps.  A group
//    takes whole ring items (every fourth), so four items are in work at the
//    same time and the fixed cost of an item (barrier wait, release) is spread
//    over eight k steps per warp.  Per k step a warp loads the 16 x 16 blocks of
//    both row tiles with ldmatrix (A operand), the matching H(X) values with two
//    32-bit loads per column tile (B operand: column g, k = 2t.. and 2t+8..) and
//    issues mma.sync m16n8k16 with fp32 accumulators kept over the whole K
//    range.  Warps release a stage through a shared counter and the last one to
//    do so refills it at once, so no warp waits for another; the partial sums
//    are reduced through shared memory once per row group.
// The row pitch of H(X) puts column g+1 four banks after column g, so the 32
// lanes of a B-operand load (8 columns x 4 k pairs) hit 32 different banks.
// ---------------------------------------------------------------------------
constexpr int GV_WARPS = 16;
constexpr int GV_THREADS = GV_WARPS * 32;
// The consume phase runs in warp groups of GW warps (template parameter of the kernel), each on a ring item of its
// own: four groups of four, or two groups of eight for a long stream with 8 x 64 k per item (the host's plan says
// which and why).
constexpr int GV_MAX_GROUP_ROWS = 32;                // rows of W per ring stage (one or two 16-row tiles)

__host__ __device__ constexpr int hxt_pitch(int N) { return N * 2 + 16; }   // bytes per column of H(X)

// Pass A of the in-place transform: index bits 0..7 (rot8) and 8..8+RB-1 (registers) of every group of
// GRP = 2^RB consecutive 256-element chunks; `mult` is applied to the result.
template <int RB>
__device__ __forceinline__ void hxt_pass_a(unsigned char *hxT, int cols, int pitch, int logn, float mult, int warp,
                                           int lane)
{
    constexpr int GRP = 1 << RB;
    uint32_t A1[4], A2[4];
    constexpr unsigned M1 = rot8_mask1(8), M2 = rot8_mask2(8);
    make_hfrag<B200HT_BF16>(A1, lane, M1, hfrag_c(popc4(M1)));
    make_hfrag<B200HT_BF16>(A2, lane, M2, hfrag_c(popc4(M2)));
    const int gpr = 1 << (logn - 8 - RB);            // chunk groups per column
    const int ntasks = cols * gpr;
    for (int task = warp; task < ntasks; task += GV_WARPS) {
        const int col = task / gpr, gi = task - col * gpr;
        uint4 *base = (uint4 *)(hxT + (size_t)col * pitch) + (size_t)gi * (GRP * 32) + lane;
        uint4 v[GRP];
#pragma unroll
        for (int u = 0; u < GRP; ++u) v[u] = base[u * 32];
        float o[GRP][8];
        rot8x<B200HT_BF16, GRP>(v, o, A1, A2);
#pragma unroll
        for (int s = 1; s < GRP; s <<= 1) {
#pragma unroll
            for (int u = 0; u < GRP; ++u) {
                if (!(u & s)) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const float x = o[u][e], y = o[u | s][e];
                        o[u][e] = x + y;
                        o[u | s][e] = x - y;
                    }
                }
            }
        }
#pragma unroll
        for (int u = 0; u < GRP; ++u) {
            uint4 r;
            r.x = pack2<B200HT_BF16>(o[u][0] * mult, o[u][1] * mult);
            r.y = pack2<B200HT_BF16>(o[u][2] * mult, o[u][3] * mult);
            r.z = pack2<B200HT_BF16>(o[u][4] * mult, o[u][5] * mult);
            r.w = pack2<B200HT_BF16>(o[u][6] * mult, o[u][7] * mult);
            base[u * 32] = r;
        }
    }
}

// Pass B: the top JB index bits, as fp32 butterflies over 2^JB vectors that sit 2^(logn-JB) elements apart.
template <int JB>
__device__ __forceinline__ void hxt_pass_b(unsigned char *hxT, int cols, int pitch, int logn, float mult, int tid)
{
    constexpr int J = 1 << JB;
    const int vps = 1 << (logn - JB - 3);            // vectors per sub-block
    const int ntasks = cols * vps;
    for (int task = tid; task < ntasks; task += GV_THREADS) {
        const int col = task / vps, p = task - col * vps;
        uint4 *base = (uint4 *)(hxT + (size_t)col * pitch) + p;
        float o[J][8];
#pragma unroll
        for (int j = 0; j < J; ++j) {
            const uint4 v = base[(size_t)j * vps];
            const float2 a = unpack2<B200HT_BF16>(v.x), b = unpack2<B200HT_BF16>(v.y),
                         c = unpack2<B200HT_BF16>(v.z), d = unpack2<B200HT_BF16>(v.w);
            o[j][0] = a.x; o[j][1] = a.y; o[j][2] = b.x; o[j][3] = b.y;
            o[j][4] = c.x; o[j][5] = c.y; o[j][6] = d.x; o[j][7] = d.y;
        }
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
            r.x = pack2<B200HT_BF16>(o[j][0] * mult, o[j][1] * mult);
            r.y = pack2<B200HT_BF16>(o[j][2] * mult, o[j][3] * mult);
            r.z = pack2<B200HT_BF16>(o[j][4] * mult, o[j][5] * mult);
            r.w = pack2<B200HT_BF16>(o[j][6] * mult, o[j][7] * mult);
            base[(size_t)j * vps] = r;
        }
    }
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t saddr)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(saddr));
}
__device__ __forceinline__ uint32_t lds32(uint32_t saddr)
{
    uint32_t v;
    asm volatile("ld.shared.b32 %0, [%1];\n" : "=r"(v) : "r"(saddr));
    return v;
}

// Row-sharded GEMV across GPUs: besides its own rows of Y the kernel sends every result, tagged with the number of the
// call, into a slot array on each of up to seven peer GPUs (plain 8-byte stores through peer-mapped pointers, no
// multicast), and collects the peers' rows from its own slot array into the full result.  n = 0: single-GPU call.
struct PeerOut {
    int n;                              // peers (0: an ordinary single-GPU call)
    unsigned long long *slots[7];       // the peers' slot arrays of this call (index: row of the full result * B + column)
    const unsigned long long *my_slots; // this GPU's slot array, filled by the peers
    void *y_full;                       // this GPU's full result (all ranks' rows)
    unsigned int *local_count;          // 8-byte aligned pair: CTAs of this launch that have finished (self-resetting), calls made
    unsigned int target;                // number of this call = tag of its slots; 0: the number counted in local_count[1]
    int row_begin, rows_total;          // this rank's first row in the full result, rows of the full result
};

template <int NT, int GW>
__global__ void __launch_bounds__(GV_THREADS, 1)
gemv_bf16_stream_kernel(const __grid_constant__ CUtensorMap tmW, const __nv_bfloat16 *X, void *Y, int M, int N,
                        int logn, int B, int b0, int Bg, int out_dtype, float scale, int rows_per_cta,
                        int group_rows, int kc, int stage_bytes, int nstages, int red_in_ring, int *status,
                        const PeerOut po)
{
    extern __shared__ unsigned char smem_dyn[];
    // ring first (1024-byte aligned stages for the 128-byte swizzle), then H(X), reduction buffer, barriers
    const uint32_t ring_s = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    unsigned char *gen = smem_dyn + (ring_s - smem_u32(smem_dyn));
    const int pitch = hxt_pitch(N);
    unsigned char *hxT = gen + (size_t)nstages * stage_bytes;                     // [Bg][pitch]
    // reduction buffer [8 warps][32 rows][NT*8]: its own space, or (red_in_ring, one row group per CTA only) the
    // start of the ring, which is idle by the time the single reduction runs
    unsigned char *after_hx = hxT + (((size_t)Bg * pitch + 127) & ~(size_t)127);
    float *red = red_in_ring ? (float *)gen : (float *)after_hx;
    unsigned char *bar_mem = after_hx + (red_in_ring ? 0 : (GV_WARPS / 2) * 32 * NT * 8 * 4);  // full[], counters, abort
    const uint32_t bar_s = smem_u32(bar_mem);
    int *released = (int *)(bar_mem + 8 * nstages);                               // warps done with stage s
    volatile int *abort_flag = (volatile int *)(bar_mem + 16 * nstages);
    auto full_bar = [&](int s) { return bar_s + 8u * s; };

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    // rows of W owned by this CTA, in groups of group_rows; one ring item = (group, 64*kc-wide k chunk)
    const int row_begin = blockIdx.x * rows_per_cta;
    const int row_end = (row_begin + rows_per_cta) < M ? (row_begin + rows_per_cta) : M;
    const int my_rows = row_end > row_begin ? row_end - row_begin : 0;
    const int ngroups = (my_rows + group_rows - 1) / group_rows;
    const int nchunks = (N / 64) / kc;     // ring items per row group
    const int total_items = ngroups * nchunks;

    if (tid == 0) {
        for (int s = 0; s < nstages; ++s) {
            mbar_init(full_bar(s), 1);
            released[s] = 0;
        }
        *abort_flag = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tmW);
    }
    __syncthreads();
    // Programmatic dependent launch: the barrier set-up above overlaps the predecessor's tail, and so does a
    // prefetch of X into L2 (a hint that returns no data, so it may run before the predecessor's writes are
    // visible; it warms the address translation for the loads below).
    pdl_launch_dependents();
    {
        const size_t xbytes = (size_t)N * B * 2;
        for (size_t off = (size_t)tid * 128; off < xbytes; off += (size_t)GV_THREADS * 128)
            asm volatile("prefetch.global.L2 [%0];\n" ::"l"((const unsigned char *)X + off));
    }
    pdl_wait();
    // row-sharded call: the number of the call tags every value sent to a peer (read now, used at the end)
    unsigned int tag = po.target;
    if (po.n && tag == 0u) {
        asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];\n" : "=r"(tag) : "l"(po.local_count + 1) : "memory");
        tag += 1u;
    }

    // one TMA op per ring item: group_rows x (64*kc) elements of W (issued by one thread)
    auto issue = [&](int item) {
        const int s = item % nstages;
        const int grp = item / nchunks, chunk = item - grp * nchunks;
        mbar_expect_tx(full_bar(s), (uint32_t)(group_rows * kc * 128));
        tma_load_3d(ring_s + (uint32_t)(s * stage_bytes), &tmW, 0, row_begin + grp * group_rows, chunk * kc,
                    full_bar(s));
    };
    // The first stages of the ring are requested by 16 lanes at once -- but only after every warp has issued its
    // first batch of X loads (below): requests of one SM are served in order, and X must not queue behind the
    // ring's first fill.
    auto start_stream = [&]() {
        __syncthreads();
        if (warp == 0 && lane < (total_items < nstages ? total_items : nstages)) issue(lane);   // nstages <= 16
    };

    // ------------------------------ X^T into shared memory ------------------------------
    // Every path issues all loads of a batch before the first store: a round trip to memory is long while the
    // ring is filling, so the copy should cost one of them.
    if (B == 1) {
        const uint4 *Xv = (const uint4 *)X;
        for (int base = 0; base < N / 8; base += GV_THREADS * 2) {
            uint4 r[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int v = base + u * GV_THREADS + tid;
                if (v < N / 8) r[u] = __ldg(Xv + v);
            }
            if (base == 0) start_stream();
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int v = base + u * GV_THREADS + tid;
                if (v < N / 8) ((uint4 *)hxT)[v] = r[u];
            }
        }
    } else if (B == 2) {
        // 16 bytes = rows k..k+3 of both columns
        const uint4 *Xv = (const uint4 *)X;
        for (int base = 0; base < N / 4; base += GV_THREADS * 4) {
            uint4 r[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int v = base + u * GV_THREADS + tid;
                if (v < N / 4) r[u] = __ldg(Xv + v);
            }
            if (base == 0) start_stream();
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int v = base + u * GV_THREADS + tid;
                const uint4 x = r[u];
                if (v < N / 4) {
                    *(uint2 *)(hxT + v * 8) = make_uint2(__byte_perm(x.x, x.y, 0x5410), __byte_perm(x.z, x.w, 0x5410));
                    *(uint2 *)(hxT + pitch + v * 8) =
                        make_uint2(__byte_perm(x.x, x.y, 0x7632), __byte_perm(x.z, x.w, 0x7632));
                }
            }
        }
    } else if (B == 4) {
        // 32 bytes = rows k..k+3 of the four columns
        const uint4 *Xv = (const uint4 *)X;
        for (int base = 0; base < N / 4; base += GV_THREADS * 4) {
            uint4 rx[4], ry[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int v = base + u * GV_THREADS + tid;
                if (v < N / 4) { rx[u] = __ldg(Xv + 2 * v); ry[u] = __ldg(Xv + 2 * v + 1); }
            }
            if (base == 0) start_stream();
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int v = base + u * GV_THREADS + tid;
                const uint4 x = rx[u], y = ry[u];   // x: rows k, k+1; y: rows k+2, k+3
                if (v < N / 4) {
                    *(uint2 *)(hxT + v * 8) = make_uint2(__byte_perm(x.x, x.z, 0x5410), __byte_perm(y.x, y.z, 0x5410));
                    *(uint2 *)(hxT + pitch + v * 8) =
                        make_uint2(__byte_perm(x.x, x.z, 0x7632), __byte_perm(y.x, y.z, 0x7632));
                    *(uint2 *)(hxT + 2 * pitch + v * 8) =
                        make_uint2(__byte_perm(x.y, x.w, 0x5410), __byte_perm(y.y, y.w, 0x5410));
                    *(uint2 *)(hxT + 3 * pitch + v * 8) =
                        make_uint2(__byte_perm(x.y, x.w, 0x7632), __byte_perm(y.y, y.w, 0x7632));
                }
            }
        }
    } else if ((B & 7) == 0 && (b0 & 7) == 0 && (Bg & 7) == 0) {
        // two rows k, k+1 of one block of 8 columns per task: two 16-byte loads, eight 4-byte stores
        const uint4 *Xv = (const uint4 *)X;
        const int vpr = B >> 3, v0 = b0 >> 3, nb8 = Bg >> 3;
        const int ntasks = (N / 2) * nb8;
        for (int base = 0; base < ntasks; base += GV_THREADS * 8) {
            uint4 r0[8], r1[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int idx = base + u * GV_THREADS + tid;
                const int kp = idx / nb8, cb = idx - kp * nb8;
                if (idx < ntasks) {
                    r0[u] = __ldg(Xv + (size_t)(2 * kp) * vpr + v0 + cb);
                    r1[u] = __ldg(Xv + (size_t)(2 * kp + 1) * vpr + v0 + cb);
                }
            }
            if (base == 0) start_stream();
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int idx = base + u * GV_THREADS + tid;
                const int kp = idx / nb8, cb = idx - kp * nb8;
                if (idx < ntasks) {
                    const uint32_t w0[4] = {r0[u].x, r0[u].y, r0[u].z, r0[u].w};
                    const uint32_t w1[4] = {r1[u].x, r1[u].y, r1[u].z, r1[u].w};
                    unsigned char *dst = hxT + (size_t)(cb * 8) * pitch + kp * 4;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        *(uint32_t *)(dst + (size_t)(2 * j) * pitch) = __byte_perm(w0[j], w1[j], 0x5410);
                        *(uint32_t *)(dst + (size_t)(2 * j + 1) * pitch) = __byte_perm(w0[j], w1[j], 0x7632);
                    }
                }
            }
        }
    } else {
        const unsigned short *Xs = (const unsigned short *)X;
        const int ntasks = (N / 2) * Bg;
        for (int base = 0; base < ntasks; base += GV_THREADS * 8) {
            uint32_t lo[8], hi[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int idx = base + u * GV_THREADS + tid;
                const int kp = idx / Bg, c = idx - kp * Bg;
                if (idx < ntasks) {
                    lo[u] = __ldg(Xs + (size_t)(2 * kp) * B + b0 + c);
                    hi[u] = __ldg(Xs + (size_t)(2 * kp + 1) * B + b0 + c);
                }
            }
            if (base == 0) start_stream();
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int idx = base + u * GV_THREADS + tid;
                const int kp = idx / Bg, c = idx - kp * Bg;
                if (idx < ntasks) *(uint32_t *)(hxT + (size_t)c * pitch + kp * 4) = lo[u] | (hi[u] << 16);
            }
        }
    }
    __syncthreads();
    {
        // pass A covers 8 + ra bits, pass B the remaining jb (N <= 8192: jb <= 3)
        const int ra = logn - 8 < 2 ? logn - 8 : 2;
        const int jb = logn - 8 - ra;
        constexpr float fa = hfrag_c(popc4(rot8_mask1(8))) * hfrag_c(popc4(rot8_mask2(8)));
        const float mult_a = jb == 0 ? scale / fa : 1.f;
        if (ra == 0) hxt_pass_a<0>(hxT, Bg, pitch, logn, mult_a, warp, lane);
        else if (ra == 1) hxt_pass_a<1>(hxT, Bg, pitch, logn, mult_a, warp, lane);
        else hxt_pass_a<2>(hxT, Bg, pitch, logn, mult_a, warp, lane);
        __syncthreads();
        if (jb == 1) hxt_pass_b<1>(hxT, Bg, pitch, logn, scale / fa, tid);
        else if (jb == 2) hxt_pass_b<2>(hxT, Bg, pitch, logn, scale / fa, tid);
        else if (jb == 3) hxt_pass_b<3>(hxT, Bg, pitch, logn, scale / fa, tid);
        if (jb) __syncthreads();
    }

    // ------------------------------ consume the ring ------------------------------
    const int g = lane >> 2, t = lane & 3;
    const uint32_t hx_s = smem_u32(hxT);
    const int rt = group_rows > 16 ? 2 : 1;               // 16-row tiles per row group
    constexpr int GROUPS = GV_WARPS / GW;
    const int wg = warp / GW, wj = warp - wg * GW;   // warp group, warp within the group
    // ldmatrix (A): lane -> (row, 16-byte k chunk) of a 16 x 16 block, 128-byte swizzle of the TMA tile
    const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8;
    const int a_chunk = lane >> 4;
    // B operand: column nt*8+g of H(X) (zero beyond Bg), k pairs 2t and 2t+8 of the k step
    uint32_t b_addr[NT];
    bool b_ok[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const int col = nt * 8 + g;
        b_ok[nt] = col < Bg;
        b_addr[nt] = hx_s + (uint32_t)((b_ok[nt] ? col : 0) * pitch) + (uint32_t)(4 * t);
    }
    constexpr int RC = NT * 8;
    constexpr int UNR = NT <= 2 ? 4 : 2;
    const int ksteps = kc * 4;
    for (int grp = 0; grp < ngroups; ++grp) {
        float acc[2][NT][4];
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) acc[h][nt][0] = acc[h][nt][1] = acc[h][nt][2] = acc[h][nt][3] = 0.f;
        // Items are dealt to the warp groups by item number, and the number of stages is a multiple of the number
        // of groups: a stage is always consumed by the same group, so its warps see every phase of its barrier
        // (a one-bit phase parity cannot tell "not yet filled" from "filled twice since").
        const int first = grp * nchunks;
        for (int item = first + ((wg - first) & (GROUPS - 1)); item < first + nchunks; item += GROUPS) {
            const int chunk = item - first;
            const int s = item % nstages;
            const uint32_t ph = (uint32_t)(item / nstages) & 1u;
            if (!mbar_wait(full_bar(s), ph, abort_flag, status)) return;
            const uint32_t stage = ring_s + (uint32_t)(s * stage_bytes);
            // this warp's k steps of the item, UNR at a time: all fragment loads first, then the products
            for (int ks0 = wj; ks0 < ksteps; ks0 += GW * UNR) {
                uint32_t a[UNR][2][4], b[UNR][NT][2];
#pragma unroll
                for (int u = 0; u < UNR; ++u) {
                    const int ks = ks0 + u * GW;
                    if (ks < ksteps) {
                        const int c = ks >> 2, ks4 = ks & 3;
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            if (h < rt) {
                                const int rowidx = c * group_rows + h * 16 + a_row;
                                ldmatrix_x4(a[u][h], stage + (uint32_t)(rowidx * 128) +
                                                         (uint32_t)((((ks4 * 2 + a_chunk) ^ rowidx) & 7) << 4));
                            }
                        }
                        const uint32_t koff = (uint32_t)(((chunk * kc + c) * 64 + ks4 * 16) * 2);
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) {
                            b[u][nt][0] = b_ok[nt] ? lds32(b_addr[nt] + koff) : 0u;
                            b[u][nt][1] = b_ok[nt] ? lds32(b_addr[nt] + koff + 16) : 0u;
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < UNR; ++u) {
                    if (ks0 + u * GW < ksteps) {
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            if (h < rt) {
#pragma unroll
                                for (int nt = 0; nt < NT; ++nt)
                                    mma16816_bf16_acc(acc[h][nt], a[u][h][0], a[u][h][1], a[u][h][2], a[u][h][3],
                                                      b[u][nt][0], b[u][nt][1]);
                            }
                        }
                    }
                }
            }
            // Release the stage.  The warp of the group that is last to do so refills it at once: no warp waits
            // for another here.  (The fence orders this warp's reads of the stage before the counter update.)
            __syncwarp();
            if (lane == 0) {
                __threadfence_block();
                const int done = atomicAdd(&released[s], 1);   // counts up over all uses of the stage
                if ((done & (GW - 1)) == GW - 1 && item + nstages < total_items) issue(item + nstages);
            }
        }
        // row group finished: reduce the 16 warps' partial sums through shared memory, upper half first
        const int grp_row0 = row_begin + grp * group_rows;
        float *mine = red + (size_t)(warp & 7) * 32 * RC;
        if (red_in_ring) __syncthreads();   // every warp is done with the ring before it is reused
        if (warp >= 8) {
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    float *p = mine + (h * 16 + g) * RC + nt * 8 + 2 * t;
                    p[0] = acc[h][nt][0];
                    p[1] = acc[h][nt][1];
                    p[8 * RC] = acc[h][nt][2];
                    p[8 * RC + 1] = acc[h][nt][3];
                }
        }
        __syncthreads();
        if (warp < 8) {
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    float *p = mine + (h * 16 + g) * RC + nt * 8 + 2 * t;
                    p[0] += acc[h][nt][0];
                    p[1] += acc[h][nt][1];
                    p[8 * RC] += acc[h][nt][2];
                    p[8 * RC + 1] += acc[h][nt][3];
                }
        }
        __syncthreads();
        for (int idx = tid; idx < rt * 16 * Bg; idx += GV_THREADS) {
            const int r = idx / Bg, c = idx - r * Bg;   // r: row within the group
            float sum = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) sum += red[((size_t)w * 32 + r) * RC + c];
            const int row = grp_row0 + r;
            if (r < group_rows && row < row_end) {
                store_out(Y, (size_t)row * B + b0 + c, sum, out_dtype);
                // the same value, with the call's tag beside it, into the slot arrays of the other ranks: one 8-byte
                // store each, which arrives whole, so a peer that reads the tag has the value
                const size_t slot = (size_t)(po.row_begin + row) * B + c;
#pragma unroll
                for (int p = 0; p < 7; ++p)
                    if (p < po.n)
                        asm volatile("st.relaxed.sys.global.v2.b32 [%0], {%1, %2};\n" ::"l"(po.slots[p] + slot),
                                     "r"(__float_as_uint(sum)), "r"(tag)
                                     : "memory");
            }
        }
        __syncthreads();
    }
    if (po.n) {
        // Collect: the other ranks' rows arrive in this GPU's slot array (value, tag); every CTA takes an equal share
        // of them, waits for each tag -- at most a second in all, then B200HT_ERR_TIMEOUT in the status word --
        // and writes the value into the full result.  No fence and no counter is on this path: a value costs one
        // trip over the link.  Kernel complete => Y complete.
        const long own0 = (long)po.row_begin * B, own_n = (long)M * B;
        const long foreign = (long)po.rows_total * B - own_n;
        const long per = (foreign + gridDim.x - 1) / gridDim.x;
        const long i0 = (long)blockIdx.x * per;
        const long i1 = i0 + per < foreign ? i0 + per : foreign;
        const uint64_t t0 = global_ns();
        for (long i = i0 + tid; i < i1; i += GV_THREADS) {
            const long g = i < own0 ? i : i + own_n;      // position in the full result
            uint32_t val = 0, seen = 0;
            uint32_t spins = 0;
            while (true) {
                asm volatile("ld.volatile.global.v2.b32 {%0, %1}, [%2];\n" : "=r"(val), "=r"(seen) : "l"(po.my_slots + g) : "memory");
                if (seen == tag) break;
                if ((++spins & 63u) == 0) {
                    if (*abort_flag) break;
                    if (global_ns() - t0 > 1000000000ull) {
                        *abort_flag = 1;
                        if (status) atomicExch(status, B200HT_ERR_TIMEOUT);
                        break;
                    }
                }
            }
            if (seen == tag) store_out(po.y_full, (size_t)g, __uint_as_float(val), out_dtype);
        }
        // count the CTA and, in the last one, the call (one 64-bit word: finished CTAs low, calls high)
        __syncthreads();
        if (tid == 0) {
            const unsigned long long old = atomicAdd((unsigned long long *)po.local_count, 1ull);
            if ((unsigned int)old + 1u == gridDim.x)
                asm volatile("red.relaxed.gpu.global.add.u64 [%0], %1;\n" ::"l"(po.local_count),
                             "l"((1ull << 32) - (unsigned long long)gridDim.x)
                             : "memory");
        }
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
    if ((N & 255) == 0) {
        // one warp per row, 16-byte loads of W (two in flight per lane), up to 8 columns of H(X) per pass over the row
        const float4 *hx4 = (const float4 *)hx;
        const int nv = N >> 2;
        for (int row = blockIdx.x * 8 + warp; row < M; row += gridDim.x * 8) {
            const float4 *w4 = (const float4 *)(W + (size_t)row * N);
            for (int c0 = 0; c0 < Bg; c0 += 8) {
                float acc[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] = 0.f;
                for (int k = lane; k < nv; k += 64) {
                    const float4 wa = __ldg(w4 + k), wb = __ldg(w4 + k + 32);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        if (c0 + j < Bg) {
                            const float4 ha = hx4[(size_t)(c0 + j) * nv + k], hb = hx4[(size_t)(c0 + j) * nv + k + 32];
                            acc[j] = fmaf(wa.x, ha.x, fmaf(wa.y, ha.y, fmaf(wa.z, ha.z, fmaf(wa.w, ha.w, acc[j]))));
                            acc[j] = fmaf(wb.x, hb.x, fmaf(wb.y, hb.y, fmaf(wb.z, hb.z, fmaf(wb.w, hb.w, acc[j]))));
                        }
                    }
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    float s = acc[j];
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                    if (lane == 0 && c0 + j < Bg) store_out(Y, (size_t)row * B + b0 + c0 + j, s, out_dtype);
                }
            }
        }
        return;
    }
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

template <int NT>
static int launch_bf16_nt(const void *W, const void *X, void *Y, int M, int N, int logn, int B, int b0,
                          int Bg, int gc, int out_dtype, float scale, size_t smem, cudaStream_t st)
{
    const int rc = ensure_dyn_smem((const void *)gemv_bf16_kernel<NT>, (int)smem);
    if (rc) return rc;
    const int tiles = (M + 15) / 16;
    const int grid = tiles < sm_count() ? tiles : sm_count();
    note_launch();
    gemv_bf16_kernel<NT><<<grid, 256, smem, st>>>((const __nv_bfloat16 *)W, (const __nv_bfloat16 *)X, Y, M,
                                                  N, logn, B, b0, Bg, gc, out_dtype, scale);
    return (int)cudaGetLastError();
}

constexpr size_t kStreamSmemLimit = 225 * 1024;
static size_t stream_fixed_smem(int N, int cols, bool red_in_ring = false)
{
    const int nt = (cols + 7) / 8;
    return (((size_t)cols * hxt_pitch(N) + 127) & ~(size_t)127) +
           (red_in_ring ? 0 : (size_t)(GV_WARPS / 2) * 32 * nt * 8 * 4) + 1024 /*alignment*/ + 16 * 16 +
           64 /*barriers, counters*/;
}
// Columns per launch on the fast path (all of B, or a multiple of 8), 0 if the shape does not take it
// (the ring needs room for at least 64 KB).
static int stream_cols_max(int N, int B)
{
    if (N < 256 || N > 8192) return 0;
    int cols = B < 32 ? B : 32;
    while (cols > 8 && stream_fixed_smem(N, cols) + 64 * 1024 > kStreamSmemLimit) cols = (cols - 1) & ~7;
    return stream_fixed_smem(N, cols) + 64 * 1024 <= kStreamSmemLimit ? cols : 0;
}

template <int NT>
static int launch_stream_nt(const void *W, const void *X, void *Y, int M, int N, int logn, int B, int b0, int Bg,
                            int out_dtype, float scale, cudaStream_t st, const PeerOut &po)
{
    // one CTA per SM, but never fewer than 8 rows per CTA
    int grid = sm_count();
    if (grid > (M + 7) / 8) grid = (M + 7) / 8;
    const int rows_per_cta = (M + grid - 1) / grid;
    grid = (M + rows_per_cta - 1) / rows_per_cta;
    const int groups = (rows_per_cta + GV_MAX_GROUP_ROWS - 1) / GV_MAX_GROUP_ROWS;
    const int group_rows = (rows_per_cta + groups - 1) / groups;
    // One TMA op = group_rows x (64*kc) elements, at most 32 KB, kc a power of two dividing N/64.  The number of
    // stages is a multiple of the number of warp groups (see the kernel).
    //   * A CTA with one row group (a short call): four groups of four warps; among the candidates take the one
    //     that keeps most bytes in flight, preferring at least one item per warp group and then the larger op.
    //   * A CTA with several row groups (a long stream): what counts is that a warp gets one unrolled batch of four
    //     k steps per item, i.e. kc = warps per group, and 1 KB of every row per op rather than 512 bytes: two
    //     groups of eight warps with kc = 8 if that fits, else four of four with kc = 4.  (28672 x 8192, B = 4:
    //     6.4 TB/s so; 5.9 with kc = 4 under two groups, 4.6-5.6 with kc = 2.)
    int wgroups = 4, only_kc = 0;
    int kc = 0, stages = 0, stage_bytes = 0;
    auto plan = [&](bool red_in_ring) {
        const size_t ring_room = kStreamSmemLimit - stream_fixed_smem(N, Bg, red_in_ring);
        size_t best = 0;
        kc = 0;
        // (kc = 4 first: with four warps per group it is the one-batch-per-warp cut, so it wins ties)
        const int order[5] = {4, 16, 8, 2, 1};
        for (int oi = 0; oi < 5; ++oi) {
            const int cand = order[oi];
            if (only_kc && cand != only_kc) continue;
            if ((N / 64) % cand || (size_t)group_rows * 128 * cand > 32 * 1024) continue;
            const int sb = ((group_rows * 128 * cand) + 1023) & ~1023;
            int st = (int)(ring_room / sb);
            st = (st > 16 ? 16 : st) & ~(wgroups - 1);
            if (st < wgroups) continue;
            const size_t score = (size_t)st * sb + ((N / 64) / cand >= wgroups ? (size_t)1 << 30 : 0);
            if (score > best) { best = score; kc = cand; stages = st; stage_bytes = sb; }
        }
    };
    // the reduction buffer reuses the start of the ring when it runs once, at the end, and fits there
    bool red_in_ring = groups == 1;
    if (groups > 1) {
        wgroups = 2, only_kc = 8;
        plan(false);
        if (!kc) {
            wgroups = 4, only_kc = 4;
            plan(false);
        }
        if (!kc) only_kc = 0;      // neither fits: any plan will do
    }
    if (!kc) {
        plan(red_in_ring);
        if (red_in_ring && (!kc || (size_t)stages * stage_bytes < (size_t)(GV_WARPS / 2) * 32 * NT * 8 * 4)) {
            red_in_ring = false;
            plan(false);
        }
    }
    if (!kc) return B200HT_ERR_SIZE;
    const size_t smem = stream_fixed_smem(N, Bg, red_in_ring) + (size_t)stages * stage_bytes;
    CUtensorMap tw;
    int rc = encode_tmap_bf16_rows_chunks(&tw, W, (uint64_t)M, (uint64_t)N, (uint32_t)group_rows, (uint32_t)kc);
    if (rc) return rc;
    auto kernel = wgroups == 4 ? gemv_bf16_stream_kernel<NT, GV_WARPS / 4> : gemv_bf16_stream_kernel<NT, GV_WARPS / 2>;
    rc = ensure_dyn_smem((const void *)kernel, (int)smem);
    if (rc) return rc;
    return launch_pdl(kernel, dim3(grid), dim3(GV_THREADS), smem, st, tw, (const __nv_bfloat16 *)X, Y, M, N, logn, B, b0,
                      Bg, out_dtype, scale, rows_per_cta, group_rows, kc, stage_bytes, stages, red_in_ring ? 1 : 0,
                      status_word_ptr(), po);
}

static int launch_stream(const void *W, const void *X, void *Y, int M, int N, int logn, int B, int b0, int Bg,
                         int out_dtype, float scale, cudaStream_t st, const PeerOut &po = PeerOut{})
{
    switch ((Bg + 7) / 8) {
    case 1: return launch_stream_nt<1>(W, X, Y, M, N, logn, B, b0, Bg, out_dtype, scale, st, po);
    case 2: return launch_stream_nt<2>(W, X, Y, M, N, logn, B, b0, Bg, out_dtype, scale, st, po);
    case 3: return launch_stream_nt<3>(W, X, Y, M, N, logn, B, b0, Bg, out_dtype, scale, st, po);
    case 4: return launch_stream_nt<4>(W, X, Y, M, N, logn, B, b0, Bg, out_dtype, scale, st, po);
    }
    return B200HT_ERR_SIZE;
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
        if (bg_max > 8) bg_max = 8;   // the row loop keeps at most 8 columns per pass over a row of W
        // balanced column groups (W is streamed once per group); one wave of CTAs, as many per SM as the slab allows
        const int ngroups = (B + bg_max - 1) / bg_max;
        bg_max = (B + ngroups - 1) / ngroups;
        for (int b0 = 0; b0 < B; b0 += bg_max) {
            const int Bg = (B - b0) < bg_max ? (B - b0) : bg_max;
            const size_t smem = (size_t)Bg * N * 4;
            const int rc = ensure_dyn_smem((const void *)gemv_f32_kernel, (int)smem);
            if (rc) return rc;
            int grid = (M + 7) / 8;
            int per_sm = (int)((220 * 1024) / (smem + 1024));
            per_sm = per_sm < 1 ? 1 : (per_sm > 8 ? 8 : per_sm);
            const int cap = sm_count() * per_sm;
            grid = grid < cap ? grid : cap;
            note_launch();
            gemv_f32_kernel<<<grid, 256, smem, st>>>((const float *)W, (const float *)X, Y, M, N, logn, B, b0,
                                                     Bg, out_dtype, scale);
            const cudaError_t e = cudaGetLastError();
            if (e != cudaSuccess) return (int)e;
        }
        return 0;
    }
    // bf16, 256 <= N <= 8192.  Two kernels cover these shapes: the mma.sync streaming kernel below (the default: it is
    // the faster one on a B200, 8.5-9 us against 9.5-9.8 us at W 4096 x 4096, B <= 4) and the tcgen05 kernel of
    // fused_gemv_tc.cu, selected with B200HT_GEMV_TCGEN05=1 (read once per process).
    static const bool use_tcgen05 = [] {
        const char *e = std::getenv("B200HT_GEMV_TCGEN05");
        return e && e[0] == '1';
    }();
    if (use_tcgen05) {
        if (const int cols_max = gemv_tc_cols_max(N, B)) {
            for (int b0 = 0; b0 < B; b0 += cols_max) {
                const int Bg = (B - b0) < cols_max ? (B - b0) : cols_max;
                const int rc = launch_gemv_tc(W, X, Y, M, N, logn, B, b0, Bg, out_dtype, scale, st);
                if (rc) return rc;
            }
            return 0;
        }
    }
    // bf16, mma.sync streaming kernel: up to 32 columns per launch
    if (const int cols_max = stream_cols_max(N, B)) {
        for (int b0 = 0; b0 < B; b0 += cols_max) {
            const int Bg = (B - b0) < cols_max ? (B - b0) : cols_max;
            const int rc = launch_stream(W, X, Y, M, N, logn, B, b0, Bg, out_dtype, scale, st);
            if (rc) return rc;
        }
        return 0;
    }
    // bf16 generic path: largest column group whose H(X) fits in shared memory
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
    if (M < 0 || B < 1 || B > 65536) return B200HT_ERR_SIZE;
    if (in_dtype == B200HT_BF16 && N < 32) return B200HT_ERR_SIZE;
    if (M == 0) return 0;
    if (!W || !X || !Y) return B200HT_ERR_NULL;
    if (!aligned16(W) || !aligned16(X) || !aligned16(Y)) return B200HT_ERR_ALIGN;
    int rc = check_device();
    if (rc) return rc;
    return launch_gemv(W, X, Y, M, N, B, in_dtype, out_dtype, scale, (cudaStream_t)stream);
}

extern "C" int b200ht_fused_gemv_peers(const void *W, const void *X, void *Y_full, int M, int N, int B, int in_dtype,
                                       int out_dtype, float scale, int row_begin, int rows_total, int n_peers,
                                       void *const *peer_slots, const void *my_slots, unsigned int *local_count,
                                       unsigned int target, void *stream)
{
    using namespace b200ht;
    if (in_dtype != B200HT_BF16) return B200HT_ERR_DTYPE;
    if (out_dtype != B200HT_F32 && out_dtype != B200HT_BF16) return B200HT_ERR_DTYPE;
    if (N < 256 || N > 8192 || !is_pow2((uint64_t)N)) return B200HT_ERR_SIZE;
    if (M < 1 || B < 1 || B > stream_cols_max(N, B)) return B200HT_ERR_SIZE;
    if (n_peers < 0 || n_peers > 7 || row_begin < 0 || rows_total < M || row_begin > rows_total - M) return B200HT_ERR_SIZE;
    if ((uint64_t)rows_total * (uint64_t)B >= (1ull << 31)) return B200HT_ERR_SIZE;
    if (!W || !X || !Y_full || !local_count || (n_peers && (!peer_slots || !my_slots))) return B200HT_ERR_NULL;
    const size_t esz = out_dtype == B200HT_F32 ? 4 : 2;
    if (!aligned16(W) || !aligned16(X) || ((uintptr_t)Y_full & (esz - 1)) || ((uintptr_t)local_count & 7u) ||
        ((uintptr_t)my_slots & 7u))
        return B200HT_ERR_ALIGN;
    int rc = check_device();
    if (rc) return rc;
    PeerOut po{};
    po.n = n_peers;
    for (int p = 0; p < n_peers; ++p) {
        if (!peer_slots[p]) return B200HT_ERR_NULL;
        if ((uintptr_t)peer_slots[p] & 7u) return B200HT_ERR_ALIGN;
        po.slots[p] = (unsigned long long *)peer_slots[p];
    }
    po.my_slots = (const unsigned long long *)my_slots;
    po.y_full = Y_full;
    po.local_count = local_count;
    po.target = target;
    po.row_begin = row_begin;
    po.rows_total = rows_total;
    // this rank's rows go straight into their place in the full result
    void *Y = (unsigned char *)Y_full + (size_t)row_begin * B * esz;
    return launch_stream(W, X, Y, M, N, ilog2((uint32_t)N), B, 0, B, out_dtype, scale, (cudaStream_t)stream, po);
}

// Inter-process mapping of device buffers (one process per GPU): export a handle for a buffer inside a cudaMalloc
// allocation, open a peer's handle.  Thin wrappers over the CUDA IPC calls so that host code needs no CUDA binding.
extern "C" int b200ht_ipc_export(const void *ptr, void *handle64, unsigned long long *offset)
{
    if (!ptr || !handle64 || !offset) return B200HT_ERR_NULL;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    CUdeviceptr base = 0;
    size_t size = 0;
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    typedef CUresult (*RangeFn)(CUdeviceptr *, size_t *, CUdeviceptr);
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess || !fn)
        return (int)cudaErrorNotSupported;
    if (((RangeFn)fn)(&base, &size, (CUdeviceptr)ptr) != CUDA_SUCCESS) return (int)cudaErrorInvalidValue;
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, (void *)base);
    if (e != cudaSuccess) return (int)e;
    memcpy(handle64, &h, 64);
    *offset = (unsigned long long)((CUdeviceptr)ptr - base);
    return 0;
}

extern "C" int b200ht_ipc_open(const void *handle64, void **base)
{
    if (!handle64 || !base) return B200HT_ERR_NULL;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    return (int)cudaIpcOpenMemHandle(base, h, cudaIpcMemLazyEnablePeerAccess);
}

extern "C" int b200ht_ipc_close(void *base)
{
    if (!base) return B200HT_ERR_NULL;
    return (int)cudaIpcCloseMemHandle(base);
}

extern "C" int b200ht_fused_gemv_max_batch(int N, int in_dtype)
{
    using namespace b200ht;
    if (N < 2 || N > (1 << kMaxLogN) || !is_pow2((uint64_t)N)) return 0;
    if (in_dtype != B200HT_BF16) return 0;
    return stream_cols_max(N, 65536);
}
