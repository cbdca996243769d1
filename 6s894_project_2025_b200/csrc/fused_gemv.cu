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
#include "tc_common.cuh"
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
// bf16, 256 <= N <= 8192: the fast path.  16 warps per CTA, one CTA per SM,
// every CTA owns a contiguous, balanced range of rows of W.
//
//  * From the first cycle the CTA streams its rows of W into a shared-memory
//    ring with TMA tile loads (cp.async.bulk.tensor.3d over a [64 k][rows][N/64]
//    view of W: one op brings all rows of a row group x 512..1024 k, 16-32 KB,
//    as consecutive 128-byte-swizzled K-major tiles; completion is counted on an
//    mbarrier per stage).  The copies hold no registers and no LSU slots, so HBM
//    traffic runs underneath the transform of X and only pauses when the ring
//    is full.  (Small ops starve the TMA engine: 1 KB per-row bulk copies and
//    28-row x 128-byte boxes both stayed below 20 GB/s per SM.)
//  * Meanwhile the warps copy X (N x B, b fastest) into shared memory and
//    transform it there.  H(X) is kept per block of 8 columns as N vectors of
//    16 bytes (vector k = columns 8cb..8cb+7 of row k): the columns are passenger
//    bits, so X needs no transpose.  Each pass sends five index bits through
//    rot8 on the lanes (identity on the three in-vector bits) and up to two more
//    through fp32 register butterflies.
//  * Then the warps consume the ring: ldmatrix of a 16-row x 16-k block of W (A
//    operand), ldmatrix.trans of the matching 16 vectors of H(X) (B operand),
//    mma.sync m16n8k16 with fp32 accumulators.  A warp owns one 16-row tile of
//    the row group and every (16/tiles)-th k step, keeps its partial sums in
//    registers over the whole K range, and the warps reduce through shared
//    memory once per row group.  A stage is refilled one iteration after it was
//    consumed, when all warps have released it.
// Vector k of H(X) lives at position k ^ f(k) (low three bits only) so that
// the contiguous accesses of the first pass, the 512-byte-strided accesses of
// later passes and the eight row addresses of each ldmatrix are conflict free.
// ---------------------------------------------------------------------------
__device__ __forceinline__ int hx_pos(int k) { return k ^ (((k >> 3) & 3) << 1) ^ ((k >> 5) & 7); }

constexpr int GV_WARPS = 16;
constexpr int GV_THREADS = GV_WARPS * 32;
constexpr int GV_MAX_GROUP_ROWS = 32;                // rows of W per ring stage (one or two 16-row tiles)

// One in-place pass over index bits [lo, lo+nb) (lanes, through rot8) and
// [lo+nb, lo+nb+JB) (registers) of every 8-column block.  With nb < 5 the spare
// lane bits carry the lowest index bits as passengers.  TPI tasks are kept in
// flight per warp so that the mma latencies overlap.
template <int JB, int TPI>
__device__ __forceinline__ void hx_pass(uint4 *hx, int nplanes, int logn, int lo, int nb, float mult, int warp,
                                        int lane)
{
    constexpr int J = 1 << JB;
    constexpr int CNT = TPI * J;
    const int idb = 5 - nb;
    const int k_lane = ((lane & ((1 << nb) - 1)) << lo) | (lane >> nb);
    const int tl_bits = lo - idb;
    const int hi = lo + nb + JB;
    const int pp_shift = logn - 5 - JB;
    const int ntasks = nplanes << pp_shift;
    uint32_t A1[4], A2[4];
    const unsigned m1 = (nb > 0 ? 2u : 0u) | (nb > 1 ? 4u : 0u);
    const unsigned m2 = (nb > 2 ? 1u : 0u) | (nb > 3 ? 2u : 0u) | (nb > 4 ? 4u : 0u);
    make_hfrag<B200HT_BF16>(A1, lane, m1, hfrag_c(popc4(m1)));
    make_hfrag<B200HT_BF16>(A2, lane, m2, hfrag_c(popc4(m2)));
    for (int task0 = warp; task0 < ntasks; task0 += GV_WARPS * TPI) {
        uint4 *ptr[CNT];
        uint4 v[CNT];
        float o[CNT][8];
#pragma unroll
        for (int q = 0; q < TPI; ++q) {
            const int task = task0 + q * GV_WARPS;
            const int tk = task < ntasks ? task : task0;
            const int plane = tk >> pp_shift, tt = tk & ((1 << pp_shift) - 1);
            const int k0 = ((tt & ((1 << tl_bits) - 1)) << idb) | ((tt >> tl_bits) << hi) | k_lane;
            uint4 *base = hx + ((size_t)plane << logn);
#pragma unroll
            for (int j = 0; j < J; ++j) ptr[q * J + j] = base + hx_pos(k0 | (j << (lo + nb)));
        }
#pragma unroll
        for (int i = 0; i < CNT; ++i) v[i] = *ptr[i];
        rot8x<B200HT_BF16, CNT>(v, o, A1, A2);
#pragma unroll
        for (int q = 0; q < TPI; ++q) {
#pragma unroll
            for (int s = 1; s < J; s <<= 1) {
#pragma unroll
                for (int j = 0; j < J; ++j) {
                    if (!(j & s)) {
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const float x = o[q * J + j][e], y = o[q * J + (j | s)][e];
                            o[q * J + j][e] = x + y;
                            o[q * J + (j | s)][e] = x - y;
                        }
                    }
                }
            }
            if (task0 + q * GV_WARPS < ntasks) {
#pragma unroll
                for (int j = 0; j < J; ++j) {
                    const float *oo = o[q * J + j];
                    uint4 r;
                    r.x = pack2<B200HT_BF16>(oo[0] * mult, oo[1] * mult);
                    r.y = pack2<B200HT_BF16>(oo[2] * mult, oo[3] * mult);
                    r.z = pack2<B200HT_BF16>(oo[4] * mult, oo[5] * mult);
                    r.w = pack2<B200HT_BF16>(oo[6] * mult, oo[7] * mult);
                    *ptr[q * J + j] = r;
                }
            }
        }
    }
    __syncthreads();
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t saddr)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(saddr));
}
__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t (&r)[2], uint32_t saddr)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n"
                 : "=r"(r[0]), "=r"(r[1])
                 : "r"(saddr));
}
#ifdef B200HT_GEMV_TRACE
__device__ unsigned long long g_gemv_trace[16];
#define GV_TRACE(i) do { if (blockIdx.x == 50 && tid == 0) g_gemv_trace[i] = global_ns(); } while (0)
#else
#define GV_TRACE(i) do { } while (0)
#endif

template <int NT>
__global__ void __launch_bounds__(GV_THREADS, 1)
gemv_bf16_stream_kernel(const __grid_constant__ CUtensorMap tmW, const __nv_bfloat16 *X, void *Y, int M, int N,
                        int logn, int B, int b0, int Bg, int out_dtype, float scale, int rows_per_cta,
                        int group_rows, int kc, int stage_bytes, int nstages, int *status)
{
    extern __shared__ unsigned char smem_dyn[];
    // ring first (1024-byte aligned stages for the 128-byte swizzle), then H(X), reduction buffer, barriers
    const uint32_t ring_s = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    unsigned char *gen = smem_dyn + (ring_s - smem_u32(smem_dyn));
    uint4 *hx = (uint4 *)(gen + (size_t)nstages * stage_bytes);                 // [NT][N] vectors
    float *red = (float *)((unsigned char *)hx + (size_t)NT * N * 16);           // [16 warps][16][NT*8]
    unsigned char *bar_mem = (unsigned char *)(red + GV_WARPS * 16 * NT * 8);    // full[], empty[], abort flag
    const uint32_t bar_s = smem_u32(bar_mem);
    volatile int *abort_flag = (volatile int *)(bar_mem + 16 * nstages);
    auto full_bar = [&](int s) { return bar_s + 8u * s; };
    auto empty_bar = [&](int s) { return bar_s + 8u * (nstages + s); };

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    GV_TRACE(0);

    // rows of W owned by this CTA, in groups of group_rows; one ring item = (group, 256-k chunk)
    const int row_begin = blockIdx.x * rows_per_cta;
    const int row_end = (row_begin + rows_per_cta) < M ? (row_begin + rows_per_cta) : M;
    const int my_rows = row_end > row_begin ? row_end - row_begin : 0;
    const int ngroups = (my_rows + group_rows - 1) / group_rows;
    const int nchunks = (N / 64) / kc;     // ring items per row group: kc 64-k chunks each
    const int total_items = ngroups * nchunks;

    if (tid == 0) {
        for (int s = 0; s < nstages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), GV_WARPS);
        }
        *abort_flag = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tmW);
    }
    __syncthreads();
    // programmatic dependent launch: barrier set-up above overlaps the predecessor's tail
    pdl_launch_dependents();
    pdl_wait();

    // one TMA op per ring item: group_rows x (64*kc) elements of W
    auto issue = [&](int item) {
        if (tid == 0) {
            const int s = item % nstages;
            const int grp = item / nchunks, chunk = item - grp * nchunks;
            mbar_expect_tx(full_bar(s), (uint32_t)(group_rows * kc * 128));
            tma_load_3d(ring_s + (uint32_t)(s * stage_bytes), &tmW, 0, row_begin + grp * group_rows, chunk * kc,
                        full_bar(s));
        }
    };
    const int prologue = total_items < nstages ? total_items : nstages;
    for (int item = 0; item < prologue; ++item) issue(item);
    GV_TRACE(1);

    // ------------------------------ H(X) into shared memory ------------------------------
    if ((B & 7) == 0 && (b0 & 7) == 0 && (Bg & 7) == 0) {
        const uint4 *Xv = (const uint4 *)X;
        const int vpr = B >> 3, v0 = b0 >> 3;
#pragma unroll 4
        for (int idx = tid; idx < NT * N; idx += GV_THREADS) {
            const int k = idx / NT, cb = idx - k * NT;
            hx[((size_t)cb << logn) + hx_pos(k)] = __ldg(Xv + (size_t)k * vpr + v0 + cb);
        }
    } else if (NT == 1 && b0 == 0 && Bg == B && (B == 1 || B == 2 || B == 4)) {
        // 16 bytes of X hold 8/B consecutive rows k: one load, 8/B vectors (columns >= B are zero)
        const uint4 *Xv = (const uint4 *)X;
        const int kpv = 8 / B;
        for (int v = tid; v < N / kpv; v += GV_THREADS) {
            const uint4 x = __ldg(Xv + v);
            const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (j < kpv) {
                    uint4 r = make_uint4(0, 0, 0, 0);
                    if (B == 1) r.x = (w[j >> 1] >> ((j & 1) * 16)) & 0xffffu;
                    else if (B == 2) r.x = w[j];
                    else { r.x = w[2 * j]; r.y = w[2 * j + 1]; }
                    hx[hx_pos(v * kpv + j)] = r;
                }
            }
        }
    } else {
        const unsigned short *Xs = (const unsigned short *)X;
#pragma unroll 2
        for (int idx = tid; idx < NT * N; idx += GV_THREADS) {
            const int k = idx / NT, cb = idx - k * NT;
            uint32_t h[8];
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const int col = cb * 8 + c;
                h[c] = col < Bg ? (uint32_t)__ldg(Xs + (size_t)k * B + b0 + col) : 0u;
            }
            hx[((size_t)cb << logn) + hx_pos(k)] =
                make_uint4(h[0] | (h[1] << 16), h[2] | (h[3] << 16), h[4] | (h[5] << 16), h[6] | (h[7] << 16));
        }
    }
    __syncthreads();
    GV_TRACE(2);
    {
        int lo = 0, rem = logn;
        float applied = 1.f;  // power-of-two factors baked into the A fragments so far
        while (rem > 0) {
            int nb, jb;
            if (lo == 0 || rem > 7) { nb = 5; jb = 0; }
            else { nb = rem < 5 ? rem : 5; jb = rem - nb; }
            const unsigned m1 = (nb > 0 ? 2u : 0u) | (nb > 1 ? 4u : 0u);
            const unsigned m2 = (nb > 2 ? 1u : 0u) | (nb > 3 ? 2u : 0u) | (nb > 4 ? 4u : 0u);
            applied *= hfrag_c(popc4(m1)) * hfrag_c(popc4(m2));
            const float mult = (rem - nb - jb) == 0 ? scale / applied : 1.f;
            if (jb == 0) hx_pass<0, 4>(hx, NT, logn, lo, nb, mult, warp, lane);
            else if (jb == 1) hx_pass<1, 2>(hx, NT, logn, lo, nb, mult, warp, lane);
            else hx_pass<2, 1>(hx, NT, logn, lo, nb, mult, warp, lane);
            lo += nb + jb;
            rem -= nb + jb;
        }
    }
    GV_TRACE(3);

    // ------------------------------ consume the ring ------------------------------
    const int g = lane >> 2, t = lane & 3;
    const uint32_t hx_s = smem_u32(hx);
    // row tiles per group (1 or 2) and this warp's share: one tile, every kstride-th k step
    const int rt = group_rows > 16 ? 2 : 1;
    const int my_tile = warp & (rt - 1);
    const int kstride = GV_WARPS / rt, kphase = warp / rt;
    // ldmatrix (A): lane -> (row, 16-byte k chunk) of the 16 x 16 block, 128-byte swizzle of the TMA tile
    const int a_row = my_tile * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
    const int a_chunk = lane >> 4;
    constexpr int RC = NT * 8;
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
    const int ksteps = kc * 4;
    for (int item = 0; item < total_items; ++item) {
        const int s = item % nstages;
        const uint32_t ph = (uint32_t)(item / nstages) & 1u;
        if (!mbar_wait(full_bar(s), ph, abort_flag, status)) return;
        if (item == 0) GV_TRACE(4);
        if (item == nstages) GV_TRACE(5);
        const int grp = item / nchunks, chunk = item - grp * nchunks;
        const uint32_t stage = ring_s + (uint32_t)(s * stage_bytes);
        for (int ks = kphase; ks < ksteps; ks += kstride) {
            const int c = ks >> 2, ks4 = ks & 3;
            const int rowidx = c * group_rows + a_row;
            uint32_t a[4];
            ldmatrix_x4(a, stage + (uint32_t)(rowidx * 128) + (uint32_t)((((ks4 * 2 + a_chunk) ^ rowidx) & 7) << 4));
            const int k = (chunk * kc + c) * 64 + ks4 * 16 + (lane & 15);
            const uint32_t boff = (uint32_t)(hx_pos(k) * 16);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                uint32_t b[2];
                ldmatrix_x2_trans(b, hx_s + (uint32_t)((nt << logn) * 16) + boff);
                mma16816_bf16_acc(acc[nt], a[0], a[1], a[2], a[3], b[0], b[1]);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar(s));
        // refill the stage consumed one iteration ago: by now every warp has released it
        if (item >= 1 && item - 1 + nstages < total_items) {
            const int prev = item - 1;
            if (!mbar_wait(empty_bar(prev % nstages), (uint32_t)(prev / nstages) & 1u, abort_flag, status)) return;
            issue(prev + nstages);
        }
        if (chunk == nchunks - 1) {
            // row group finished: reduce the warps' partial sums through shared memory
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                float *p = red + ((size_t)warp * 16 + g) * RC + nt * 8 + 2 * t;
                p[0] = acc[nt][0];
                p[1] = acc[nt][1];
                p[8 * RC] = acc[nt][2];
                p[8 * RC + 1] = acc[nt][3];
                acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
            }
            __syncthreads();
            const int grp_row0 = row_begin + grp * group_rows;
            for (int idx = tid; idx < rt * 16 * Bg; idx += GV_THREADS) {
                const int r = idx / Bg, c = idx - r * Bg;   // r: row within the group
                const int tile = r >> 4, rin = r & 15;
                float sum = 0.f;
                for (int w = tile; w < GV_WARPS; w += rt) sum += red[((size_t)w * 16 + rin) * RC + c];
                const int row = grp_row0 + r;
                if (r < group_rows && row < row_end) store_out(Y, (size_t)row * B + b0 + c, sum, out_dtype);
            }
            __syncthreads();
        }
    }
    GV_TRACE(6);
}

#ifdef B200HT_GEMV_TRACE
extern "C" int b200ht_debug_gemv_trace(unsigned long long *out)
{
    return (int)cudaMemcpyFromSymbol(out, g_gemv_trace, sizeof(g_gemv_trace));
}
#endif

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

constexpr size_t kStreamSmemLimit = 225 * 1024;
static size_t stream_fixed_smem(int N, int nt)
{
    return (size_t)nt * N * 16 + (size_t)GV_WARPS * 16 * nt * 8 * 4 + 1024 /*alignment*/ + 16 * 16 + 64 /*barriers*/;
}
// Column blocks (of 8) per launch on the fast path, 0 if the shape does not take it
// (the ring needs room for at least two stages of up to 32 KB).
static int stream_nt_max(int N, int B)
{
    if (N < 256 || N > 8192) return 0;
    int nt = (B + 7) / 8;
    if (nt > 4) nt = 4;
    while (nt > 1 && stream_fixed_smem(N, nt) + 64 * 1024 > kStreamSmemLimit) --nt;
    return stream_fixed_smem(N, nt) + 64 * 1024 <= kStreamSmemLimit ? nt : 0;
}

template <int NT>
static int launch_stream_nt(const void *W, const void *X, void *Y, int M, int N, int logn, int B, int b0, int Bg,
                            int out_dtype, float scale, cudaStream_t st)
{
    // one CTA per SM, but never fewer than 8 rows per CTA
    int grid = sm_count();
    if (grid > (M + 7) / 8) grid = (M + 7) / 8;
    const int rows_per_cta = (M + grid - 1) / grid;
    grid = (M + rows_per_cta - 1) / rows_per_cta;
    const int groups = (rows_per_cta + GV_MAX_GROUP_ROWS - 1) / GV_MAX_GROUP_ROWS;
    const int group_rows = (rows_per_cta + groups - 1) / groups;
    // one TMA op = group_rows x (64*kc) elements, about 16-32 KB; kc is a power of two dividing N/64
    int kc = 1;
    while (kc * 2 <= N / 64 && group_rows * 128 * kc * 2 <= 32 * 1024 && kc < 16) kc *= 2;
    const int stage_bytes = ((group_rows * 128 * kc) + 1023) & ~1023;
    int stages = (int)((kStreamSmemLimit - stream_fixed_smem(N, NT)) / stage_bytes);
    if (stages > 16) stages = 16;
    if (stages < 2) return B200HT_ERR_SIZE;
    const size_t smem = stream_fixed_smem(N, NT) + (size_t)stages * stage_bytes;
    CUtensorMap tw;
    int rc = encode_tmap_bf16_rows_chunks(&tw, W, (uint64_t)M, (uint64_t)N, (uint32_t)group_rows, (uint32_t)kc);
    if (rc) return rc;
    cudaError_t e =
        cudaFuncSetAttribute(gemv_bf16_stream_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    return launch_pdl(gemv_bf16_stream_kernel<NT>, dim3(grid), dim3(GV_THREADS), smem, st, tw,
                      (const __nv_bfloat16 *)X, Y, M, N, logn, B, b0, Bg, out_dtype, scale, rows_per_cta, group_rows, kc,
                      stage_bytes, stages, status_word_ptr());
}

static int launch_stream(const void *W, const void *X, void *Y, int M, int N, int logn, int B, int b0, int Bg,
                         int out_dtype, float scale, cudaStream_t st)
{
    switch ((Bg + 7) / 8) {
    case 1: return launch_stream_nt<1>(W, X, Y, M, N, logn, B, b0, Bg, out_dtype, scale, st);
    case 2: return launch_stream_nt<2>(W, X, Y, M, N, logn, B, b0, Bg, out_dtype, scale, st);
    case 3: return launch_stream_nt<3>(W, X, Y, M, N, logn, B, b0, Bg, out_dtype, scale, st);
    case 4: return launch_stream_nt<4>(W, X, Y, M, N, logn, B, b0, Bg, out_dtype, scale, st);
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
    // bf16 fast path: up to 4 blocks of 8 columns per launch
    if (const int nt_max = stream_nt_max(N, B)) {
        for (int b0 = 0; b0 < B; b0 += nt_max * 8) {
            const int Bg = (B - b0) < nt_max * 8 ? (B - b0) : nt_max * 8;
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
    if (M < 0 || B < 1 || B > 64) return B200HT_ERR_SIZE;
    if (in_dtype == B200HT_BF16 && N < 32) return B200HT_ERR_SIZE;
    if (M == 0) return 0;
    if (!W || !X || !Y) return B200HT_ERR_NULL;
    if (!aligned16(W) || !aligned16(X) || !aligned16(Y)) return B200HT_ERR_ALIGN;
    int rc = check_device();
    if (rc) return rc;
    return launch_gemv(W, X, Y, M, N, B, in_dtype, out_dtype, scale, (cudaStream_t)stream);
}
