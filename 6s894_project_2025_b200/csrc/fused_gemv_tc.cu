// Small-batch fused Y = W . H(X) on the 5th-generation tensor cores (bf16,
// 256 <= N <= 8192, H(X) resident in shared memory).  Replaces
// fused_hadamard_gemv_kernel(_vec) (fused_ht/fwht_gemv_fusion.cu:98-244), where one
// block per column of X streams all of W; here the grid runs over ROWS of W, so W
// is read from HBM exactly once and H(X) never leaves the SM.
//
// One CTA per SM owns a contiguous range of rows of W, cut into groups of at most
// 32 rows.  Per CTA:
//   * W streams through a shared-memory ring by TMA.  The tensor map is a 4-D view
//     [64 k][rows of a group][group][N/64] of W whose box is 32 rows high: rows
//     beyond the group's are filled with zeros by the copy engine, so every 64-k
//     tile of the ring is four whole 1024-byte swizzle atoms and is directly a
//     K-major tensor-core operand.  The ring's first fill is requested by sixteen
//     lanes at once, right after every warp has issued its first loads of X.
//   * Meanwhile all sixteen warps copy X (N x B, b fastest) into shared memory in
//     operand layout -- per 64-k chunk NU rows (one per column of X, NU = B rounded
//     up to 8 / 16 / 32 / 64) of 128 bytes, 128-byte swizzle -- and transform the
//     columns there in place (rot8 on 256-element chunks, fp32 register
//     butterflies for the remaining index bits).  16-byte vectors of a column
//     stay 16-byte vectors under the swizzle, so the transform works on the
//     operand layout directly.
//   * Then one thread issues the MMAs.  What an instruction costs here is set by the rows it fetches from shared
//     memory, about 0.8 cycles per row of the A operand plus some 50 cycles, whatever its N (measured: 100 cycles
//     for M = 64, 150 for M = 128), so the operand with few rows goes on the A side and every instruction takes
//     as much of W as an instruction can: A = H(X), 128 operand rows = the NU-row tiles of 128 / NU consecutive
//     64-k chunks; B = the 32-row W tiles of CPN = min(8, 128 / NU) consecutive chunks, N = 32 * CPN <= 256.  The
//     accumulator then holds every (chunk j' of H(X), chunk j of W) pair; the CPN pairs with j' = j are the wanted
//     partial sums, the others are ignored.  32 instructions cover a row group at N = 4096.  tcgen05.commit hands
//     each ring stage back to the producer thread.  Four warps drain a finished accumulator with tcgen05.ld, add
//     the CPN diagonal blocks through shared memory and store the rows of Y; a second accumulator lets the next
//     row group start meanwhile.
// Every mbarrier wait is time-limited (B200HT_ERR_TIMEOUT in the status word).
#include "tc_common.cuh"

namespace b200ht {

constexpr int GT_WARPS = 16;
constexpr int GT_THREADS = GT_WARPS * 32;
constexpr int GT_TILE_ROWS = 32;         // rows of a ring tile (a row group has at most that many rows of W)
constexpr int GT_MAX_STAGES = 16;        // the first fill is issued by one lane per stage
constexpr int GT_RED_PITCH = 33;         // floats per accumulator row of the reduction buffer (odd: no bank conflicts)

// Byte offset of the 16-byte vector v (elements 8v .. 8v+7) of column `col` in the B operand: 64-k chunks of NU
// rows x 128 bytes, 16-byte pieces XOR-swizzled by the row's low three bits.
template <int NU>
__device__ __forceinline__ uint32_t hx_vec_off(int col, int v)
{
    return (uint32_t)((v >> 3) * (NU * 128) + col * 128 + (((v & 7) ^ (col & 7)) << 4));
}
template <int NU>
__device__ __forceinline__ uint32_t hx_off(int col, int k)
{
    return hx_vec_off<NU>(col, k >> 3) + (uint32_t)((k & 7) * 2);
}

// Pass A of the in-place transform: index bits 0..7 (rot8) and 8..8+RB-1 (registers) of every group of 2^RB
// consecutive 256-element chunks of a column; `mult` is applied to the result.
template <int NU, int RB>
__device__ __forceinline__ void gt_pass_a(unsigned char *hx, int cols, int logn, float mult, int warp, int lane)
{
    constexpr int GRP = 1 << RB;
    uint32_t A1[4], A2[4];
    constexpr unsigned M1 = rot8_mask1(8), M2 = rot8_mask2(8);
    make_hfrag<B200HT_BF16>(A1, lane, M1, hfrag_c(popc4(M1)));
    make_hfrag<B200HT_BF16>(A2, lane, M2, hfrag_c(popc4(M2)));
    const int gpr = 1 << (logn - 8 - RB);            // chunk groups per column
    const int ntasks = cols * gpr;
    for (int task = warp; task < ntasks; task += GT_WARPS) {
        const int col = task / gpr, gi = task - col * gpr;
        const int v0 = gi * (GRP * 32) + lane;
        uint4 v[GRP];
#pragma unroll
        for (int u = 0; u < GRP; ++u) v[u] = *(const uint4 *)(hx + hx_vec_off<NU>(col, v0 + u * 32));
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
            *(uint4 *)(hx + hx_vec_off<NU>(col, v0 + u * 32)) = r;
        }
    }
}

// Pass B: the top JB index bits, as fp32 butterflies over 2^JB vectors that sit 2^(logn-JB) elements apart.
template <int NU, int JB>
__device__ __forceinline__ void gt_pass_b(unsigned char *hx, int cols, int logn, float mult, int tid)
{
    constexpr int J = 1 << JB;
    const int vps = 1 << (logn - JB - 3);            // vectors per sub-block
    const int ntasks = cols * vps;
    for (int task = tid; task < ntasks; task += GT_THREADS) {
        const int col = task / vps, p = task - col * vps;
        float o[J][8];
#pragma unroll
        for (int j = 0; j < J; ++j) {
            const uint4 v = *(const uint4 *)(hx + hx_vec_off<NU>(col, p + j * vps));
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
            *(uint4 *)(hx + hx_vec_off<NU>(col, p + j * vps)) = r;
        }
    }
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, int x, int y, int z, int w,
                                            uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];\n" ::
            "r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(w), "r"(bar)
        : "memory");
}

// 8 consecutive fp32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t *r)
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}

// Chunks of W per instruction (the B side, N = 32 * CPN) and TMEM columns: two accumulators of N columns.
template <int NU>
struct GtAcc {
    static constexpr int CPN = 128 / NU < 8 ? 128 / NU : 8;
    static constexpr int NMMA = GT_TILE_ROWS * CPN;
    static constexpr uint32_t TMEM_COLS = 2 * NMMA;   // 512, 256 or 128
};

template <int NU>
__global__ void __launch_bounds__(GT_THREADS, 1)
gemv_bf16_tc_kernel(const __grid_constant__ CUtensorMap tmMain, const __grid_constant__ CUtensorMap tmTail,
                    const __nv_bfloat16 *X, void *Y, int M, int N, int logn, int B, int b0, int Bg, int out_dtype,
                    float scale, int groups_per_cta, int group_rows, int n_full_groups, int kc, int stage_bytes,
                    int nstages, int *status)
{
    extern __shared__ unsigned char smem_dyn[];
    // ring first (1024-byte aligned; stage sizes are multiples of 1024), then the B operand H(X), then barriers
    const uint32_t ring_s = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    unsigned char *gen = smem_dyn + (ring_s - smem_u32(smem_dyn));
    unsigned char *hx = gen + (size_t)nstages * stage_bytes;                      // [N/64][NU][128 bytes]
    const uint32_t hx_s = ring_s + (uint32_t)(nstages * stage_bytes);
    float *red = (float *)(hx + (size_t)N * NU * 2);                      // [128 accumulator rows][GT_RED_PITCH]
    unsigned char *bar_mem = (unsigned char *)(red + 128 * GT_RED_PITCH);
    const uint32_t bar_s = smem_u32(bar_mem);
    auto full_bar = [&](int s) { return bar_s + 8u * s; };                        // TMA landed
    auto empty_bar = [&](int s) { return bar_s + 8u * (GT_MAX_STAGES + s); };     // the MMAs reading the stage are done
    auto accf_bar = [&](int a) { return bar_s + 8u * (2 * GT_MAX_STAGES + a); };  // accumulator slot complete
    auto acce_bar = [&](int a) { return bar_s + 8u * (2 * GT_MAX_STAGES + 2 + a); };  // accumulator slot drained
    uint32_t *tmem_slot = (uint32_t *)(bar_mem + 8 * (2 * GT_MAX_STAGES + 4));
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);
    volatile int *epi_ok = (volatile int *)(tmem_slot + 2);
    constexpr uint32_t TMEM_COLS = GtAcc<NU>::TMEM_COLS;
    constexpr int NMMA = GtAcc<NU>::NMMA;                                  // accumulator stride in TMEM columns
    const int cpn = (N / 64) < GtAcc<NU>::CPN ? (N / 64) : GtAcc<NU>::CPN;   // chunks of W per instruction
    constexpr int r8 = GT_TILE_ROWS;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    // row groups of this CTA; one ring item = (group, 64*kc-wide k chunk)
    const int total_groups = (M + group_rows - 1) / group_rows;
    const int g_begin = blockIdx.x * groups_per_cta;
    const int ngroups = total_groups - g_begin < groups_per_cta ? (total_groups - g_begin > 0 ? total_groups - g_begin : 0)
                                                                : groups_per_cta;
    const int nchunks = (N / 64) / kc;      // ring items per row group
    const int total_items = ngroups * nchunks;

    if (tid == 0) {
        for (int s = 0; s < nstages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(accf_bar(a), 1);
            mbar_init(acce_bar(a), 4);   // one arrival per epilogue warp
        }
        *abort_flag = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tmMain);
        tma_prefetch_desc(&tmTail);
    }
    if (warp == 2) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // Programmatic dependent launch: the set-up above overlaps the predecessor's tail, and so does a prefetch of X
    // into L2 (a hint that returns no data).
    pdl_launch_dependents();
    {
        const size_t xbytes = (size_t)N * B * 2;
        for (size_t off = (size_t)tid * 128; off < xbytes; off += (size_t)GT_THREADS * 128)
            asm volatile("prefetch.global.L2 [%0];\n" ::"l"((const unsigned char *)X + off));
    }
    pdl_wait();

    // one TMA op per ring item: the rows of a group x (64*kc) elements of W, as kc tiles of r8 x 128 bytes
    auto issue = [&](int item) {
        const int s = item % nstages;
        const int g = item / nchunks, ci = item - g * nchunks;
        const int G = g_begin + g;
        const uint32_t dst = ring_s + (uint32_t)(s * stage_bytes);
        mbar_expect_tx(full_bar(s), (uint32_t)(r8 * 128 * kc));
        if (G < n_full_groups) tma_load_4d(dst, &tmMain, 0, 0, G, ci * kc, full_bar(s));
        else tma_load_3d(dst, &tmTail, 0, 0, ci * kc, full_bar(s));   // the rows behind the last full group
    };
    // The first fill of the ring is requested by up to 16 lanes at once -- but only after every warp has issued its
    // first batch of X loads: requests of one SM are served in order, and X must not queue behind the ring.
    auto start_stream = [&]() {
        __syncthreads();
        if (warp == 1 && lane < (total_items < nstages ? total_items : nstages)) issue(lane);
    };

    // ------------------------------ X^T into the operand layout ------------------------------
    // Every path issues all loads of a batch before the first store.
    if (B == 1) {
        const uint4 *Xv = (const uint4 *)X;
        for (int base = 0; base < N / 8; base += GT_THREADS * 2) {
            uint4 r[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int v = base + u * GT_THREADS + tid;
                if (v < N / 8) r[u] = __ldg(Xv + v);
            }
            if (base == 0) start_stream();
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int v = base + u * GT_THREADS + tid;
                if (v < N / 8) *(uint4 *)(hx + hx_vec_off<NU>(0, v)) = r[u];
            }
        }
    } else if (B == 2) {
        // 16 bytes = rows k..k+3 of both columns
        const uint4 *Xv = (const uint4 *)X;
        for (int base = 0; base < N / 4; base += GT_THREADS * 4) {
            uint4 r[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int v = base + u * GT_THREADS + tid;
                if (v < N / 4) r[u] = __ldg(Xv + v);
            }
            if (base == 0) start_stream();
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int v = base + u * GT_THREADS + tid;
                const uint4 x = r[u];
                if (v < N / 4) {
                    *(uint2 *)(hx + hx_off<NU>(0, 4 * v)) = make_uint2(__byte_perm(x.x, x.y, 0x5410), __byte_perm(x.z, x.w, 0x5410));
                    *(uint2 *)(hx + hx_off<NU>(1, 4 * v)) = make_uint2(__byte_perm(x.x, x.y, 0x7632), __byte_perm(x.z, x.w, 0x7632));
                }
            }
        }
    } else if (B == 4) {
        // 32 bytes = rows k..k+3 of the four columns
        const uint4 *Xv = (const uint4 *)X;
        for (int base = 0; base < N / 4; base += GT_THREADS * 4) {
            uint4 rx[4], ry[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int v = base + u * GT_THREADS + tid;
                if (v < N / 4) { rx[u] = __ldg(Xv + 2 * v); ry[u] = __ldg(Xv + 2 * v + 1); }
            }
            if (base == 0) start_stream();
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int v = base + u * GT_THREADS + tid;
                const uint4 x = rx[u], y = ry[u];   // x: rows k, k+1; y: rows k+2, k+3
                if (v < N / 4) {
                    *(uint2 *)(hx + hx_off<NU>(0, 4 * v)) = make_uint2(__byte_perm(x.x, x.z, 0x5410), __byte_perm(y.x, y.z, 0x5410));
                    *(uint2 *)(hx + hx_off<NU>(1, 4 * v)) = make_uint2(__byte_perm(x.x, x.z, 0x7632), __byte_perm(y.x, y.z, 0x7632));
                    *(uint2 *)(hx + hx_off<NU>(2, 4 * v)) = make_uint2(__byte_perm(x.y, x.w, 0x5410), __byte_perm(y.y, y.w, 0x5410));
                    *(uint2 *)(hx + hx_off<NU>(3, 4 * v)) = make_uint2(__byte_perm(x.y, x.w, 0x7632), __byte_perm(y.y, y.w, 0x7632));
                }
            }
        }
    } else if ((B & 7) == 0 && (b0 & 7) == 0 && (Bg & 7) == 0) {
        // two rows k, k+1 of one block of 8 columns per task: two 16-byte loads, eight 4-byte stores
        const uint4 *Xv = (const uint4 *)X;
        const int vpr = B >> 3, v0 = b0 >> 3, nb8 = Bg >> 3;
        const int ntasks = (N / 2) * nb8;
        for (int base = 0; base < ntasks; base += GT_THREADS * 8) {
            uint4 r0[8], r1[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int idx = base + u * GT_THREADS + tid;
                const int kp = idx / nb8, cb = idx - kp * nb8;
                if (idx < ntasks) {
                    r0[u] = __ldg(Xv + (size_t)(2 * kp) * vpr + v0 + cb);
                    r1[u] = __ldg(Xv + (size_t)(2 * kp + 1) * vpr + v0 + cb);
                }
            }
            if (base == 0) start_stream();
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int idx = base + u * GT_THREADS + tid;
                const int kp = idx / nb8, cb = idx - kp * nb8;
                if (idx < ntasks) {
                    const uint32_t w0[4] = {r0[u].x, r0[u].y, r0[u].z, r0[u].w};
                    const uint32_t w1[4] = {r1[u].x, r1[u].y, r1[u].z, r1[u].w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        *(uint32_t *)(hx + hx_off<NU>(cb * 8 + 2 * j, 2 * kp)) = __byte_perm(w0[j], w1[j], 0x5410);
                        *(uint32_t *)(hx + hx_off<NU>(cb * 8 + 2 * j + 1, 2 * kp)) = __byte_perm(w0[j], w1[j], 0x7632);
                    }
                }
            }
        }
    } else {
        const unsigned short *Xs = (const unsigned short *)X;
        const int ntasks = (N / 2) * Bg;
        for (int base = 0; base < ntasks; base += GT_THREADS * 8) {
            uint32_t lo[8], hi[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int idx = base + u * GT_THREADS + tid;
                const int kp = idx / Bg, c = idx - kp * Bg;
                if (idx < ntasks) {
                    lo[u] = __ldg(Xs + (size_t)(2 * kp) * B + b0 + c);
                    hi[u] = __ldg(Xs + (size_t)(2 * kp + 1) * B + b0 + c);
                }
            }
            if (base == 0) start_stream();
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int idx = base + u * GT_THREADS + tid;
                const int kp = idx / Bg, c = idx - kp * Bg;
                if (idx < ntasks) *(uint32_t *)(hx + hx_off<NU>(c, 2 * kp)) = lo[u] | (hi[u] << 16);
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
        if (ra == 0) gt_pass_a<NU, 0>(hx, Bg, logn, mult_a, warp, lane);
        else if (ra == 1) gt_pass_a<NU, 1>(hx, Bg, logn, mult_a, warp, lane);
        else gt_pass_a<NU, 2>(hx, Bg, logn, mult_a, warp, lane);
        if (jb) __syncthreads();
        if (jb == 1) gt_pass_b<NU, 1>(hx, Bg, logn, scale / fa, tid);
        else if (jb == 2) gt_pass_b<NU, 2>(hx, Bg, logn, scale / fa, tid);
        else if (jb == 3) gt_pass_b<NU, 3>(hx, Bg, logn, scale / fa, tid);
    }
    // H(X) was written with ordinary stores; the MMAs read it through the async proxy
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    if (warp == 0) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            // NU = 8: the eight chunk blocks that matter are 64 operand rows, and an M = 64 instruction costs its
            // issuer 52 ns against 84 ns for M = 128
            const uint32_t idesc = umma_idesc_bf16(NU == 8 ? 64 : 128, r8 * cpn);
            const int steps = kc / cpn;   // instruction groups (cpn chunks each) per ring item
            bool ok = true;
            for (int g = 0; g < ngroups && ok; ++g) {
                const int slot = g & 1;
                if (!mbar_wait(acce_bar(slot), ((uint32_t)(g >> 1) & 1u) ^ 1u, abort_flag, status)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(slot * NMMA);
                for (int ci = 0; ci < nchunks; ++ci) {
                    const int item = g * nchunks + ci;
                    const int s = item % nstages;
                    if (!mbar_wait(full_bar(s), (uint32_t)(item / nstages) & 1u, abort_flag, status)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t w_s = ring_s + (uint32_t)(s * stage_bytes);
                    const uint32_t h_s = hx_s + (uint32_t)(ci * kc * (NU * 128));
                    for (int c = 0; c < steps; ++c) {
                        // A: 128 operand rows of H(X) from chunk ci*kc + c*cpn on (the first cpn chunks matter; the
                        // window may run further, at the very end into the reduction buffer);
                        // B: the cpn W tiles of the same chunks
                        const uint64_t adesc = umma_desc_k_sw128(h_s + (uint32_t)(c * cpn * (NU * 128)));
                        const uint64_t bdesc = umma_desc_k_sw128(w_s + (uint32_t)(c * cpn * (r8 * 128)));
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks)
                            umma_bf16_ss(d_tmem, adesc + 2 * ks, bdesc + 2 * ks, idesc, (ci | c | ks) ? 1u : 0u);
                    }
                    umma_commit(empty_bar(s));
                }
                if (ok) umma_commit(accf_bar(slot));
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------ TMA producer (items behind the first fill) ------------------------------
        if (lane == 0) {
            int issued = total_items < nstages ? total_items : nstages;
            for (int item = nstages; item < total_items; ++item) {
                const int s = item % nstages;
                if (!mbar_wait(empty_bar(s), ((uint32_t)(item / nstages) & 1u) ^ 1u, abort_flag, status)) break;
                issue(item);
                issued = item + 1;
            }
            if (*abort_flag) {
                // copies already issued still land in this CTA's shared memory: give them time
                const int pending = issued < nstages ? issued : nstages;
                for (int j = 0; j < pending; ++j) {
                    const int i2 = issued - 1 - j;
                    const uint64_t t0 = global_ns();
                    while (!mbar_test(full_bar(i2 % nstages), (uint32_t)(i2 / nstages) & 1u) &&
                           global_ns() - t0 < 100000000ull) {}
                }
            }
        }
        __syncwarp();
    } else if (warp >= 4 && warp < 8) {
        // ------------------------------ epilogue ------------------------------
        // Accumulator lane L = 32 * q + lane holds column b = L % NU of H(X) for chunk block j' = L / NU; its wanted
        // values are the 32 accumulator columns of the same chunk block (the rows of the group), if j' < cpn.
        const int q = warp & 3;
        // (an M = 64 accumulator, NU = 8, keeps 16 operand rows per lane quadrant, in lanes 0..15)
        constexpr int RPQ = NU == 8 ? 16 : 32;        // accumulator rows per lane quadrant
        const bool has_row = lane < RPQ;
        const int L = q * RPQ + (has_row ? lane : 0);
        const int jmine = has_row ? L / NU : -1;
        constexpr int JPW = NU >= RPQ ? 1 : RPQ / NU;  // chunk blocks per warp
        const int et = tid - 4 * 32;                  // 0..127 within the epilogue warps
        // Warp 4 waits for the accumulator and publishes the outcome; the named barrier that follows is executed by
        // all four warps whatever the outcome, so they leave the loop together if the wait gave up.  The same
        // barrier separates the previous group's reads of `red` from this group's writes.
        for (int g = 0; g < ngroups; ++g) {
            const int slot = g & 1;
            if (warp == 4) {
                const bool got = mbar_wait(accf_bar(slot), (uint32_t)(g >> 1) & 1u, abort_flag, status);
                if (lane == 0) *epi_ok = got ? 1 : 0;
            }
            asm volatile("bar.sync 1, 128;\n" ::: "memory");
            if (!*epi_ok) break;
            tc_fence_after();
            uint32_t keep[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) keep[j] = 0u;
            const int jfirst = (q * RPQ) / NU;
#pragma unroll
            for (int sub = 0; sub < JPW; ++sub) {
                const int jb = jfirst + sub;          // warp-uniform
                if (jb < cpn) {
                    uint32_t r[32];
                    tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(slot * NMMA + jb * 32), r);
                    tmem_ld_wait();
                    if (jb == jmine) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) keep[j] = r[j];
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acce_bar(slot));
            // add the chunk blocks through shared memory and store
            // (rows of GT_RED_PITCH floats: the lanes of a warp write, and later read, different banks.  With rows of
            // 128 bytes the 16-byte stores of a warp all fell on the same four banks, and the loads queued behind
            // them: 0.5 us per row group at one column, 2.5 us at sixteen.)
            if (has_row) {
#pragma unroll
                for (int j = 0; j < 32; ++j) red[L * GT_RED_PITCH + j] = __uint_as_float(keep[j]);
            }
            asm volatile("bar.sync 1, 128;\n" ::: "memory");
            const long row0 = (long)(g_begin + g) * group_rows;
            for (int idx = et; idx < group_rows * Bg; idx += 128) {
                const int rg = idx / Bg, c = idx - rg * Bg;
                float sum = 0.f;
                for (int j = 0; j < cpn; ++j) sum += red[(j * NU + c) * GT_RED_PITCH + rg];
                const long row = row0 + rg;
                if (row < M) {
                    const size_t o = (size_t)row * B + b0 + c;
                    if (out_dtype == B200HT_F32) ((float *)Y)[o] = sum;
                    else ((__nv_bfloat16 *)Y)[o] = __float2bfloat16_rn(sum);
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 2) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------
// host
// ---------------------------------------------------------------------------
constexpr size_t kTcSmemLimit = 225 * 1024;
constexpr size_t kTcMinRing = 48 * 1024;
static size_t tc_fixed_smem(int N, int nu)
{
    return (size_t)N * nu * 2 + (size_t)128 * GT_RED_PITCH * 4 /*reduction*/ + 1024 /*alignment*/ + 8 * (2 * GT_MAX_STAGES + 4) + 64;
}
static int nu_of(int cols) { return cols <= 8 ? 8 : (cols <= 16 ? 16 : (cols <= 32 ? 32 : 64)); }

// Columns per launch of the tcgen05 kernel (all of B if H(X) fits beside a ring of at least 48 KB), 0 if the shape
// does not take it.
int gemv_tc_cols_max(int N, int B)
{
    if (N < 256 || N > 8192) return 0;
    int cols = B < 64 ? B : 64;
    while (cols > 8 && tc_fixed_smem(N, nu_of(cols)) + kTcMinRing > kTcSmemLimit) cols = nu_of(cols) / 2;
    return tc_fixed_smem(N, nu_of(cols)) + kTcMinRing <= kTcSmemLimit ? cols : 0;
}

template <int NU>
static int launch_gemv_tc_nu(const void *W, const void *X, void *Y, int M, int N, int logn, int B, int b0, int Bg,
                             int out_dtype, float scale, cudaStream_t st)
{
    // One CTA per SM, but never fewer than 8 rows per CTA.  The rows of a CTA go in equal groups of at most 32 rows
    // (the rest of a 32-row ring tile is zero-filled and costs shared memory only).
    int grid = sm_count();
    if (grid > (M + 7) / 8) grid = (M + 7) / 8;
    int rows_per_cta = (M + grid - 1) / grid;
    const int groups = (rows_per_cta + GT_TILE_ROWS - 1) / GT_TILE_ROWS;
    const int group_rows = (rows_per_cta + groups - 1) / groups;
    constexpr int r8 = GT_TILE_ROWS;
    const int ch = (N / 64) < GtAcc<NU>::CPN ? (N / 64) : GtAcc<NU>::CPN;   // chunks per instruction
    rows_per_cta = groups * group_rows;
    grid = (M + rows_per_cta - 1) / rows_per_cta;
    const int n_full = M / group_rows;          // groups with all their rows; >= 1 because group_rows <= M
    const int tail_rows = M - n_full * group_rows;
    // One TMA op = 32 x (64*kc) elements, at most 32 KB, kc a power of two dividing N/64 and a multiple of the
    // chunks per instruction; at most 16 stages.  Take the plan that keeps most bytes in flight, and among equals the finer one.
    const size_t ring_room = kTcSmemLimit - tc_fixed_smem(N, NU);
    int kc = 0, stages = 0, stage_bytes = 0;
    size_t best = 0;
    for (int cand = ch; cand <= 16; cand <<= 1) {
        if ((N / 64) % cand || (size_t)r8 * 128 * cand > 32 * 1024) continue;
        const int sb = r8 * 128 * cand;
        int nst = (int)(ring_room / sb);
        nst = nst > GT_MAX_STAGES ? GT_MAX_STAGES : nst;
        if (nst < 2) continue;
        const size_t score = (size_t)nst * sb;
        if (score > best) { best = score; kc = cand; stages = nst; stage_bytes = sb; }
    }
    if (!kc) return B200HT_ERR_SIZE;
    const size_t smem = tc_fixed_smem(N, NU) + (size_t)stages * stage_bytes;
    CUtensorMap tmain, ttail;
    int rc = encode_tmap_bf16_row_groups(&tmain, W, (uint64_t)group_rows, (uint64_t)n_full, (uint64_t)N, (uint32_t)r8,
                                         (uint32_t)kc);
    if (rc) return rc;
    ttail = tmain;
    if (tail_rows) {
        rc = encode_tmap_bf16_rows_chunks(&ttail, (const unsigned char *)W + (size_t)n_full * group_rows * N * 2,
                                          (uint64_t)tail_rows, (uint64_t)N, (uint32_t)r8, (uint32_t)kc);
        if (rc) return rc;
    }
    rc = ensure_dyn_smem((const void *)gemv_bf16_tc_kernel<NU>, (int)smem);
    if (rc) return rc;
    return launch_pdl(gemv_bf16_tc_kernel<NU>, dim3(grid), dim3(GT_THREADS), smem, st, tmain, ttail,
                      (const __nv_bfloat16 *)X, Y, M, N, logn, B, b0, Bg, out_dtype, scale, groups, group_rows, n_full, kc,
                      stage_bytes, stages, status_word_ptr());
}

int launch_gemv_tc(const void *W, const void *X, void *Y, int M, int N, int logn, int B, int b0, int Bg, int out_dtype,
                   float scale, cudaStream_t st)
{
    switch (nu_of(Bg)) {
    case 8: return launch_gemv_tc_nu<8>(W, X, Y, M, N, logn, B, b0, Bg, out_dtype, scale, st);
    case 16: return launch_gemv_tc_nu<16>(W, X, Y, M, N, logn, B, b0, Bg, out_dtype, scale, st);
    case 32: return launch_gemv_tc_nu<32>(W, X, Y, M, N, logn, B, b0, Bg, out_dtype, scale, st);
    default: return launch_gemv_tc_nu<64>(W, X, Y, M, N, logn, B, b0, Bg, out_dtype, scale, st);
    }
}

}  // namespace b200ht
