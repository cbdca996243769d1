// Standalone Walsh-Hadamard transform on the 5th-generation tensor cores, for
// 16-bit rows of n = 256 .. 32768 (dispatched for n = 32768, where it beats the
// mma.sync kernel by 25 %; at n = 4096 .. 16384 the two are within a few percent
// and the single TMA unit per SM, not the tensor pipe, limits this kernel).  Replaces RowHandler (csrc/hada_handler.cuh:
// 78-219) and its mma.sync rotations (csrc/hada.cuh:104-285) of the reference.
//
// The (rows x n) array is viewed as a matrix of 128-element chunks, one chunk
// per matrix row.  A tile is 128 chunks x 128 elements (32 KB) and goes through
// two dense contractions whose constant operands carry the whole structure of
// the transform ("the permutation is metadata"):
//
//   D1 = T . (s1 H_128)                 tile T as the K-major A operand straight
//                                       from TMA; transforms the 7 low index bits
//   D2 = (I (x) s2 H_cpr) . bf16(D1)    cpr = n/128 chunks per row (<= 128): the
//                                       block-diagonal constant is the A operand,
//                                       D1 (rounded once) is written back into the
//                                       tile's buffer as an MN-major B operand;
//                                       transforms the index bits 7 .. log2(n)-1
//   n = 32768: a row spans the two tiles of a pair; the last bit is an fp32
//              add / subtract between their accumulators in the epilogue.
//
// Accumulators live in TMEM (three 128-column slots used round-robin; D2 overwrites
// D1 once the epilogue has drained it), and so does the constant A operand of the
// second MMA (64 columns), which leaves shared memory for one more tile buffer.  One 32 KB
// shared-memory buffer carries a tile through its life: TMA load -> A operand of
// the first MMA -> B operand of the second -> output staging -> TMA store (plain
// 16-byte stores of one 256-byte chunk per thread were 5x slower).  Six such
// buffers are in flight per SM; warp 11 issues the stores and frees each buffer
// as soon as the store has read it.  Roles: warps 0-3 and 4-7 are two epilogue
// groups (one per tile of a pair), warp 8 issues TMA loads, warp 9 owns TMEM and
// issues the first MMA of every tile, warp 10 the second (two independent issue
// streams, so neither waits behind the other's dependencies).  Every mbarrier wait is time-limited (B200HT_ERR_TIMEOUT).
#include "tc_common.cuh"

namespace b200ht {

constexpr int FT_TILE_BYTES = 32768;
constexpr int FT_NBUF = 6;
constexpr int FT_THREADS = 384;
constexpr int FT_SMEM_BYTES = FT_TILE_BYTES /*H_128*/ + FT_NBUF * FT_TILE_BYTES + 1024 /*align*/ + 512;
constexpr int FT_NSLOT = 3;           // TMEM accumulator slots of 128 columns, used round-robin by the tiles
constexpr uint32_t FT_A2_COL = 384;  // TMEM columns 384..447 hold the constant A operand of the second MMA

// byte offset of element (row, col) of a 128 x 128 16-bit matrix stored as two
// 64-column halves of 128 rows x 128 bytes with the 128-byte swizzle
__device__ __forceinline__ uint32_t sw128_off(int row, int col)
{
    return (uint32_t)((col >> 6) * 16384 + row * 128 + ((((col & 63) >> 3) ^ (row & 7)) << 4) + (col & 7) * 2);
}

// MN-major operand (N contiguous), 128-byte swizzle: 64 N-elements per 128-byte
// row, 8 K-rows per 1024-byte atom, next 8 K-rows 1024 B further (SBO), next 64
// N-elements 16384 B further (LBO).
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t saddr)
{
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(16384 >> 4) << 16;  // leading byte offset
    d |= (uint64_t)(1024 >> 4) << 32;   // stride byte offset
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

template <int DT>
__host__ __device__ constexpr uint32_t ft_idesc(bool b_mn_major)
{
    const uint32_t fmt = DT == B200HT_BF16 ? 1u : 0u;
    return (1u << 4) | (fmt << 7) | (fmt << 10) | (b_mn_major ? (1u << 16) : 0u) | ((uint32_t)(128 >> 3) << 17) |
           ((uint32_t)(128 >> 4) << 24);
}

__device__ __forceinline__ void umma_f16_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// A operand in TMEM (lanes = M rows, two 16-bit K elements per 32-bit column), B from shared memory.
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n" ::"r"(tmem_d),
        "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 32 consecutive 32-bit columns of this thread's TMEM lane <- registers
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t *r)
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
        "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, uint32_t src, int x, int y)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];\n" ::"l"(map), "r"(src),
                 "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;\n" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read1() { asm volatile("cp.async.bulk.wait_group.read 1;\n" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all0() { asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory"); }

// Barrier indices inside the barrier block of shared memory.
struct FtBars {
    uint32_t base;
    __device__ uint32_t full(int b) const { return base + 8u * b; }                  // TMA load landed
    __device__ uint32_t empty(int b) const { return base + 8u * (FT_NBUF + b); }     // TMA store has read the buffer
    __device__ uint32_t b2_ready(int b) const { return base + 8u * (2 * FT_NBUF + b); }  // epilogue 1 wrote B operand
    __device__ uint32_t staged(int b) const { return base + 8u * (3 * FT_NBUF + b); }        // output tile staged in the buffer
    __device__ uint32_t d1_full(int t) const { return base + 8u * (4 * FT_NBUF + t); }
    __device__ uint32_t d2_full(int t) const { return base + 8u * (4 * FT_NBUF + FT_NSLOT + t); }
    __device__ uint32_t tmem_empty(int t) const { return base + 8u * (4 * FT_NBUF + 2 * FT_NSLOT + t); }
};


template <int DT>
__global__ void __launch_bounds__(FT_THREADS, 1)
fwht_tc_kernel(const __grid_constant__ CUtensorMap tmIn, const __grid_constant__ CUtensorMap tmOut, int ntiles,
               int logn, float mult, int *status)
{
    extern __shared__ unsigned char smem_dyn[];
    const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    unsigned char *gen = smem_dyn + (base - smem_u32(smem_dyn));
    const uint32_t b1_s = base, buf_s = base + FT_TILE_BYTES;
    unsigned char *bar_mem = gen + (1 + FT_NBUF) * FT_TILE_BYTES;
    FtBars bars{smem_u32(bar_mem)};
    uint32_t *tmem_slot = (uint32_t *)(bar_mem + 8 * (4 * FT_NBUF + 3 * FT_NSLOT));
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cpr_log = logn - 7;                       // chunks per row, log2 (1..8)
    const bool pair_mode = cpr_log == 8;                // n = 32768: a row spans both tiles of a pair
    const int hbits = cpr_log > 7 ? 7 : cpr_log;        // index bits handled by the second MMA

    // ---- constant B1 = s1 * H_128 (K-major [j'][j]) in shared memory
    {
        const float s1 = 0.125f;
        for (int v = tid; v < 128 * 16; v += FT_THREADS) {   // one 16-byte vector = 8 consecutive columns
            const int r = v >> 4, c0 = (v & 15) * 8;
            uint32_t w1[4];
#pragma unroll
            for (int e = 0; e < 8; e += 2) {
                const float a0 = (__popc((unsigned)(r & (c0 + e))) & 1) ? -s1 : s1;
                const float a1 = (__popc((unsigned)(r & (c0 + e + 1))) & 1) ? -s1 : s1;
                w1[e >> 1] = pack2<DT>(a0, a1);
            }
            *(uint4 *)(gen + sw128_off(r, c0)) = make_uint4(w1[0], w1[1], w1[2], w1[3]);
        }
    }
    if (tid == 0) {
        for (int b = 0; b < FT_NBUF; ++b) {
            mbar_init(bars.full(b), 1);
            mbar_init(bars.empty(b), 1);
            mbar_init(bars.b2_ready(b), 4);   // one arrival per warp of the epilogue group
            mbar_init(bars.staged(b), 4);
        }
        for (int t = 0; t < FT_NSLOT; ++t) {
            mbar_init(bars.d1_full(t), 1);
            mbar_init(bars.d2_full(t), 1);
            mbar_init(bars.tmem_empty(t), pair_mode ? 8 : 4);
        }
        *abort_flag = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tmIn);
        tma_prefetch_desc(&tmOut);
    }
    if (warp == 9) tmem_alloc(smem_u32(tmem_slot), 512);
    fence_proxy_async();   // the constants were written with ordinary stores; the MMAs read them through the async proxy
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // ---- constant A2 = I (x) s2 * H_2^hbits ([c'][c], K = c packed two per 32-bit column) into TMEM
    if (warp < 4) {
        const float s2 = hfrag_c(hbits >= 4 ? 4 : hbits) * (hbits >= 6 ? 0.5f : 1.f);  // 2^-floor(hbits/2)
        const unsigned hmask = (1u << hbits) - 1u;
        const int r = warp * 32 + lane;
        uint32_t w[64];
#pragma unroll
        for (int c = 0; c < 128; c += 2) {
            float a[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                a[h] = 0.f;
                if ((((unsigned)(r ^ (c + h))) & ~hmask & 127u) == 0)
                    a[h] = (__popc((unsigned)(r & (c + h)) & hmask) & 1) ? -s2 : s2;
            }
            w[c >> 1] = pack2<DT>(a[0], a[1]);
        }
        const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + FT_A2_COL;
        tmem_st32(taddr, w);
        tmem_st32(taddr + 32, w + 32);
        asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    // the set-up above touched no global memory; from here on the predecessors' results are needed
    pdl_launch_dependents();
    pdl_wait();

    // work: pairs of consecutive tiles; iteration i of this CTA handles tile (i & 1) of pair blockIdx.x + (i >> 1) * grid
    const int npairs = (ntiles + 1) >> 1;
    const int my_pairs = npairs > (int)blockIdx.x ? (npairs - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    const int iters = 2 * my_pairs;
    auto tile_of = [&](int i) { return 2 * ((int)blockIdx.x + (i >> 1) * (int)gridDim.x) + (i & 1); };

    if (warp == 8) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            int issued = 0;
            for (int i = 0; i < iters; ++i) {
                const int b = i % FT_NBUF;
                const uint32_t ph = (uint32_t)(i / FT_NBUF) & 1u;
                if (!mbar_wait(bars.empty(b), ph ^ 1u, abort_flag, status)) break;
                const int tile = tile_of(i);
                mbar_expect_tx(bars.full(b), FT_TILE_BYTES);
                const uint32_t dst = buf_s + (uint32_t)(b * FT_TILE_BYTES);
                tma_load_2d(dst, &tmIn, 0, tile * 128, bars.full(b));
                tma_load_2d(dst + 16384, &tmIn, 64, tile * 128, bars.full(b));
                issued = i + 1;
            }
            if (*abort_flag) {
                const int pending = issued < FT_NBUF ? issued : FT_NBUF;
                for (int j = 0; j < pending; ++j) {
                    const int i2 = issued - 1 - j;
                    const uint64_t t0 = global_ns();
                    while (!mbar_test(bars.full(i2 % FT_NBUF), (uint32_t)(i2 / FT_NBUF) & 1u) &&
                           global_ns() - t0 < 100000000ull) {}
                }
            }
        }
        __syncwarp();
    } else if (warp == 9) {
        // ------------------------------ first MMA of every tile ------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc1 = ft_idesc<DT>(false);
            for (int i = 0; i < iters; ++i) {
                const int b = i % FT_NBUF, t = i % FT_NSLOT;
                if (!mbar_wait(bars.full(b), (uint32_t)(i / FT_NBUF) & 1u, abort_flag, status)) break;
                if (!mbar_wait(bars.tmem_empty(t), ((uint32_t)(i / FT_NSLOT) & 1u) ^ 1u, abort_flag, status)) break;
                tc_fence_after();
                const uint32_t a_s = buf_s + (uint32_t)(b * FT_TILE_BYTES);
                const uint32_t d1 = tmem_base + (uint32_t)(t * 128);
#pragma unroll
                for (int s = 0; s < 8; ++s) {
                    const uint32_t koff = (uint32_t)((s >> 2) * 16384 + (s & 3) * 32);
                    umma_f16_ss(d1, umma_desc_k_sw128(a_s + koff), umma_desc_k_sw128(b1_s + koff), idesc1, s ? 1u : 0u);
                }
                umma_commit(bars.d1_full(t));
            }
        }
        __syncwarp();
    } else if (warp == 10) {
        // ------------------------------ second MMA of every tile ------------------------------
        if (lane == 0 && cpr_log > 0) {
            constexpr uint32_t idesc2 = ft_idesc<DT>(true);
            for (int j = 0; j < iters; ++j) {
                const int b = j % FT_NBUF, t = j % FT_NSLOT;
                if (!mbar_wait(bars.b2_ready(b), (uint32_t)(j / FT_NBUF) & 1u, abort_flag, status)) break;
                tc_fence_after();
                const uint32_t b_s = buf_s + (uint32_t)(b * FT_TILE_BYTES);
                const uint32_t d2 = tmem_base + (uint32_t)(t * 128);   // overwrites D1, which epilogue 1 has drained
#pragma unroll
                for (int s = 0; s < 8; ++s) {
                    umma_f16_ts(d2, tmem_base + FT_A2_COL + (uint32_t)(s * 8), umma_desc_mn_sw128(b_s + (uint32_t)(s * 2048)),
                                idesc2, s ? 1u : 0u);
                }
                umma_commit(bars.d2_full(t));
            }
        }
        __syncwarp();
    } else if (warp < 8) {
        // ------------------------------ epilogue groups ------------------------------
        const int grp = warp >> 2;            // tile of the pair handled by this group
        const int q = warp & 3;               // TMEM lane quadrant
        const int row = q * 32 + lane;        // chunk index inside the tile = TMEM lane
        const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
        bool ok = true;
        for (int i = grp; i < iters && ok; i += 2) {
            const int b = i % FT_NBUF, t = i % FT_NSLOT;
            const int io = i ^ 1, to = io % FT_NSLOT;          // the other tile of the pair and its slot
            const uint32_t tph = (uint32_t)(i / FT_NSLOT) & 1u, tpho = (uint32_t)(io / FT_NSLOT) & 1u;
            unsigned char *bufp = gen + (1 + b) * FT_TILE_BYTES;
            if (cpr_log > 0) {
                // D1 -> 16-bit -> MN-major B operand in the tile's own buffer (the first MMA is done with it)
                if (!mbar_wait(bars.d1_full(t), tph, abort_flag, status)) { ok = false; break; }
                tc_fence_after();
                {
                    uint32_t r[4][32];
#pragma unroll
                    for (int c = 0; c < 4; ++c) tmem_ld32(tmem_base + lane_addr + (uint32_t)(t * 128 + 32 * c), r[c]);
                    tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
#pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            uint4 o;
                            o.x = pack2<DT>(__uint_as_float(r[c][8 * v + 0]), __uint_as_float(r[c][8 * v + 1]));
                            o.y = pack2<DT>(__uint_as_float(r[c][8 * v + 2]), __uint_as_float(r[c][8 * v + 3]));
                            o.z = pack2<DT>(__uint_as_float(r[c][8 * v + 4]), __uint_as_float(r[c][8 * v + 5]));
                            o.w = pack2<DT>(__uint_as_float(r[c][8 * v + 6]), __uint_as_float(r[c][8 * v + 7]));
                            *(uint4 *)(bufp + sw128_off(row, 32 * c + 8 * v)) = o;
                        }
                    }
                }
                fence_proxy_async();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bars.b2_ready(b));
                if (!mbar_wait(bars.d2_full(t), tph, abort_flag, status)) { ok = false; break; }
                if (pair_mode && !mbar_wait(bars.d2_full(to), tpho, abort_flag, status)) { ok = false; break; }
            } else {
                if (!mbar_wait(bars.d1_full(t), tph, abort_flag, status)) { ok = false; break; }
            }
            tc_fence_after();
            // final accumulator -> scale -> 16 bit -> output staging in the same buffer (the second MMA is done with it)
            const uint32_t dcol = (uint32_t)(t * 128);
            const uint32_t ocol = (uint32_t)(to * 128);
#pragma unroll 1
            for (int c0 = 0; c0 < 128; c0 += 64) {
                uint32_t r[2][32];
                float f[2][32];
                tmem_ld32(tmem_base + lane_addr + dcol + (uint32_t)c0, r[0]);
                tmem_ld32(tmem_base + lane_addr + dcol + (uint32_t)(c0 + 32), r[1]);
                if (pair_mode) {
                    uint32_t r2[2][32];
                    tmem_ld32(tmem_base + lane_addr + ocol + (uint32_t)c0, r2[0]);
                    tmem_ld32(tmem_base + lane_addr + ocol + (uint32_t)(c0 + 32), r2[1]);
                    tmem_ld_wait();
#pragma unroll
                    for (int h = 0; h < 2; ++h)
#pragma unroll
                        for (int e = 0; e < 32; ++e) {
                            const float mine = __uint_as_float(r[h][e]), other = __uint_as_float(r2[h][e]);
                            f[h][e] = (grp == 0 ? mine + other : other - mine) * mult;   // tile 0: a + b, tile 1: a - b
                        }
                } else {
                    tmem_ld_wait();
#pragma unroll
                    for (int h = 0; h < 2; ++h)
#pragma unroll
                        for (int e = 0; e < 32; ++e) f[h][e] = __uint_as_float(r[h][e]) * mult;
                }
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        uint4 o;
                        o.x = pack2<DT>(f[h][8 * v + 0], f[h][8 * v + 1]);
                        o.y = pack2<DT>(f[h][8 * v + 2], f[h][8 * v + 3]);
                        o.z = pack2<DT>(f[h][8 * v + 4], f[h][8 * v + 5]);
                        o.w = pack2<DT>(f[h][8 * v + 6], f[h][8 * v + 7]);
                        *(uint4 *)(bufp + sw128_off(row, c0 + 32 * h + 8 * v)) = o;
                    }
            }
            // accumulators drained and tile staged: hand the TMEM slot(s) to the MMA warp, the buffer to the store warp
            fence_proxy_async();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(bars.tmem_empty(t));
                if (pair_mode) mbar_arrive(bars.tmem_empty(to));
                mbar_arrive(bars.staged(b));
            }
        }
    }
    if (warp == 11 && lane == 0) {
        // ------------------------------ TMA store ------------------------------
        int prev_b = -1;
        for (int i = 0; i < iters; ++i) {
            const int b = i % FT_NBUF;
            if (!mbar_wait(bars.staged(b), (uint32_t)(i / FT_NBUF) & 1u, abort_flag, status)) break;
            const int tile = tile_of(i);
            const uint32_t src = buf_s + (uint32_t)(b * FT_TILE_BYTES);
            tma_store_2d(&tmOut, src, 0, tile * 128);
            tma_store_2d(&tmOut, src + 16384, 64, tile * 128);
            bulk_commit();
            if (prev_b >= 0) {
                bulk_wait_read1();                 // the previous store has read its buffer
                mbar_arrive(bars.empty(prev_b));
            }
            prev_b = b;
        }
        bulk_wait_read0();
        if (prev_b >= 0) mbar_arrive(bars.empty(prev_b));
        bulk_wait_all0();                          // all stores complete before the CTA exits
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}


template <int DT>
static int launch_ft(const void *in, void *out, uint64_t chunk_rows, int logn, float scale, cudaStream_t st)
{
    CUtensorMap tin, tout;
    int rc = encode_tmap_b16_2d(&tin, in, chunk_rows, 128, 128, DT);
    if (rc) return rc;
    rc = encode_tmap_b16_2d(&tout, out, chunk_rows, 128, 128, DT);
    if (rc) return rc;
    rc = ensure_dyn_smem((const void *)fwht_tc_kernel<DT>, FT_SMEM_BYTES);
    if (rc) return rc;
    const int ntiles = (int)((chunk_rows + 127) / 128);
    const int npairs = (ntiles + 1) / 2;
    const int grid = npairs < sm_count() ? npairs : sm_count();
    // factors baked into the constants: 2^-3 for H_128, 2^-floor(hbits/2) for the second contraction
    const int cpr_log = logn - 7;
    const int hbits = cpr_log > 7 ? 7 : cpr_log;
    const float applied = 0.125f * exp2f(-(float)(hbits / 2));
    return launch_pdl(fwht_tc_kernel<DT>, dim3(grid), dim3(FT_THREADS), (size_t)FT_SMEM_BYTES, st, tin, tout, ntiles,
                      logn, scale / applied, status_word_ptr());
}

// rows x n 16-bit, 128 <= n <= 32768, in/out 128-byte aligned (TMA); returns B200HT_ERR_ALIGN otherwise.
int launch_fwht_tc(const void *in, void *out, uint64_t rows, int logn, int dtype, float scale, cudaStream_t st)
{
    if (logn < 7 || logn > 15) return B200HT_ERR_SIZE;
    if ((reinterpret_cast<uintptr_t>(in) & 127u) || (reinterpret_cast<uintptr_t>(out) & 127u)) return B200HT_ERR_ALIGN;
    const uint64_t chunk_rows = rows << (logn - 7);
    if (chunk_rows > 0x7fffffffull) return B200HT_ERR_SIZE;
    return dtype == B200HT_BF16 ? launch_ft<B200HT_BF16>(in, out, chunk_rows, logn, scale, st)
                                : launch_ft<B200HT_F16>(in, out, chunk_rows, logn, scale, st);
}

}  // namespace b200ht
