// bf16 x bf16 -> fp32 contraction  C[m, t] = sum_k W[m, k] * Y[t, k]  on the
// 5th-generation tensor cores.  Y = scale * H(X) is the transformed token
// matrix produced by fwht.cu; this kernel is the second phase of
// b200ht_fused_gemm for bf16 inputs and replaces the scalar-FMA GEMM of
// fused_ht_gemm_pipelined (fused_ht/fusion_pipelined.cu:468-543).
//
// Persistent, warp-specialised, one CTA per SM:
//   warp 0      TMA producer: W tile (128 x 64) and Y tile (256 x 64) per stage,
//               128-byte swizzle, 4-stage mbarrier ring
//   warp 1      allocates TMEM (512 columns = two 128 x 256 fp32 accumulators)
//               and issues tcgen05.mma (M=128, N=256, K=16) from one thread
//   warps 2..5  epilogue: tcgen05.ld of the finished accumulator, convert,
//               store, while the next tile accumulates in the other TMEM half.
//               Token-major results are stored directly (a warp writes 32
//               consecutive elements); M x N results are staged per warp in
//               shared memory and written by TMA (32 rows x 128 bytes per op)
// Every mbarrier wait is time-limited; on expiry the CTA drains and exits and
// the device status word carries B200HT_ERR_TIMEOUT.
#include <cstdlib>
#include <mutex>

#include "tc_common.cuh"

namespace b200ht {

// CTA tile: (128 * MT) rows of W x 256 tokens x 64 k per stage.  MT = 2 halves the operand bytes fetched per flop
// (the token tile is shared by two 128-row MMAs) at the price of a single accumulator set, i.e. an epilogue that
// is not overlapped with the next tile; MT = 1 double-buffers the accumulator and gives twice as many tiles.
constexpr int TC_BN = 256, TC_BK = 64;
template <int MT>
struct TcCfg {
    static constexpr int BM = 128 * MT;
    static constexpr int STAGES = MT == 1 ? 4 : 3;
    static constexpr int A_BYTES = BM * TC_BK * 2;      // 16 / 32 KB
    static constexpr int B_BYTES = TC_BN * TC_BK * 2;   // 32 KB
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STORE_BUFS = MT == 1 ? 2 : 1;    // 4 KB staging buffers per epilogue warp (M x N layout)
    static constexpr int STORE_BYTES = 4 * MT * STORE_BUFS * 4096;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STORE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
    static constexpr int NACC = MT == 1 ? 2 : 1;        // accumulator sets in TMEM
    static constexpr int THREADS = 64 + 128 * MT;       // TMA warp, MMA warp, 4 * MT epilogue warps
};

// Optional epilogue scales: C[m, t] is multiplied by row_scale[m] (per output channel) and tok_scale[t] (per token)
// before the store; `rs` is this lane's row factor (1 when there is none), `n` the token of r[0].
__device__ __forceinline__ void tc_scale_chunk(uint32_t (&r)[32], float rs, const float *tok_scale, int n, int N)
{
    if (tok_scale) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const float ts = n + j < N ? __ldg(tok_scale + n + j) : 0.f;
            r[j] = __float_as_uint(__uint_as_float(r[j]) * (rs * ts));
        }
    } else if (rs != 1.f) {
#pragma unroll
        for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * rs);
    }
}

// `ld` is the leading dimension of C in elements (N for M x N, M for N x M, larger when C is a block of a bigger
// matrix).
template <int OUT_DT, int LAYOUT>
__device__ __forceinline__ void tc_store_chunk(void *C, int M, int N, size_t ld, int m, int n, const uint32_t (&r)[32])
{
    if (m >= M || n >= N) return;
    if constexpr (LAYOUT == B200HT_OUT_NM) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            if (n + j < N) {
                const size_t idx = (size_t)(n + j) * ld + m;
                if constexpr (OUT_DT == B200HT_F32) ((float *)C)[idx] = __uint_as_float(r[j]);
                else ((__nv_bfloat16 *)C)[idx] = __float2bfloat16_rn(__uint_as_float(r[j]));
            }
        }
    } else {
        if constexpr (OUT_DT == B200HT_F32) {
            float *p = (float *)C + (size_t)m * ld + n;
            if ((ld & 3) == 0 && n + 32 <= N) {
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                    *(float4 *)(p + j) = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                                     __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (n + j < N) p[j] = __uint_as_float(r[j]);
            }
        } else {
            __nv_bfloat16 *p = (__nv_bfloat16 *)C + (size_t)m * ld + n;
            if ((ld & 7) == 0 && n + 32 <= N) {
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                    uint4 v;
                    v.x = pack2<B200HT_BF16>(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
                    v.y = pack2<B200HT_BF16>(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                    v.z = pack2<B200HT_BF16>(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]));
                    v.w = pack2<B200HT_BF16>(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
                    *(uint4 *)(p + j) = v;
                }
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (n + j < N) p[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
            }
        }
    }
}

// Tile order.  The tiles of one "wave" (one per SM, consecutive tile numbers) should share operand blocks, and what
// one wave leaves in the 126 MB L2 should serve the next.
//   order 0: groups of `group` row blocks of W; inside a group the token blocks advance slowest, so the W rows of
//            the group stay L2-resident while the whole token range streams past them.
//   order 1: groups of `group` token blocks; inside a group the row blocks of W advance slowest, so the tokens of
//            the group (transformed just before, still in L2) stay resident while W streams past them once.
struct TileOrder {
    int group;
    int order;
};
__device__ __forceinline__ void tc_tile_coord(int tile, int mt, int nt, TileOrder ord, int &mb, int &nb)
{
    const int inner_cnt = ord.order == 0 ? mt : nt;    // blocks along the grouped dimension
    const int outer_cnt = ord.order == 0 ? nt : mt;
    const int per_group = ord.group * outer_cnt;
    const int grp = tile / per_group;
    const int rem = tile - grp * per_group;
    const int left = inner_cnt - grp * ord.group;
    const int gsz = left < ord.group ? left : ord.group;
    const int o = rem / gsz;
    const int i = grp * ord.group + (rem - o * gsz);
    mb = ord.order == 0 ? i : o;
    nb = ord.order == 0 ? o : i;
}

template <int OUT_DT, int LAYOUT, int MT>
__global__ void __launch_bounds__(TcCfg<MT>::THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmY,
               const __grid_constant__ CUtensorMap tmC, int tma_store, void *C, int M, int N, int K, size_t ldc,
               int ntiles_run, int pdl_mode, TileOrder ord, const float *row_scale, const float *tok_scale, int *status)
{
    using Cfg = TcCfg<MT>;
    constexpr int STAGES = Cfg::STAGES, STAGE_BYTES = Cfg::STAGE_BYTES, NACC = Cfg::NACC;
    extern __shared__ unsigned char smem_dyn[];
    const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    const uint32_t store_base = base + STAGES * STAGE_BYTES;   // 1024-byte aligned staging for the TMA-store epilogue
    const uint32_t bar_base = store_base + Cfg::STORE_BYTES;
    // barriers: full[S], empty[S], tmem_full[2], tmem_empty[2]; then tmem address slot, abort flag
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
    unsigned char *gen_base = smem_dyn + (base - smem_u32(smem_dyn));
    uint32_t *tmem_slot = (uint32_t *)(gen_base + STAGES * STAGE_BYTES + Cfg::STORE_BYTES + 8 * (2 * STAGES + 4));
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 4 * MT);  // one arrival per epilogue warp
        }
        *abort_flag = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tmW);
        tma_prefetch_desc(&tmY);
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // programmatic dependent launch: everything above overlapped the tail of the transform kernel that
    // produces the token operand; from here on its output is needed
    // Programmatic dependent launch.  Mode 0: let the next kernel of the stream be scheduled at once, then wait for
    // everything before this kernel.  A GEMM that is split into two launches (256-row tiles for the whole waves,
    // 128-row tiles for the rest) uses mode 1 for the first -- the second launch is released only after this one has
    // seen the transform complete -- and mode 2 for the second: it starts without waiting (its inputs are complete
    // by then and its output block is disjoint from the first launch's) and waits for the first launch before it
    // ends, so that later work in the stream still sees both finished.
    if (pdl_mode == 1) {
        pdl_wait();
        pdl_launch_dependents();
    } else {
        pdl_launch_dependents();
        if (pdl_mode == 0) pdl_wait();
    }

    const int mt = (M + Cfg::BM - 1) / Cfg::BM, nt = (N + TC_BN - 1) / TC_BN;
    const int ntiles = ntiles_run < mt * nt ? ntiles_run : mt * nt;   // tiles beyond it belong to a second launch
    const int kblocks = K / TC_BK;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
                int mb, nb;
                tc_tile_coord(tile, mt, nt, ord, mb, nb);
                const int m0 = mb * Cfg::BM, n0 = nb * TC_BN;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1u;
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, status)) { ok = false; break; }
                    mbar_expect_tx(full_bar(s), STAGE_BYTES);
                    const uint32_t sa = base + s * STAGE_BYTES;
                    tma_load_2d(sa, &tmW, kb * TC_BK, m0, full_bar(s));
                    tma_load_2d(sa + Cfg::A_BYTES, &tmY, kb * TC_BK, n0, full_bar(s));
                }
            }
            if (!ok) {
                // copies already issued still land in this CTA's shared memory: give them time
                const uint32_t pending = it < (uint32_t)STAGES ? it : (uint32_t)STAGES;
                for (uint32_t j = 0; j < pending; ++j) {
                    const uint32_t i2 = it - 1 - j;
                    const uint64_t t0 = global_ns();
                    while (!mbar_test(full_bar(i2 % STAGES), (i2 / STAGES) & 1u) &&
                           global_ns() - t0 < 100000000ull) {}
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(128, TC_BN);
            uint32_t it = 0, tcount = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, ++tcount) {
                const int acc = tcount % NACC;
                const uint32_t aph = (tcount / NACC) & 1u;
                if (!mbar_wait(tempty_bar(acc), aph ^ 1u, abort_flag, status)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * TC_BN;   // MT == 2: halves at columns 0 and 256
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1u;
                    if (!mbar_wait(full_bar(s), ph, abort_flag, status)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = base + s * STAGE_BYTES;
                    const uint64_t bdesc = umma_desc_k_sw128(sa + Cfg::A_BYTES);
#pragma unroll
                    for (int h = 0; h < MT; ++h) {
                        const uint64_t adesc = umma_desc_k_sw128(sa + h * 16384);
#pragma unroll
                        for (int k = 0; k < TC_BK / 16; ++k)
                            umma_bf16_ss(d_tmem + h * TC_BN, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) ? 1u : 0u);
                    }
                    umma_commit(empty_bar(s));
                }
                if (ok) umma_commit(tfull_bar(acc));
            }
        }
        __syncwarp();
    } else {
        const int q = warp & 3;          // TMEM lane quadrant this warp may read
        const int h = (warp - 2) >> 2;   // 128-row half of the tile drained by this warp
        uint32_t tcount = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, ++tcount) {
            const int acc = tcount % NACC;
            const uint32_t aph = (tcount / NACC) & 1u;
            int mb, nb;
            tc_tile_coord(tile, mt, nt, ord, mb, nb);
            const int m0 = mb * Cfg::BM, n0 = nb * TC_BN;
            if (!mbar_wait(tfull_bar(acc), aph, abort_flag, status)) { ok = false; break; }
            tc_fence_after();
            bool released = false;   // set where the accumulator is handed back before the stores
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (acc + h) * TC_BN;
            const int m = m0 + h * 128 + q * 32 + lane;
            const float rs = row_scale && m < M ? __ldg(row_scale + m) : 1.f;
            if (LAYOUT == B200HT_OUT_MN && tma_store) {
                // M x N layout: a lane owns a row, so plain stores would scatter 16-byte pieces over 32 rows.
                // Stage 32 rows x 128 bytes per warp in shared memory (128-byte swizzle) and let TMA write them.
                constexpr int COLS = OUT_DT == B200HT_F32 ? 32 : 64;       // columns per 128-byte staging row
                unsigned char *stage_gen = gen_base + STAGES * STAGE_BYTES + (warp - 2) * Cfg::STORE_BUFS * 4096;
                const uint32_t stage_s = store_base + (uint32_t)((warp - 2) * Cfg::STORE_BUFS * 4096);
                int sb = 0;
#pragma unroll 1
                for (int c = 0; c < TC_BN; c += COLS) {
                    uint32_t r[32], r2[32];
                    tmem_ld32(taddr + c, r);
                    if (OUT_DT != B200HT_F32) tmem_ld32(taddr + c + 32, r2);
                    tmem_ld_wait();
                    tc_scale_chunk(r, rs, tok_scale, n0 + c, N);
                    if (OUT_DT != B200HT_F32) tc_scale_chunk(r2, rs, tok_scale, n0 + c + 32, N);
                    // the buffer about to be overwritten must have been read by its previous store
                    if (lane == 0) {
                        if (Cfg::STORE_BUFS == 2) asm volatile("cp.async.bulk.wait_group.read 1;\n" ::: "memory");
                        else asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory");
                    }
                    __syncwarp();
                    unsigned char *row = stage_gen + sb * 4096 + lane * 128;
#pragma unroll
                    for (int v = 0; v < 8; ++v) {
                        uint4 o;
                        if (OUT_DT == B200HT_F32) {
                            o = make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
                        } else {
                            const uint32_t *src = v < 4 ? r + 8 * v : r2 + 8 * (v - 4);
                            o.x = pack2<B200HT_BF16>(__uint_as_float(src[0]), __uint_as_float(src[1]));
                            o.y = pack2<B200HT_BF16>(__uint_as_float(src[2]), __uint_as_float(src[3]));
                            o.z = pack2<B200HT_BF16>(__uint_as_float(src[4]), __uint_as_float(src[5]));
                            o.w = pack2<B200HT_BF16>(__uint_as_float(src[6]), __uint_as_float(src[7]));
                        }
                        *(uint4 *)(row + ((v ^ (lane & 7)) << 4)) = o;
                    }
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) {
                        asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];\n" ::"l"(&tmC),
                                     "r"(stage_s + (uint32_t)(sb * 4096)), "r"(n0 + c), "r"(m0 + h * 128 + q * 32)
                                     : "memory");
                        asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
                    }
                    sb = (sb + 1) % Cfg::STORE_BUFS;
                }
            } else if (LAYOUT == B200HT_OUT_NM && OUT_DT == B200HT_BF16 && m0 + Cfg::BM <= M && n0 + TC_BN <= N &&
                       (ldc & 7) == 0 && ((uintptr_t)C & 15u) == 0) {
                // Token-major bf16 result, tile fully inside C.  A lane owns a row m, so stores straight from the
                // registers are 2 bytes per lane and 64 contiguous bytes per instruction.  Instead the four warps of
                // a 128-row half stage 32 tokens x 128 rows in shared memory (two buffers, one named barrier per
                // chunk) and write them out as 16 bytes per lane, 256 contiguous bytes per token.
                unsigned char *stage_gen = gen_base + STAGES * STAGE_BYTES + h * 16384;
                const int bar_id = 1 + h;
                const int tok_sub = lane >> 4, seg = lane & 15;   // read-back: 2 tokens per instruction, 16 lanes each
                // 1. drain the accumulator into registers (two bf16 per register: 128 registers for 256 tokens) and
                //    hand the TMEM columns back at once, so the next tile's MMAs run underneath the stores
                uint32_t pk[TC_BN / 2];
#pragma unroll
                for (int cc = 0; cc < TC_BN / 32; ++cc) {
                    uint32_t r[32];
                    tmem_ld32(taddr + cc * 32, r);
                    tmem_ld_wait();
                    tc_scale_chunk(r, rs, tok_scale, n0 + cc * 32, N);
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        pk[cc * 16 + j] = pack2<B200HT_BF16>(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tempty_bar(acc));
                released = true;
                // 2. stage and store, 32 tokens at a time
#pragma unroll
                for (int cc = 0; cc < TC_BN / 32; ++cc) {
                    unsigned char *buf = stage_gen + (cc & 1) * 8192;
                    unsigned short *col = (unsigned short *)buf + q * 32 + lane;
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        col[(2 * j) * 128] = (unsigned short)(pk[cc * 16 + j] & 0xffffu);
                        col[(2 * j + 1) * 128] = (unsigned short)(pk[cc * 16 + j] >> 16);
                    }
                    asm volatile("bar.sync %0, 128;\n" ::"r"(bar_id) : "memory");
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int j = q * 8 + i * 2 + tok_sub;   // token of the chunk written by this lane
                        const uint4 v = *(const uint4 *)(buf + j * 256 + seg * 16);
                        *(uint4 *)((__nv_bfloat16 *)C + (size_t)(n0 + cc * 32 + j) * ldc + m0 + h * 128 + seg * 8) = v;
                    }
                }
            } else {
#pragma unroll 1
                for (int c = 0; c < TC_BN; c += 32) {
                    uint32_t r[32];
                    tmem_ld32(taddr + c, r);
                    tmem_ld_wait();
                    tc_scale_chunk(r, rs, tok_scale, n0 + c, N);
                    tc_store_chunk<OUT_DT, LAYOUT>(C, M, N, ldc, m, n0 + c, r);
                }
            }
            if (!released) {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tempty_bar(acc));
            }
        }
        if (LAYOUT == B200HT_OUT_MN && tma_store && lane == 0)
            asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory");   // this warp's stores are complete
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
    if (pdl_mode == 2 && threadIdx.x == 0) pdl_wait();
}

// ---------------------------------------------------------------------------
// K < 64 (the 128-byte swizzled tile needs 64 bf16 per row): plain SIMT kernel.
// ---------------------------------------------------------------------------
__global__ void gemm_bf16_smallk_kernel(const __nv_bfloat16 *Y, const __nv_bfloat16 *W, void *C, int M, int N,
                                        int K, int out_dtype, int out_layout, const float *row_scale,
                                        const float *tok_scale)
{
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    const int m = blockIdx.y * blockDim.y + threadIdx.y;
    if (m >= M || n >= N) return;
    float acc = 0.f;
    for (int k = 0; k < K; ++k)
        acc = fmaf(__bfloat162float(W[(size_t)m * K + k]), __bfloat162float(Y[(size_t)n * K + k]), acc);
    if (row_scale) acc *= row_scale[m];
    if (tok_scale) acc *= tok_scale[n];
    const size_t idx = out_layout == B200HT_OUT_MN ? (size_t)m * N + n : (size_t)n * M + m;
    if (out_dtype == B200HT_F32) ((float *)C)[idx] = acc;
    else ((__nv_bfloat16 *)C)[idx] = __float2bfloat16_rn(acc);
}

// ---------------------------------------------------------------------------
// host
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn()
{
    static std::mutex mu;
    static EncodeTiledFn fn = nullptr;
    std::lock_guard<std::mutex> lk(mu);
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// Tensor maps depend only on (address, shape, box, element type), so the maps of buffers a caller reuses call after
// call are kept in a small per-thread table (no lock); a miss encodes through the driver and replaces one entry.
struct TmapKey {
    const void *base;
    uint64_t rows, cols, ld;
    uint32_t box_rows, box_chunks;
    int kind, dtype, dev;
    bool operator==(const TmapKey &o) const
    {
        return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows &&
               box_chunks == o.box_chunks && kind == o.kind && dtype == o.dtype && dev == o.dev;
    }
};
struct TmapSlot {
    TmapKey key;
    CUtensorMap map;
    bool valid;
};
constexpr int kTmapSlots = 64;

template <typename Encode>
static int tmap_cached(CUtensorMap *out, TmapKey key, Encode encode)
{
    static thread_local TmapSlot table[kTmapSlots];
    if (cudaGetDevice(&key.dev) != cudaSuccess) key.dev = -1;
    uint64_t h = (uint64_t)(uintptr_t)key.base * 0x9E3779B97F4A7C15ull;
    h ^= (key.rows * 31 + key.cols * 17 + key.ld * 13 + key.box_rows * 7 + key.box_chunks * 5 + (uint64_t)key.kind * 3 +
          (uint64_t)key.dtype) * 0xC2B2AE3D27D4EB4Full;
    TmapSlot &slot = table[(h >> 32) % kTmapSlots];
    if (slot.valid && slot.key == key) {
        *out = slot.map;
        return 0;
    }
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return (int)cudaErrorNotSupported;
    const CUresult r = encode(fn, out);
    if (r != CUDA_SUCCESS) return (int)cudaErrorInvalidValue;
    slot.key = key;
    slot.map = *out;
    slot.valid = true;
    return 0;
}

int encode_tmap_b16_2d(CUtensorMap *map, const void *base, uint64_t rows, uint64_t cols, uint32_t box_rows,
                       int dtype)
{
    return tmap_cached(map, TmapKey{base, rows, cols, cols, box_rows, 0, 0, dtype, 0},
                       [&](EncodeTiledFn fn, CUtensorMap *m) {
        const cuuint64_t dims[2] = {cols, rows};
        const cuuint64_t strides[1] = {cols * 2};
        const cuuint32_t box[2] = {64, box_rows};
        const cuuint32_t estr[2] = {1, 1};
        const CUtensorMapDataType dt =
            dtype == B200HT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
        return fn(m, dt, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    });
}

int encode_tmap_bf16_2d(CUtensorMap *map, const void *base, uint64_t rows, uint64_t cols, uint32_t box_rows)
{
    return encode_tmap_b16_2d(map, base, rows, cols, box_rows, B200HT_BF16);
}

// 3-D view of a row-major bf16 matrix (rows x cols, cols % 64 == 0) as [64 k][rows][cols/64 chunks], so that
// one box {64, box_rows, box_chunks} fetches box_rows x (64*box_chunks) elements and lands in shared memory as
// box_chunks consecutive K-major tiles of box_rows x 128 bytes with 128-byte swizzle.
int encode_tmap_bf16_rows_chunks(CUtensorMap *map, const void *base, uint64_t rows, uint64_t cols,
                                 uint32_t box_rows, uint32_t box_chunks)
{
    return tmap_cached(map, TmapKey{base, rows, cols, cols, box_rows, box_chunks, 1, B200HT_BF16, 0},
                       [&](EncodeTiledFn fn, CUtensorMap *m) {
        const cuuint64_t dims[3] = {64, rows, cols / 64};
        const cuuint64_t strides[2] = {cols * 2, 128};
        const cuuint32_t box[3] = {64, box_rows, box_chunks};
        const cuuint32_t estr[3] = {1, 1, 1};
        return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    });
}

int encode_tmap_bf16_row_groups(CUtensorMap *map, const void *base, uint64_t group_rows, uint64_t groups, uint64_t cols,
                                uint32_t box_rows, uint32_t box_chunks)
{
    return tmap_cached(map, TmapKey{base, groups, cols, group_rows, box_rows, box_chunks, 3, B200HT_BF16, 0},
                       [&](EncodeTiledFn fn, CUtensorMap *m) {
        const cuuint64_t dims[4] = {64, group_rows, groups, cols / 64};
        const cuuint64_t strides[3] = {cols * 2, group_rows * cols * 2, 128};
        const cuuint32_t box[4] = {64, box_rows, 1, box_chunks};
        const cuuint32_t estr[4] = {1, 1, 1, 1};
        return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void *>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    });
}

// Output map for the TMA-store epilogue: rows x cols of fp32 or bf16, box = 32 rows x 128 bytes, 128-byte swizzle.
static int encode_tmap_out_2d(CUtensorMap *map, const void *base, uint64_t rows, uint64_t cols, uint64_t ld, int dtype)
{
    return tmap_cached(map, TmapKey{base, rows, cols, ld, 32, 0, 2, dtype, 0}, [&](EncodeTiledFn fn, CUtensorMap *m) {
        const uint64_t esz = dtype == B200HT_F32 ? 4 : 2;
        const cuuint64_t dims[2] = {cols, rows};
        const cuuint64_t strides[1] = {ld * esz};
        const cuuint32_t box[2] = {(cuuint32_t)(128 / esz), 32};
        const cuuint32_t estr[2] = {1, 1};
        return fn(m, dtype == B200HT_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                  const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    });
}

template <int OUT_DT, int LAYOUT, int MT>
static int launch_tc_mt(const void *Y, const void *W, void *C, int M, int N, int K, size_t ldc, int skip_last_tiles,
                        int pdl_mode, TileOrder ord, const float *row_scale, const float *tok_scale, cudaStream_t st)
{
    using Cfg = TcCfg<MT>;
    CUtensorMap tw, ty;
    int rc = encode_tmap_bf16_2d(&tw, W, (uint64_t)M, (uint64_t)K, Cfg::BM);
    if (rc) return rc;
    rc = encode_tmap_bf16_2d(&ty, Y, (uint64_t)N, (uint64_t)K, TC_BN);
    if (rc) return rc;
    // M x N results go out through TMA (32 rows x 128 bytes per op) when rows of C are 16-byte multiples
    CUtensorMap tc = tw;
    int tma_store = 0;
    if (LAYOUT == B200HT_OUT_MN) {
        const uint64_t esz = OUT_DT == B200HT_F32 ? 4 : 2;
        if (((uint64_t)ldc * esz) % 16 == 0 && ((uintptr_t)C & 15u) == 0 &&
            encode_tmap_out_2d(&tc, C, (uint64_t)M, (uint64_t)N, (uint64_t)ldc, OUT_DT) == 0)
            tma_store = 1;
    }
    rc = ensure_dyn_smem((const void *)gemm_tc_kernel<OUT_DT, LAYOUT, MT>, Cfg::SMEM_BYTES);
    if (rc) return rc;
    const int tiles = ((M + Cfg::BM - 1) / Cfg::BM) * ((N + TC_BN - 1) / TC_BN) - skip_last_tiles;
    const int grid = tiles < sm_count() ? tiles : sm_count();
    return launch_pdl(gemm_tc_kernel<OUT_DT, LAYOUT, MT>, dim3(grid), dim3(Cfg::THREADS), (size_t)Cfg::SMEM_BYTES, st,
                      tw, ty, tc, tma_store, C, M, N, K, ldc, tiles, pdl_mode, ord, row_scale, tok_scale, status_word_ptr());
}

template <int OUT_DT, int LAYOUT>
static int launch_tc(const void *Y, const void *W, void *C, int M, int N, int K, size_t ldc_arg, const float *row_scale,
                     const float *tok_scale, cudaStream_t st)
{
    // 256-row or 128-row CTA tiles: whichever needs less time in units of a 128-row tile, counting whole waves
    // over the SMs (a 256-row tile costs two units; 128-row tiles pay about 3 % more for operand traffic).
    // B200HT_GEMM_MT=1|2 forces one of them, B200HT_GEMM_SPLIT=0 disables the two-launch form (tuning knobs).
    static const int force_mt = [] {
        const char *e = std::getenv("B200HT_GEMM_MT");
        return e ? std::atoi(e) : 0;
    }();
    static const bool allow_split = [] {
        const char *e = std::getenv("B200HT_GEMM_SPLIT");
        return !(e && e[0] == '0');
    }();
    // Default: groups of 8 token blocks (2048 tokens: one 32 MB chunk of transformed tokens at K = 8192), the order
    // with the least DRAM traffic measured on the K = 8192, M = 28672 shape (L2 eviction hints on the TMA loads were
    // tried on top of it and raised the traffic).  B200HT_GEMM_GROUP=<blocks> and B200HT_GEMM_ORDER=0|1 override it
    // (tuning knobs).
    static const TileOrder ord = [] {
        TileOrder o{8, 1};
        if (const char *e = std::getenv("B200HT_GEMM_GROUP")) {
            const int v = std::atoi(e);
            if (v >= 1 && v <= 1024) o.group = v;
        }
        if (const char *e = std::getenv("B200HT_GEMM_ORDER")) o.order = e[0] == '1' ? 1 : 0;
        return o;
    }();
    const size_t ldc = ldc_arg ? ldc_arg : (LAYOUT == B200HT_OUT_MN ? (size_t)N : (size_t)M);
    const long sms = sm_count();
    const long nt = (N + TC_BN - 1) / TC_BN;
    const long mt256 = (M + 255) / 256;
    const long tiles128 = (long)((M + 127) / 128) * nt, tiles256 = mt256 * nt;
    // With 256-row tiles the last, partial wave costs a whole tile time.  When the tiles of that wave form a rectangle
    // at the end of the tile order (blocks of the last group x the last blocks of the other dimension) and fit one
    // wave as 128-row tiles, they can be computed by a second launch with 128-row tiles: half the time for the tail.
    const long inner_cnt = ord.order == 0 ? mt256 : nt, outer_cnt = ord.order == 0 ? nt : mt256;
    const long rem = tiles256 % sms;
    const long gl = inner_cnt % ord.group ? inner_cnt % ord.group : (inner_cnt < ord.group ? inner_cnt : ord.group);
    const bool can_split = allow_split && tiles256 > sms && rem > 0 && 2 * rem <= sms && (rem <= gl || rem % gl == 0) &&
                           rem < gl * outer_cnt;
    const double cost128 = 1.03 * (double)((tiles128 + sms - 1) / sms);
    const double cost256 = can_split ? 2.0 * (double)(tiles256 / sms) + 1.03 : 2.0 * (double)((tiles256 + sms - 1) / sms);
    const bool big = force_mt ? force_mt == 2 : (tiles256 >= sms && cost256 <= cost128);
    if (!big) return launch_tc_mt<OUT_DT, LAYOUT, 1>(Y, W, C, M, N, K, ldc, 0, 0, ord, row_scale, tok_scale, st);
    if (can_split && !force_mt) {
        const long in_blocks = rem <= gl ? rem : gl;          // blocks of the rectangle along the grouped dimension
        const long out_blocks = rem <= gl ? 1 : rem / gl;     // ... and along the other one
        const long rows = ord.order == 0 ? in_blocks : out_blocks;   // 256-row blocks
        const long cols = ord.order == 0 ? out_blocks : in_blocks;   // token blocks
        const long row_off = (mt256 - rows) * 256, tok_off = (nt - cols) * TC_BN;
        int rc = launch_tc_mt<OUT_DT, LAYOUT, 2>(Y, W, C, M, N, K, ldc, (int)rem, 1, ord, row_scale, tok_scale, st);
        if (rc) return rc;
        const size_t esz = OUT_DT == B200HT_F32 ? 4 : 2;
        const size_t coff = LAYOUT == B200HT_OUT_MN ? (size_t)row_off * ldc + (size_t)tok_off : (size_t)tok_off * ldc + (size_t)row_off;
        return launch_tc_mt<OUT_DT, LAYOUT, 1>((const unsigned char *)Y + (size_t)tok_off * K * 2,
                                               (const unsigned char *)W + (size_t)row_off * K * 2,
                                               (unsigned char *)C + coff * esz, (int)(M - row_off), (int)(N - tok_off), K, ldc,
                                               0, 2, ord, row_scale ? row_scale + row_off : nullptr,
                                               tok_scale ? tok_scale + tok_off : nullptr, st);
    }
    return launch_tc_mt<OUT_DT, LAYOUT, 2>(Y, W, C, M, N, K, ldc, 0, 0, ord, row_scale, tok_scale, st);
}

// `ldc` = leading dimension of C in elements when C is a block of a larger matrix (0: the block is the matrix).
int launch_gemm_bf16_tcgen05(const void *Y, const void *W, void *C, int M, int N, int K, int out_dtype,
                             int out_layout, cudaStream_t st, const float *row_scale, const float *tok_scale, size_t ldc)
{
    if (K < TC_BK) {
        dim3 blk(32, 8), grd((N + 31) / 32, (M + 7) / 8);
        note_launch();
        gemm_bf16_smallk_kernel<<<grd, blk, 0, st>>>((const __nv_bfloat16 *)Y, (const __nv_bfloat16 *)W, C, M, N, K,
                                                     out_dtype, out_layout, row_scale, tok_scale);
        return (int)cudaGetLastError();
    }
    if (out_dtype == B200HT_F32) {
        return out_layout == B200HT_OUT_MN
                   ? launch_tc<B200HT_F32, B200HT_OUT_MN>(Y, W, C, M, N, K, ldc, row_scale, tok_scale, st)
                   : launch_tc<B200HT_F32, B200HT_OUT_NM>(Y, W, C, M, N, K, ldc, row_scale, tok_scale, st);
    }
    return out_layout == B200HT_OUT_MN
               ? launch_tc<B200HT_BF16, B200HT_OUT_MN>(Y, W, C, M, N, K, ldc, row_scale, tok_scale, st)
               : launch_tc<B200HT_BF16, B200HT_OUT_NM>(Y, W, C, M, N, K, ldc, row_scale, tok_scale, st);
}

}  // namespace b200ht
