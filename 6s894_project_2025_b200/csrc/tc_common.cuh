// Blackwell (sm_100a) plumbing shared by the tcgen05 kernels: mbarriers with
// bounded waits, TMA tile loads, TMEM allocation, UMMA descriptors.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace b200ht {

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ uint64_t global_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
    return t;
}

// Wait for `parity` of the barrier with a time limit (about two seconds) and an
// early exit when another role of the CTA has already given up.  Returns false
// on give-up; the caller then leaves its loop, the CTA drains and exits, and the
// host finds B200HT_ERR_TIMEOUT in the device status word.
constexpr uint64_t kWaitLimitNs = 2000000000ull;
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int *status,
                                          uint64_t limit_ns = kWaitLimitNs)
{
    if (mbar_test(bar, parity)) return true;
    const uint64_t t0 = global_ns();
    uint32_t spins = 0;
    while (true) {
        if (mbar_test(bar, parity)) return true;
        if ((++spins & 255u) == 0) {
            if (*abort_flag) return false;
            if (global_ns() - t0 > limit_ns) {
                *abort_flag = 1;
                if (status) atomicExch(status, B200HT_ERR_TIMEOUT);
                return false;
            }
        }
    }
}

__device__ __forceinline__ void fence_barrier_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async()
{
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }

// 2-D tiled TMA load into this CTA's shared memory (no multicast).
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(dst),
        "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, int x, int y, int z, uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n" ::"r"(dst),
        "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap *map)
{
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(map) : "memory");
}

// TMEM: one warp allocates / frees `cols` (power of two >= 32) columns.
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(dst_smem), "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(cols) : "memory");
}

// Shared-memory matrix descriptor, K-major operand, 128-byte swizzle: rows of
// 64 bf16 (128 B), 8-row groups 1024 B apart.  The tile base is 1024-B aligned;
// advancing K by 16 elements adds 32 B to the start address.
__device__ __forceinline__ uint64_t umma_desc_k_sw128(uint32_t saddr)
{
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);  // start address
    d |= (uint64_t)1 << 16;                     // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;           // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                     // descriptor version (Blackwell)
    d |= (uint64_t)2 << 61;                     // SWIZZLE_128B
    return d;
}

// Instruction descriptor: bf16 x bf16 -> fp32, both operands K-major.
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int M, int N)
{
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrive on an mbarrier of this CTA when all tcgen05.mma issued so far by this thread are done.
__device__ __forceinline__ void umma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar)
                 : "memory");
}

// 32 consecutive fp32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

// Host: encode a 2-D bf16 row-major tensor map (rows x cols, cols contiguous)
// with a box of box_rows x 64 columns and 128-byte swizzle.  Returns 0 or a
// CUresult (positive).
int encode_tmap_bf16_2d(CUtensorMap *map, const void *base, uint64_t rows, uint64_t cols, uint32_t box_rows);
// Same for fp16 or bf16 (dtype = B200HT_F16 | B200HT_BF16).
int encode_tmap_b16_2d(CUtensorMap *map, const void *base, uint64_t rows, uint64_t cols, uint32_t box_rows,
                       int dtype);
// Host: 3-D view [64 k][rows][cols/64] of the same matrix; box = box_rows x (64*box_chunks) elements.
int encode_tmap_bf16_rows_chunks(CUtensorMap *map, const void *base, uint64_t rows, uint64_t cols,
                                 uint32_t box_rows, uint32_t box_chunks);
// Host: 4-D view [64 k][group_rows][groups][cols/64] of the first groups*group_rows rows of the same matrix; box =
// {64, box_rows, 1, box_chunks} with box_rows >= group_rows: the surplus rows of a box lie outside the second
// dimension and are filled with zeros, so each 64-k tile in shared memory has box_rows rows.
int encode_tmap_bf16_row_groups(CUtensorMap *map, const void *base, uint64_t group_rows, uint64_t groups, uint64_t cols,
                                uint32_t box_rows, uint32_t box_chunks);

}  // namespace b200ht
