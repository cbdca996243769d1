/*
 * b200ht — C ABI of the B200 (sm_100a) Walsh-Hadamard library.
 *
 * Plain pointers and sizes only; every pointer is a DEVICE pointer owned by the
 * caller unless stated otherwise.  No function allocates or frees device
 * memory, none synchronises the host with the device: work is enqueued on the
 * `stream` argument (a cudaStream_t passed as void*; NULL = default stream).
 *
 * Return value of every launcher: 0 on success, a negative B200HT_ERR_* code
 * for a rejected argument (nothing was launched), or a positive cudaError_t
 * reported by the runtime at launch.  b200ht_error_string() turns any of them
 * into text.  Nothing throws, nothing calls exit().
 *
 * "Reference" below is Alan-Chen99/6s894_project_2025; paths are relative to it.
 */
#ifndef B200HT_H
#define B200HT_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types */
#define B200HT_F16  0
#define B200HT_BF16 1
#define B200HT_F32  2

/* layouts of the fused-GEMM result */
#define B200HT_OUT_MN 0 /* C[m*N+n], M x N row-major: the reference layout     */
#define B200HT_OUT_NM 1 /* C[n*M+m], token-major: one contiguous row per token */

/* argument errors (negative) */
#define B200HT_ERR_NULL       (-1) /* a required pointer is NULL                     */
#define B200HT_ERR_SIZE       (-2) /* size not a power of two / out of range          */
#define B200HT_ERR_DTYPE      (-3) /* unsupported element type combination            */
#define B200HT_ERR_ALIGN      (-4) /* pointer not 16-byte aligned                     */
#define B200HT_ERR_WORKSPACE  (-5) /* workspace missing or too small                  */
#define B200HT_ERR_OVERLAP    (-6) /* in/out partially overlap                        */
#define B200HT_ERR_DEVICE     (-7) /* current device is not compute capability 10.x   */
#define B200HT_ERR_TIMEOUT    (-8) /* a bounded device-side wait expired (see status) */
#define B200HT_ERR_STATIC_SCRATCH (-9) /* problem exceeds B200HT_STATIC_SCRATCH_BYTES       */

/* Library version (major*10000 + minor*100 + patch). */
int b200ht_version(void);

/* Text for a return code of any function below. Never NULL. */
const char *b200ht_error_string(int code);

/*
 * Standalone transform: out[r, :] = scale * in[r, :] . H_n for r < rows, H_n the
 * Sylvester-ordered Hadamard matrix of size n (a power of two, 2 <= n <= 32768).
 * Arithmetic in fp32, one rounding to `dtype` on store.  `dtype` is B200HT_F16
 * or B200HT_BF16 (B200HT_F32 is also accepted: exact fp32 butterflies).
 * in == out (exactly) is allowed; partial overlap is not.  Both pointers must be
 * 16-byte aligned.  rows may be any value >= 0 (0 is a no-op).
 *
 * Replaces  template<DType> void run_fht(void* a, void* out, uint32_t numel,
 *           uint32_t had_size, cudaStream_t stream)   (csrc/main.cuh:5-6,
 * csrc/main.cu:79-122), which the reference's op calls with scale 1/sqrt(n)
 * baked in (csrc/hada.cuh:49-57) and which accepts only n = 2^8..2^15 and row
 * counts divisible by its rows-per-block (csrc/main.cu:64,108).
 */
int b200ht_fwht(const void *in, void *out, uint64_t rows, uint32_t n, int dtype,
                float scale, void *stream);

/*
 * Randomised Hadamard transform: out[r, :] = scale * (in[r, :] * d) . H_n with a +-1
 * diagonal d in front of the transform.  `signs` holds n 16-bit words, 0x8000
 * where d is -1 and 0 where it is +1 (16-byte aligned device memory); the kernel
 * flips the sign bits of the loaded elements, so the option costs one cached
 * 16-byte load per vector.  dtype F16 | BF16.  Everything else as b200ht_fwht.
 * No counterpart in the reference, whose callers would multiply by d in a
 * separate pass before csrc.hadamard_transform (bench/bench.py:79-81).
 */
int b200ht_fwht_signed(const void *in, void *out, uint64_t rows, uint32_t n, int dtype,
                       float scale, const void *signs, void *stream);

/*
 * Fused C = W . H(X):  C[m, t] = sum_k W[m, k] * (scale * H_K x_t)[k].
 *   X  N x K, token-major (X[t*K + k])           in_dtype  F32 | BF16
 *   W  M x K, row-major   (W[m*K + k])           in_dtype  (same as X)
 *   C  M x N (B200HT_OUT_MN) or N x M (B200HT_OUT_NM), out_dtype F32 | BF16
 * K must be a power of two, 2 <= K <= 32768.  BF16 inputs go through the bf16
 * tensor cores with fp32 accumulation.  F32 inputs are multiplied in fp32
 * (FFMA) by default; given a workspace of
 * b200ht_fused_gemm_tc_workspace_bytes(M, N, K, in_dtype) bytes they are split
 * into three bf16 terms each and contracted on the tensor cores (six bf16
 * products per fp32 product, fp32 accumulation; K <= 4096, measured relative
 * error 1e-6 .. 4.4e-6 against 0.6e-6 .. 1.2e-6 for FFMA, about four times
 * its speed on large shapes).
 * `workspace` must hold at least
 * b200ht_fused_gemm_workspace_bytes(M, N, K, in_dtype) bytes, 256-byte
 * aligned; it carries the transformed tokens between the two phases of the
 * operation.  Argument order X, W, C as in
 *   __global__ void fused_ht_gemm_pipelined(const float* X, const float* W,
 *   float* C)   (fused_ht/fusion_pipelined.cu:306-310; dims are compile-time
 * constants there, :51-53, and the transform is unscaled: pass scale = 1.0f to
 * reproduce it).
 */
size_t b200ht_fused_gemm_workspace_bytes(int M, int N, int K, int in_dtype);
/* Workspace size that selects the tensor-core contraction for F32 inputs (equal to the
 * size above for BF16 and for shapes too small to gain from it).  No counterpart in the
 * reference, whose fused kernel is fp32 SIMT throughout (fused_ht/fusion_pipelined.cu:306-563). */
size_t b200ht_fused_gemm_tc_workspace_bytes(int M, int N, int K, int in_dtype);
int b200ht_fused_gemm(const void *X, const void *W, void *C, int M, int N, int K,
                      int in_dtype, int out_dtype, int out_layout, float scale,
                      void *workspace, size_t workspace_bytes, void *stream);

/* b200ht_fused_gemm with the +-1 diagonal of b200ht_fwht_signed applied to the
 * tokens before the transform: C = W . H(d * X).  BF16 inputs only. */
int b200ht_fused_gemm_signed(const void *X, const void *W, void *C, int M, int N, int K,
                             int in_dtype, int out_dtype, int out_layout, float scale,
                             const void *signs, void *workspace, size_t workspace_bytes,
                             void *stream);

/* b200ht_fused_gemm with epilogue scales, the cast step of a quantised linear layer:
 *   C[m, t] = row_scale[m] * tok_scale[t] * sum_k W[m, k] * (scale * H_K (d * x_t))[k]
 * row_scale (M floats, per output channel), tok_scale (N floats, per token) and signs (as in
 * b200ht_fused_gemm_signed, BF16 only) may each be NULL.  The factors are applied to the fp32
 * accumulator before the single rounding of the store.  No counterpart in the reference. */
int b200ht_fused_gemm_scaled(const void *X, const void *W, void *C, int M, int N, int K,
                             int in_dtype, int out_dtype, int out_layout, float scale,
                             const void *signs, const float *row_scale, const float *tok_scale,
                             void *workspace, size_t workspace_bytes, void *stream);

/*
 * b200ht_fused_gemm without a caller-provided workspace and without any
 * allocation.  No counterpart in the reference (its program allocates all its
 * buffers with cudaMalloc in main()).
 *
 * For callers that cannot allocate device memory where they call from: a
 * process whose own memory pool reserved the whole GPU at start-up, a plugin
 * whose execute hook must not allocate, a latency-critical loop that must
 * never take the driver's allocation lock.  The transformed tokens live in a
 * fixed B200HT_STATIC_SCRATCH_BYTES array inside the library image (each GPU
 * that loads the library holds that much memory until the process exits).
 *
 * Limits and rules:
 *  - N*K*sizeof(input element), rounded up to 256, must not exceed
 *    B200HT_STATIC_SCRATCH_BYTES (e.g. 2048 tokens at K=8192 bf16); larger
 *    problems return B200HT_ERR_STATIC_SCRATCH and launch nothing.  Split the
 *    tokens into several calls, or use b200ht_fused_gemm.
 *  - The function calls no cudaMalloc/cudaFree and no allocating library
 *    routine.  Its first call on a device resolves the device address of the
 *    array (cudaGetSymbolAddress) and caches it; make that first call during
 *    set-up, before any stream capture is started.  The CUDA driver itself may
 *    still load kernel code, and reserve memory for it, the first time a kernel
 *    variant runs (each combination of in_dtype, out_dtype, out_layout and tile
 *    shape is its own kernel): make one set-up call per combination that will
 *    be used later, or run the process with CUDA_MODULE_LOADING=EAGER.
 *  - All calls on one device share the array, and it keeps the previous call's
 *    contents (nothing needs clearing: each call overwrites what it reads).
 *    Two calls whose kernels may run at the same time on one GPU (different
 *    streams, different threads) race on it: serialise them.
 * Other arguments, layouts and return codes: as b200ht_fused_gemm.
 */
#define B200HT_STATIC_SCRATCH_BYTES (32u << 20)
int b200ht_fused_gemm_static(const void *X, const void *W, void *C, int M, int N, int K,
                             int in_dtype, int out_dtype, int out_layout, float scale,
                             void *stream);

/*
 * Small-batch fused Y = W . H(X):  Y[m*B + b] = sum_k W[m*N + k] * (scale * H_N x_b)[k]
 *   W  M x N row-major, X  N x B with b fastest (X[i*B + b]), Y  M x B, b fastest.
 * N must be a power of two, 2 <= N <= 32768 (>= 32 for BF16); 1 <= B <= 65536
 * (the reference's own benchmark calls it with B up to 2048,
 * fused_ht/fwht_gemv_fusion.cu:643-653).
 * in_dtype F32 | BF16 (W and X alike), out_dtype F32 | BF16.  For BF16 with
 * 256 <= N <= 8192 the transformed X stays in shared memory and W is streamed
 * from HBM once per group of up to b200ht_fused_gemv_max_batch(N, B200HT_BF16)
 * columns (32 for N <= 1024, 24 at N = 2048, 16 at N = 4096, 8 at N = 8192); other shapes use
 * smaller column groups.  The entry is built for small B: beyond that batch
 * b200ht_fused_gemm (tokens = columns of X) reads W once and is the faster call.
 * Argument order W, X, Y, M, N, B as in
 *   __global__ void fused_hadamard_gemv_kernel(const float* W, const float* X,
 *   float* Y, int M, int N, int B)   (fused_ht/fwht_gemv_fusion.cu:98-105; the
 * float4 variant :176-183 has the same signature).  The reference is unscaled:
 * pass scale = 1.0f to reproduce it.
 */
int b200ht_fused_gemv(const void *W, const void *X, void *Y, int M, int N, int B,
                      int in_dtype, int out_dtype, float scale, void *stream);

/*
 * Largest batch B for which b200ht_fused_gemv streams W exactly once (the transformed X of all columns fits in shared
 * memory beside the ring of W tiles); 0 when the shape takes a path without that property.  A caller with more
 * columns should use b200ht_fused_gemm.  No counterpart in the reference, which streams W once per column at any B
 * (fused_ht/fwht_gemv_fusion.cu:98-159).
 */
int b200ht_fused_gemv_max_batch(int N, int in_dtype);

/*
 * Row-sharded small-batch GEMV across the GPUs of one node (one process per GPU).  Every rank keeps M rows of W (its
 * shard: rows row_begin .. row_begin + M - 1 of the rows_total rows of the full matrix) and the same X; after the call
 * every rank holds all rows of Y = W . H(X).  The exchange is part of the kernel: it writes its own rows into Y_full
 * and sends each value, as one 8-byte store (value, number of the call), into a slot array on every other rank
 * through peer-mapped pointers; then its CTAs collect the other ranks' rows from this GPU's slot array, waiting for
 * each slot's tag, and write them into Y_full.  No collective, no fence and no flag on the path: a value costs one
 * trip over the link.  No counterpart in the reference, which is single-GPU.
 *   Y_full        this rank's full result, rows_total x B values of out_dtype
 *   peer_slots[p] the slot array in peer p's memory (n_peers <= 7 pointers valid on this GPU, e.g. from
 *                 b200ht_ipc_open), rows_total x B slots of 8 bytes, zero-initialised once
 *   my_slots      this GPU's slot array, of the same size (the peers write it)
 *   local_count   two zero-initialised 32-bit words in this GPU's memory, 8-byte aligned (the kernel updates them as
 *                 one 64-bit word): [0] scratch, left at zero; [1] calls made so far, counted by the kernel
 *   target        number of this call on this exchange, 1, 2, 3, ...: all ranks call in lockstep.  0 = take it from
 *                 local_count[1]: no argument then changes from call to call, so a CUDA graph can replay the call
 *                 (use one way of counting per exchange, not both)
 * A rank waits at most one second for the other ranks' values; if one never arrives the status word
 * (b200ht_device_status) reports B200HT_ERR_TIMEOUT and nothing hangs.  A rank must not start call k + 2 before its
 * consumers of call k's result are enqueued, and slots are reused every second call: alternate between two result
 * buffers and two slot arrays (the Python wrapper does).
 * BF16 inputs, 256 <= N <= 8192, B <= b200ht_fused_gemv_max_batch(N, B200HT_BF16), rows_total * B < 2^31; other
 * shapes return B200HT_ERR_SIZE (gather the shards with a collective instead).
 */
int b200ht_fused_gemv_peers(const void *W, const void *X, void *Y_full, int M, int N, int B, int in_dtype,
                            int out_dtype, float scale, int row_begin, int rows_total, int n_peers,
                            void *const *peer_slots, const void *my_slots, unsigned int *local_count,
                            unsigned int target, void *stream);

/*
 * Inter-process mapping of device buffers for b200ht_fused_gemv_peers: b200ht_ipc_export writes a 64-byte handle for
 * the cudaMalloc allocation that contains `ptr` and the offset of `ptr` inside it; b200ht_ipc_open maps a handle
 * received from another process (peer access is enabled on demand) and returns the mapped base address;
 * b200ht_ipc_close unmaps it.  Set-up calls, not for the hot path.  No counterpart in the reference.
 */
int b200ht_ipc_export(const void *ptr, void *handle64, unsigned long long *offset);
int b200ht_ipc_open(const void *handle64, void **base);
int b200ht_ipc_close(void *base);

/*
 * Number of kernels this library has launched in the calling process so far (all entry points, all streams).
 * A benchmark reads it before and after a timed region to report its launch count.  No counterpart in the reference.
 */
unsigned long long b200ht_launch_count(void);

/*
 * Device-side status word of the calling thread's current device: 0, or the
 * B200HT_ERR_TIMEOUT code left by a kernel whose bounded wait on an mbarrier
 * expired.  Synchronises the device.  `clear` != 0 resets it.  The reference has
 * no counterpart (its kernels have no waits that can expire).
 */
int b200ht_device_status(int clear);

/*
 * Self-test of the time-limited waits used by the tcgen05 / TMA kernels: runs a
 * one-thread kernel that waits, for at most `limit_us` microseconds (1 ..
 * 1 000 000), on a barrier that is never completed.  Returns B200HT_ERR_TIMEOUT
 * when the wait gave up as designed (the device status word then holds the same
 * code; clear it with b200ht_device_status(1)), 0 if it did not, or a CUDA
 * error.  Synchronises the stream.  No counterpart in the reference.
 */
int b200ht_selftest_wait_timeout(unsigned int limit_us, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* B200HT_H */
