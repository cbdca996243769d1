// Version, error text, device check and the device status word.
#include <atomic>
#include <mutex>

#include "tc_common.cuh"

namespace b200ht {

__device__ int g_status_word = 0;

static std::atomic<unsigned long long> g_launches{0};
void note_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

int *status_word_ptr()
{
    int *p = nullptr;
    if (cudaGetSymbolAddress((void **)&p, g_status_word) != cudaSuccess) return nullptr;
    return p;
}

int check_device()
{
    static std::mutex mu;
    static int ok_mask[64] = {0};  // 0 unknown, 1 ok, 2 wrong architecture
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return B200HT_ERR_DEVICE;
    std::lock_guard<std::mutex> lk(mu);
    if (ok_mask[dev] == 0) {
        int major = 0;
        e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
        if (e != cudaSuccess) return (int)e;
        ok_mask[dev] = (major == 10) ? 1 : 2;
    }
    return ok_mask[dev] == 1 ? 0 : B200HT_ERR_DEVICE;
}

}  // namespace b200ht

extern "C" int b200ht_version(void) { return 100; }

extern "C" unsigned long long b200ht_launch_count(void)
{
    return b200ht::g_launches.load(std::memory_order_relaxed);
}

extern "C" const char *b200ht_error_string(int code)
{
    switch (code) {
    case 0: return "success";
    case B200HT_ERR_NULL: return "b200ht: a required pointer is NULL";
    case B200HT_ERR_SIZE: return "b200ht: size must be a power of two in the supported range";
    case B200HT_ERR_DTYPE: return "b200ht: unsupported element type";
    case B200HT_ERR_ALIGN: return "b200ht: pointer is not 16-byte aligned";
    case B200HT_ERR_WORKSPACE: return "b200ht: workspace missing or too small";
    case B200HT_ERR_OVERLAP: return "b200ht: input and output partially overlap";
    case B200HT_ERR_DEVICE: return "b200ht: current device is not an sm_100 (B200) GPU";
    case B200HT_ERR_TIMEOUT: return "b200ht: a bounded device-side wait expired";
    case B200HT_ERR_STATIC_SCRATCH:
        return "b200ht: problem too large for the built-in static scratch (B200HT_STATIC_SCRATCH_BYTES); "
               "split the tokens or pass a workspace to b200ht_fused_gemm";
    default: break;
    }
    if (code > 0) return cudaGetErrorString((cudaError_t)code);
    return "b200ht: unknown error code";
}

extern "C" int b200ht_device_status(int clear)
{
    int rc = b200ht::check_device();
    if (rc) return rc;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return (int)e;
    int v = 0;
    e = cudaMemcpyFromSymbol(&v, b200ht::g_status_word, sizeof(int));
    if (e != cudaSuccess) return (int)e;
    if (clear && v != 0) {
        const int zero = 0;
        e = cudaMemcpyToSymbol(b200ht::g_status_word, &zero, sizeof(int));
        if (e != cudaSuccess) return (int)e;
    }
    return v;
}

// ---------------------------------------------------------------------------
// Self-test of the bounded-wait mechanism that every mbarrier wait of the
// tcgen05 / TMA kernels goes through: one thread waits on a barrier that nobody
// will ever complete, with a caller-chosen limit.  The wait must give up, leave
// B200HT_ERR_TIMEOUT in the device status word and the kernel must return, so
// that the context stays usable.  Nothing faults, traps or hangs.
// ---------------------------------------------------------------------------
namespace b200ht {
__global__ void wait_timeout_probe_kernel(unsigned long long limit_ns, int *status, int *gave_up)
{
    __shared__ __align__(8) unsigned long long bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_flag = 0;
        fence_barrier_init();
        const bool ok = mbar_wait(smem_u32(&bar), 0u, &abort_flag, status, limit_ns);
        *gave_up = ok ? 0 : 1;
    }
}
}  // namespace b200ht

namespace b200ht {
__device__ int g_selftest_flag = 0;
}

extern "C" int b200ht_selftest_wait_timeout(unsigned int limit_us, void *stream)
{
    using namespace b200ht;
    int rc = check_device();
    if (rc) return rc;
    if (limit_us == 0 || limit_us > 1000000u) return B200HT_ERR_SIZE;   // at most one second
    int *flag = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void **)&flag, g_selftest_flag);
    if (e != cudaSuccess) return (int)e;
    cudaStream_t st = (cudaStream_t)stream;
    e = cudaMemsetAsync(flag, 0, sizeof(int), st);
    if (e != cudaSuccess) return (int)e;
    note_launch();
    wait_timeout_probe_kernel<<<1, 32, 0, st>>>((unsigned long long)limit_us * 1000ull, status_word_ptr(), flag);
    e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    int gave_up = 0;
    e = cudaMemcpyAsync(&gave_up, flag, sizeof(int), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return (int)e;
    return gave_up ? B200HT_ERR_TIMEOUT : 0;
}
