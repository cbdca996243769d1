// Version, error text, device check and the device status word.
#include <atomic>
#include <mutex>

#include "tc_common.cuh"

namespace b200ht {

__device__ int g_status_word = 0;

static std::atomic<unsigned long long> g_launches{0};
void note_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

// Per-device facts resolved once (mutex-guarded), then read without a lock: architecture check, SM count and the
// device address of the status word.  Every launcher needs them on every call, and each costs a runtime query.
struct DeviceFacts {
    std::atomic<int> state{0};   // 0 unknown, 1 sm_100, 2 other architecture
    int sms = 148;
    int *status = nullptr;
};
static DeviceFacts g_dev[64];
static std::mutex g_dev_mu;

static int device_facts(const DeviceFacts **out)
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return B200HT_ERR_DEVICE;
    DeviceFacts &f = g_dev[dev];
    if (f.state.load(std::memory_order_acquire) == 0) {
        std::lock_guard<std::mutex> lk(g_dev_mu);
        if (f.state.load(std::memory_order_relaxed) == 0) {
            int major = 0, sms = 148;
            e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
            if (e != cudaSuccess) return (int)e;
            if (major == 10) {
                e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
                if (e != cudaSuccess) return (int)e;
                int *p = nullptr;
                e = cudaGetSymbolAddress((void **)&p, g_status_word);
                if (e != cudaSuccess) return (int)e;
                f.sms = sms;
                f.status = p;
            }
            f.state.store(major == 10 ? 1 : 2, std::memory_order_release);
        }
    }
    *out = &f;
    return 0;
}

int *status_word_ptr()
{
    const DeviceFacts *f = nullptr;
    if (device_facts(&f) != 0 || f->state.load(std::memory_order_relaxed) != 1) return nullptr;
    return f->status;
}

int sm_count()
{
    const DeviceFacts *f = nullptr;
    if (device_facts(&f) != 0) return 148;
    return f->sms;
}

int check_device()
{
    const DeviceFacts *f = nullptr;
    const int rc = device_facts(&f);
    if (rc) return rc;
    return f->state.load(std::memory_order_relaxed) == 1 ? 0 : B200HT_ERR_DEVICE;
}

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per (device, kernel) and size: repeated calls with a size
// that is already granted return at once.
int ensure_dyn_smem(const void *func, int bytes)
{
    struct Entry { const void *func; int dev; int bytes; };
    static std::mutex mu;
    static Entry table[256];
    static int used = 0;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    std::lock_guard<std::mutex> lk(mu);
    Entry *slot = nullptr;
    for (int i = 0; i < used; ++i)
        if (table[i].func == func && table[i].dev == dev) { slot = &table[i]; break; }
    if (slot && slot->bytes >= bytes) return 0;
    e = cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return (int)e;
    if (!slot && used < 256) slot = &table[used++];
    if (slot) { slot->func = func; slot->dev = dev; slot->bytes = bytes; }
    return 0;
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
