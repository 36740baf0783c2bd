// Error reporting, version string and launch accounting of libssb_b200.
#include "ssb_common.cuh"

#include <atomic>
#include <mutex>
#include <stdarg.h>
#include <string.h>

namespace ssb {

static thread_local char g_error[512] = "";
static std::atomic<int64_t> g_launches{0};

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int check_cuda(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return SSB_OK;
    set_error("CUDA error %d (%s) at %s", (int)e, cudaGetErrorString(e), what);
    return e == cudaErrorMemoryAllocation ? SSB_ERR_OUT_OF_MEMORY : SSB_ERR_CUDA;
}

// The opt-in to more than 48 KB of dynamic shared memory is a per-device attribute of a kernel:
// remembered per (kernel, device), under a lock, so any thread may launch on any device.
int ensure_dynamic_smem(const void* kernel, int bytes) {
    constexpr int kMaxKernels = 32;
    static std::mutex mu;
    static const void* known[kMaxKernels];
    static uint64_t devices_done[kMaxKernels];          // bit d: done on device d (no heap: a fixed table)
    int dev = 0;
    int e = check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
    if (e != SSB_OK) return e;
    std::lock_guard<std::mutex> lock(mu);
    int slot = 0;
    while (slot < kMaxKernels && known[slot] && known[slot] != kernel) ++slot;
    const bool tracked = slot < kMaxKernels && dev >= 0 && dev < kMaxDevices;
    if (tracked && known[slot] == kernel && (devices_done[slot] >> dev & 1)) return SSB_OK;
    e = check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes), "cudaFuncSetAttribute");
    if (e == SSB_OK && tracked) { known[slot] = kernel; devices_done[slot] |= (uint64_t)1 << dev; }
    return e;
}

// One sticky status word per device, set by kernels that met something they had to refuse
// (a list index outside its buffer, more pairs than the caller's buffers hold) instead of
// touching memory they were not given.
__device__ unsigned int g_device_status;

static std::mutex g_status_mutex;
static unsigned int* g_status_addr[kMaxDevices];

unsigned int* device_status_word() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    std::lock_guard<std::mutex> lock(g_status_mutex);
    if (!g_status_addr[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess) { cudaGetLastError(); return nullptr; }
        g_status_addr[dev] = (unsigned int*)p;
    }
    return g_status_addr[dev];
}

}  // namespace ssb

extern "C" {

int ssb_device_status(int32_t* h_bits, void* stream) {
    using namespace ssb;
    unsigned int* word = device_status_word();
    SSB_REQUIRE(word != nullptr, "ssb_device_status: no current CUDA device");
    unsigned int bits = 0;
    cudaStream_t st = (cudaStream_t)stream;
    SSB_CUDA(cudaMemcpyAsync(&bits, word, sizeof(bits), cudaMemcpyDeviceToHost, st));
    SSB_CUDA(cudaMemsetAsync(word, 0, sizeof(bits), st));
    SSB_CUDA(cudaStreamSynchronize(st));
    if (h_bits) *h_bits = (int32_t)bits;
    if (bits & SSB_STATUS_BAD_INDEX) {
        set_error("a kernel met a list entry or record index outside its buffer and skipped it (status bits 0x%x)", bits);
        return SSB_ERR_INVALID_ARGUMENT;
    }
    if (bits & SSB_STATUS_PAIRS_DROPPED) {
        set_error("more (splat, tile) pairs than the caller's buffers hold: the pairs beyond the capacity were dropped (status bits 0x%x)", bits);
        return SSB_ERR_CAPACITY;
    }
    return SSB_OK;
}

const char* ssb_last_error_string(void) { return ssb::g_error; }

const char* ssb_version_string(void) { return "ssb_b200 0.1 sm_100a"; }

int64_t ssb_launch_count(void) { return ssb::g_launches.load(std::memory_order_relaxed); }

}  // extern "C"
