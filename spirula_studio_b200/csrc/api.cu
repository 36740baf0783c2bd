// Error reporting, version string and launch accounting of libssb_b200.
#include "ssb_common.cuh"

#include <atomic>
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

}  // namespace ssb

extern "C" {

const char* ssb_last_error_string(void) { return ssb::g_error; }

const char* ssb_version_string(void) { return "ssb_b200 0.1 sm_100a"; }

int64_t ssb_launch_count(void) { return ssb::g_launches.load(std::memory_order_relaxed); }

}  // extern "C"
