// Error text, launch counter and version string shared by all kernel entry points.
#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "common.cuh"

namespace rb200 {

static thread_local char g_error[512] = "";
static std::atomic<uint64_t> g_launches{0};

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

int check_cuda(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return RB200_OK;
    set_error("%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
    return RB200_E_CUDA;
}

// One status word per device that loads the library, written by kernels that were launched without a status
// pointer of their own.
__device__ int g_status_word = 0;

int* default_status_word() {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return static_cast<int*>(p);
}

int read_default_status_word() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_status_word, sizeof(int)) != cudaSuccess) return -1;
    if (v && cudaMemcpyToSymbol(g_status_word, &zero, sizeof(int)) != cudaSuccess) return -1;
    return v ? 1 : 0;
}

}  // namespace rb200

extern "C" int rb200k_device_status(void) { return rb200::read_default_status_word(); }
extern "C" const char* rb200k_last_error(void) { return rb200::g_error; }
extern "C" uint64_t rb200k_launch_count(void) { return rb200::g_launches.load(std::memory_order_relaxed); }
#ifdef RB200_DEBUG_BOUNDS
extern "C" const char* rb200k_version(void) { return "rocal_b200 0.1 sm_100a+bounds"; }
#else
extern "C" const char* rb200k_version(void) { return "rocal_b200 0.1 sm_100a"; }
#endif
