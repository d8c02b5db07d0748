// Error channel of the C interface, and a query of the device the library
// was built for.
#include <atomic>
#include "common.cuh"

#include <cstdlib>
#include <cstring>

namespace {
thread_local char g_error[1024] = "";
}

int li_fail(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return 1;
}

int li_check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) return 0;
    return li_fail("%s: launch failed: %s", what, cudaGetErrorString(e));
}

// Which of the caller's next launches may overlap (li_pdl_allow): a mask of kinds (LI_PDL_KIND) that may NOT.  The step
// function sets it per step.
static std::atomic<int> g_pdl_off{0};

LI_EXPORT void li_pdl_allow(int kinds_off) { g_pdl_off.store(kinds_off, std::memory_order_relaxed); }

bool li_pdl_enabled(int kind) {
    if (g_pdl_off.load(std::memory_order_relaxed) & kind) return false;
    static const bool on = [] {
        const char* v = getenv("LITINFER_B200_PDL");
        return !(v && v[0] == '0');
    }();
    static const int off_mask = [] {
        const char* v = getenv("LITINFER_B200_PDL_OFF");
        return v ? atoi(v) : 0;
    }();
    return on && !(off_mask & kind);
}

LI_EXPORT const char* li_last_error() { return g_error; }

// 0 if the current device can run this library (compute capability 10.x), else an error.
LI_EXPORT int li_check_device() {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return li_fail("no CUDA device: %s", cudaGetErrorString(e));
    cudaDeviceProp p;
    e = cudaGetDeviceProperties(&p, dev);
    if (e != cudaSuccess) return li_fail("cudaGetDeviceProperties: %s", cudaGetErrorString(e));
    if (p.major != 10) return li_fail("this library is built for sm_100a (B200); device %d is sm_%d%d", dev, p.major, p.minor);
    return 0;
}
