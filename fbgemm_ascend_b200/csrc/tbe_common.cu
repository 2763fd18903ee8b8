// Error reporting and cached device properties for the tbe_b200 library.
#include <stdarg.h>
#include <stdio.h>

#include <atomic>

#include "tbe_common.cuh"

namespace tbe {

namespace {
thread_local char g_last_error[512] = "";
}

int fail(int code, const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
    return code;
}

int check_launch(const char* what)
{
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(TBE_B200_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
    return TBE_B200_OK;
}

int sm_count()
{
    constexpr int kMaxDev = 64;
    static std::atomic<int> cached[kMaxDev];   // zero-initialised; a lost race only repeats the query
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return 148;
    int n = cached[dev].load(std::memory_order_relaxed);
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

}  // namespace tbe

extern "C" const char* tbe_b200_last_error(void) { return tbe::g_last_error; }

extern "C" int tbe_b200_version(void) { return 100; }
