// Error text, version and device queries behind the C ABI.
#include <stdarg.h>
#include <string.h>

#include "common.cuh"

namespace sgnn {

static thread_local char g_err[512] = "";

void set_error(const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int sm_count()
{
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

}  // namespace sgnn

extern "C" SGNN_API int sgnn_version(void) { return 100; }

extern "C" SGNN_API const char *sgnn_last_error_string(void) { return sgnn::g_err; }
