// Error record and device queries shared by the kernels' entry points.
#include "common.cuh"
#include <stdarg.h>

static thread_local char g_error[512] = "";

char* dl_error_buffer() { return g_error; }

int dl_fail(int status, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return status;
}

extern "C" const char* dl_last_error() { return g_error; }

// Compute capability of the current device as major*10+minor, or a negative CUDA error.
extern "C" int dl_device_arch() {
    int dev = 0, major = 0, minor = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev);
    if (e != cudaSuccess) {
        dl_fail(DL_ERR_LAUNCH, "device query: %s", cudaGetErrorString(e));
        return -(int)e;
    }
    return major * 10 + minor;
}

extern "C" int dl_sm_count() {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return -1;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
    return n;
}
