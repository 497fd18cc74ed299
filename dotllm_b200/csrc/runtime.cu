// Error record and device queries shared by the kernels' entry points.
#include "common.cuh"
#include <stdarg.h>
#include <stdlib.h>

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

static int g_dependent_launch = -1;          // -1: not decided yet

bool dl_dependent_launch_enabled() {
    if (g_dependent_launch < 0) {
        const char* v = getenv("DOTLLM_DEPENDENT_LAUNCH");
        g_dependent_launch = (v && v[0] == '0') ? 0 : 1;
    }
    return g_dependent_launch != 0;
}

// Switch programmatic dependent launch on or off for later launches (tests compare both).
extern "C" int dl_set_dependent_launch(int on) {
    g_dependent_launch = on ? 1 : 0;
    return DL_OK;
}

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
