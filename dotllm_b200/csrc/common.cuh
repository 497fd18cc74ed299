// Shared helpers of the sm_100a kernels: status codes, dtype conversion, reductions,
// and the paged cache's addressing.
//
// Every exported function is `extern "C" int dl_*(..., void* stream)`: it checks its
// arguments on the host, launches on the given stream, and returns 0 or a status code
// whose text `dl_last_error()` gives.  Nothing here allocates device memory.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <math.h>

#define DL_PAGE 64            // tokens per cache page

enum DlStatus { DL_OK = 0, DL_ERR_ARGUMENT = 1, DL_ERR_LAUNCH = 2, DL_ERR_UNSUPPORTED = 3 };
enum DlDtype { DL_F32 = 0, DL_BF16 = 1 };

// Host-side record of the last failure of this thread (read through dl_last_error).
char* dl_error_buffer();
int dl_fail(int status, const char* fmt, ...);

#define DL_REQUIRE(cond, ...)                                         \
    do {                                                              \
        if (!(cond)) return dl_fail(DL_ERR_ARGUMENT, __VA_ARGS__);    \
    } while (0)

#define DL_CHECK_LAUNCH(name)                                                         \
    do {                                                                              \
        cudaError_t e__ = cudaGetLastError();                                         \
        if (e__ != cudaSuccess)                                                       \
            return dl_fail(DL_ERR_LAUNCH, "%s: %s", name, cudaGetErrorString(e__));   \
    } while (0)

// Programmatic dependent launch.  A kernel launched through dl_launch_dependent may begin while its
// predecessor on the stream is still running: its blocks start as soon as every block of the
// predecessor has called dl_launch_dependents() (or exited) and there is room on a multiprocessor.
// Such a kernel must call dl_grid_dependency_wait() before it reads anything an earlier kernel
// wrote and before it writes any global memory (an earlier kernel may still be reading it); what
// it does before the wait may touch only memory that no kernel of the stream writes (weights).
// dl_launch_dependents() is harmless in a kernel that nothing depends on.
bool dl_dependent_launch_enabled();          // false when DOTLLM_DEPENDENT_LAUNCH=0 is set

#ifdef __CUDACC__
__device__ __forceinline__ void dl_grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void dl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
static inline cudaError_t dl_launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                              cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = dl_dependent_launch_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

template <typename T> __device__ __forceinline__ float dl_to_f32(T v);
template <> __device__ __forceinline__ float dl_to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float dl_to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T dl_from_f32(float v);
template <> __device__ __forceinline__ float dl_from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 dl_from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float dl_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float dl_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  The order of
// additions is fixed by the block size alone, so a row's result does not depend on
// which other rows are in the launch.
__device__ __forceinline__ float dl_block_sum(float v, float* scratch /* >= 33 floats */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n_warps = (blockDim.x + 31) >> 5;
    v = dl_warp_sum(v);
    __syncthreads();                       // scratch may still be read from a previous call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float w = lane < n_warps ? scratch[lane] : 0.f;
        w = dl_warp_sum(w);
        if (lane == 0) scratch[32] = w;
    }
    __syncthreads();
    return scratch[32];
}

// Cache pools.  K page: [kv_head][token in page][head_dim].  V page is stored transposed,
// [kv_head][head_dim][token in page], so that a run of tokens of one dimension is contiguous.
__device__ __forceinline__ size_t dl_k_offset(int page, int n_kv, int kvh, int in_page, int hd) {
    return (((size_t)page * n_kv + kvh) * DL_PAGE + in_page) * hd;
}
__device__ __forceinline__ size_t dl_v_offset(int page, int n_kv, int kvh, int dim, int hd) {
    return (((size_t)page * n_kv + kvh) * hd + dim) * DL_PAGE;
}
