// SwiGLU gating: out = gate * sigmoid(gate) * up, float32 arithmetic.
// Reference: native/kernels/swiglu_f32.cu:5-15 and the scalar CPU twin
// src/DotLLM.Cpu/Kernels/FusedOps.cs:69-78 (sigmoid = 1 / (1 + exp(-g))).
#include "common.cuh"

template <typename T>
__global__ void __launch_bounds__(256)
swiglu_kernel(const T* __restrict__ gate, const T* __restrict__ up, int in_stride, T* __restrict__ out,
              int rows, int width) {
    const size_t n = (size_t)rows * width;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / width, c = i - r * width;
        const float g = dl_to_f32<T>(gate[r * in_stride + c]);
        const float u = dl_to_f32<T>(up[r * in_stride + c]);
        out[i] = dl_from_f32<T>(g * (1.0f / (1.0f + expf(-g))) * u);
    }
}

// gate, up: [rows, width] views with a common row stride; out: contiguous [rows, width].
extern "C" int dl_swiglu(const void* gate, const void* up, int in_stride, void* out, int dtype, int rows,
                         int width, void* stream) {
    DL_REQUIRE(rows >= 0 && width > 0 && in_stride >= width, "swiglu: bad sizes");
    if (rows == 0) return DL_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t n = (size_t)rows * width;
    const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    if (dtype == DL_F32)
        swiglu_kernel<float><<<blocks, 256, 0, s>>>((const float*)gate, (const float*)up, in_stride, (float*)out,
                                                    rows, width);
    else if (dtype == DL_BF16)
        swiglu_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>((const __nv_bfloat16*)gate, (const __nv_bfloat16*)up,
                                                            in_stride, (__nv_bfloat16*)out, rows, width);
    else
        return dl_fail(DL_ERR_UNSUPPORTED, "swiglu: dtype %d", dtype);
    DL_CHECK_LAUNCH("swiglu");
    return DL_OK;
}
