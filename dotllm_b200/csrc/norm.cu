// RMSNorm over the float32 residual stream, with the residual add fused in.
//
//   y = x * (1 / sqrt(mean(x^2) + eps)) * gain          (eps inside the root)
//
// Same statistics as the reference's rmsnorm_f32 / fused_add_rmsnorm_f16
// (native/kernels/rmsnorm_f32.cu:3-36, native/kernels/fused_add_rmsnorm.cu:9-72): the sum
// of squares, the root and the add are float32; only the normalised output may be
// bfloat16.  One block per row, a fixed block size, so a row's rounding does not depend
// on the rest of the batch.
//
// Rows of up to 8192 values whose width is a multiple of 4 take the register path: every
// thread loads its float4 pieces at once (a decode step has a handful of rows, so the
// kernel's time is one round of memory latency, not a loop of them), keeps them in
// registers across the reduction, and reads nothing twice.  Other widths take the looped path.
#include "common.cuh"

#define NORM_THREADS 256
#define NORM_MAX_VEC 8            // float4 pieces per thread on the register path

template <typename T> struct Vec4;
template <> struct Vec4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<__nv_bfloat16> {
    static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
        return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<uint32_t*>(&a);
        raw.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = raw;
    }
};

template <typename TDelta, typename TOut, bool ADD>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_vec_kernel(float* __restrict__ residual, const TDelta* __restrict__ delta,
                   const float* __restrict__ gain, TOut* __restrict__ out, int width, float eps) {
    __shared__ float scratch[33];
    dl_launch_dependents();
    dl_grid_dependency_wait();
    const size_t base = (size_t)blockIdx.x * width;
    const int n_vec = width / 4;
    float4 v[NORM_MAX_VEC];
#pragma unroll
    for (int i = 0; i < NORM_MAX_VEC; ++i) {
        const int c = threadIdx.x + i * NORM_THREADS;
        v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < n_vec) v[i] = Vec4<float>::load(residual + base + 4 * c);
    }
    if (ADD) {
#pragma unroll
        for (int i = 0; i < NORM_MAX_VEC; ++i) {
            const int c = threadIdx.x + i * NORM_THREADS;
            if (c < n_vec) {
                const float4 d = Vec4<TDelta>::load(delta + base + 4 * c);
                v[i].x += d.x; v[i].y += d.y; v[i].z += d.z; v[i].w += d.w;
                Vec4<float>::store(residual + base + 4 * c, v[i]);
            }
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NORM_MAX_VEC; ++i) ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    ss = dl_block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)width + eps);
#pragma unroll
    for (int i = 0; i < NORM_MAX_VEC; ++i) {
        const int c = threadIdx.x + i * NORM_THREADS;
        if (c < n_vec) {
            const float4 gn = Vec4<float>::load(gain + 4 * c);
            Vec4<TOut>::store(out + base + 4 * c, make_float4(v[i].x * scale * gn.x, v[i].y * scale * gn.y,
                                                              v[i].z * scale * gn.z, v[i].w * scale * gn.w));
        }
    }
}

template <typename TDelta, typename TOut, bool ADD>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_kernel(float* __restrict__ residual, const TDelta* __restrict__ delta,
               const float* __restrict__ gain, TOut* __restrict__ out, int width, float eps) {
    __shared__ float scratch[33];
    dl_launch_dependents();
    dl_grid_dependency_wait();
    const size_t base = (size_t)blockIdx.x * width;
    float ss = 0.f;
    for (int c = threadIdx.x; c < width; c += NORM_THREADS) {
        float v = residual[base + c];
        if (ADD) {
            v += dl_to_f32<TDelta>(delta[base + c]);
            residual[base + c] = v;
        }
        ss += v * v;
    }
    ss = dl_block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)width + eps);
    for (int c = threadIdx.x; c < width; c += NORM_THREADS)
        out[base + c] = dl_from_f32<TOut>(residual[base + c] * scale * gain[c]);
}

template <typename TDelta, typename TOut>
static int launch_norm(float* residual, const void* delta, const float* gain, void* out, int rows, int width,
                       float eps, cudaStream_t s) {
    const bool aligned = ((uintptr_t)residual % 16 == 0) && ((uintptr_t)gain % 16 == 0) && ((uintptr_t)out % 16 == 0) &&
                         (!delta || (uintptr_t)delta % 16 == 0);
    const bool vec = aligned && width % 4 == 0 && width <= 4 * NORM_THREADS * NORM_MAX_VEC;
    const TDelta* d = (const TDelta*)delta;
    TOut* o = (TOut*)out;
    cudaError_t e;
    const dim3 grid(rows), block(NORM_THREADS);
    const TDelta* none = nullptr;
    if (vec) {
        if (delta) e = dl_launch_dependent(rmsnorm_vec_kernel<TDelta, TOut, true>, grid, block, 0, s, residual, d, gain, o, width, eps);
        else e = dl_launch_dependent(rmsnorm_vec_kernel<TDelta, TOut, false>, grid, block, 0, s, residual, none, gain, o, width, eps);
    } else {
        if (delta) e = dl_launch_dependent(rmsnorm_kernel<TDelta, TOut, true>, grid, block, 0, s, residual, d, gain, o, width, eps);
        else e = dl_launch_dependent(rmsnorm_kernel<TDelta, TOut, false>, grid, block, 0, s, residual, none, gain, o, width, eps);
    }
    if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "rmsnorm: %s", cudaGetErrorString(e));
    return DL_OK;
}

// residual: float32 [rows, width], updated in place to residual + delta when delta != NULL.
// delta: [rows, width] of delta_dtype or NULL.  out: [rows, width] of out_dtype.
extern "C" int dl_add_rmsnorm(float* residual, const void* delta, int delta_dtype, const float* gain, void* out,
                              int out_dtype, int rows, int width, float eps, void* stream) {
    DL_REQUIRE(rows >= 0 && width > 0, "rmsnorm: bad sizes rows=%d width=%d", rows, width);
    DL_REQUIRE(eps > 0.f, "rmsnorm: eps must be positive");
    if (rows == 0) return DL_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const bool df = (delta_dtype == DL_F32), of = (out_dtype == DL_F32);
    DL_REQUIRE(df || delta_dtype == DL_BF16, "rmsnorm: delta dtype %d", delta_dtype);
    DL_REQUIRE(of || out_dtype == DL_BF16, "rmsnorm: out dtype %d", out_dtype);
    if (df && of) return launch_norm<float, float>(residual, delta, gain, out, rows, width, eps, s);
    if (df && !of) return launch_norm<float, __nv_bfloat16>(residual, delta, gain, out, rows, width, eps, s);
    if (!df && of) return launch_norm<__nv_bfloat16, float>(residual, delta, gain, out, rows, width, eps, s);
    return launch_norm<__nv_bfloat16, __nv_bfloat16>(residual, delta, gain, out, rows, width, eps, s);
}
