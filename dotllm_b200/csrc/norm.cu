// RMSNorm over the float32 residual stream, with the residual add fused in.
//
//   y = x * (1 / sqrt(mean(x^2) + eps)) * gain          (eps inside the root)
//
// Same statistics as the reference's rmsnorm_f32 / fused_add_rmsnorm_f16
// (native/kernels/rmsnorm_f32.cu:3-36, native/kernels/fused_add_rmsnorm.cu:9-72): the sum
// of squares, the root and the add are float32; only the normalised output may be
// bfloat16.  One block per row, a fixed block size, so a row's rounding does not depend
// on the rest of the batch.
#include "common.cuh"

#define NORM_THREADS 256

template <typename TDelta, typename TOut, bool ADD>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_kernel(float* __restrict__ residual, const TDelta* __restrict__ delta,
               const float* __restrict__ gain, TOut* __restrict__ out, int width, float eps) {
    __shared__ float scratch[33];
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
    if (delta)
        rmsnorm_kernel<TDelta, TOut, true><<<rows, NORM_THREADS, 0, s>>>(residual, (const TDelta*)delta, gain,
                                                                          (TOut*)out, width, eps);
    else
        rmsnorm_kernel<TDelta, TOut, false><<<rows, NORM_THREADS, 0, s>>>(residual, nullptr, gain, (TOut*)out,
                                                                           width, eps);
    DL_CHECK_LAUNCH("rmsnorm");
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
