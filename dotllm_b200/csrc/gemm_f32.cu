// y = x W^T in true float32: FFMA only, no tensor cores, no reduced-precision mode.
//
// The reference's 32-bit model runs its projections as per-row dot products
// (src/DotLLM.Cpu/Kernels/MatMul.cs:1121-1134, GemmF32 over GemvF32 :55-64).  This kernel is
// the same contraction tiled through shared memory.  Each output element is accumulated over k
// in ascending order by one thread, so its value does not depend on how many rows x has or on
// which rows share the launch: the 32-bit path gives the same bits however the tokens are cut
// into steps.
#include "common.cuh"

#define GF_BM 64
#define GF_BN 64
#define GF_BK 16

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ x, int x_stride, const float* __restrict__ w,
                float* __restrict__ y, int y_stride, int M, int N, int K) {
    __shared__ float xs[GF_BK][GF_BM + 4];
    __shared__ float ws[GF_BK][GF_BN + 4];
    const int tid = threadIdx.x;
    const int ty = tid / 16, tx = tid % 16;
    const int m0 = blockIdx.y * GF_BM, n0 = blockIdx.x * GF_BN;
    const int lrow = tid / 4, lk = (tid % 4) * 4;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += GF_BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int k = k0 + lk + i;
            const int xr = m0 + lrow, wr = n0 + lrow;
            xs[lk + i][lrow] = (xr < M && k < K) ? x[(size_t)xr * x_stride + k] : 0.f;
            ws[lk + i][lrow] = (wr < N && k < K) ? w[(size_t)wr * K + k] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GF_BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = m0 + ty * 4 + i;
        if (r >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = n0 + tx * 4 + j;
            if (c < N) y[(size_t)r * y_stride + c] = acc[i][j];
        }
    }
}

// x: [M, K] rows x_stride apart; w: contiguous [N, K]; y: [M, N] rows y_stride apart.
extern "C" int dl_gemm_f32(const float* x, int x_stride, const float* w, float* y, int y_stride, int M, int N,
                           int K, void* stream) {
    DL_REQUIRE(M >= 0 && N > 0 && K > 0 && x_stride >= K && y_stride >= N, "gemm_f32: bad sizes M=%d N=%d K=%d",
               M, N, K);
    if (M == 0) return DL_OK;
    dim3 grid((N + GF_BN - 1) / GF_BN, (M + GF_BM - 1) / GF_BM);
    DL_REQUIRE(grid.y <= 65535, "gemm_f32: too many rows (%d)", M);
    gemm_f32_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(x, x_stride, w, y, y_stride, M, N, K);
    DL_CHECK_LAUNCH("gemm_f32");
    return DL_OK;
}
