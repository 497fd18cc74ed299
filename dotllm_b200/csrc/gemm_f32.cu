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

// The same product for many rows: tiles of 128 x 128, eight by eight outputs per thread, operands
// fetched sixteen bytes at a time and the next block of k on its way while this one is multiplied.
// Every output is still one thread's chain of fused multiply-adds over k in ascending order, so the
// bits are those of the kernel above (a row's result does not depend on which kernel its step met).
#define GL_BM 128
#define GL_BN 128
#define GL_BK 16

__global__ void __launch_bounds__(256)
gemm_f32_large_kernel(const float* __restrict__ x, int x_stride, const float* __restrict__ w,
                      float* __restrict__ y, int y_stride, int M, int N, int K) {
    __shared__ __align__(16) float xs[2][GL_BK][GL_BM + 4];
    __shared__ __align__(16) float ws[2][GL_BK][GL_BN + 4];
    const int tid = threadIdx.x;
    const int ty = tid / 16, tx = tid % 16;                  // outputs rows ty*8 .., columns tx*8 ..
    const int m0 = blockIdx.y * GL_BM, n0 = blockIdx.x * GL_BN;
    // loads: 128 rows x 16 k per operand = 512 pieces of four k; a thread takes two of each operand
    const int lrow = tid / 4, lk = (tid % 4) * 4;            // rows lrow and lrow + 64
    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

    float4 px[2], pw[2];
    auto fetch = [&](int k0) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int xr = m0 + lrow + 64 * h, wr = n0 + lrow + 64 * h, k = k0 + lk;
            px[h] = (xr < M && k < K) ? *reinterpret_cast<const float4*>(x + (size_t)xr * x_stride + k) : make_float4(0.f, 0.f, 0.f, 0.f);
            pw[h] = (wr < N && k < K) ? *reinterpret_cast<const float4*>(w + (size_t)wr * K + k) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    auto stash = [&](int b) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = lrow + 64 * h;
            xs[b][lk + 0][r] = px[h].x; xs[b][lk + 1][r] = px[h].y; xs[b][lk + 2][r] = px[h].z; xs[b][lk + 3][r] = px[h].w;
            ws[b][lk + 0][r] = pw[h].x; ws[b][lk + 1][r] = pw[h].y; ws[b][lk + 2][r] = pw[h].z; ws[b][lk + 3][r] = pw[h].w;
        }
    };
    fetch(0);
    stash(0);
    __syncthreads();
    int b = 0;
    for (int k0 = 0; k0 < K; k0 += GL_BK, b ^= 1) {
        const bool more = k0 + GL_BK < K;
        if (more) fetch(k0 + GL_BK);
#pragma unroll
        for (int kk = 0; kk < GL_BK; ++kk) {
            float a[8], c[8];
            const float4 a0 = *reinterpret_cast<const float4*>(&xs[b][kk][ty * 8]), a1 = *reinterpret_cast<const float4*>(&xs[b][kk][ty * 8 + 4]);
            const float4 c0 = *reinterpret_cast<const float4*>(&ws[b][kk][tx * 8]), c1 = *reinterpret_cast<const float4*>(&ws[b][kk][tx * 8 + 4]);
            a[0] = a0.x, a[1] = a0.y, a[2] = a0.z, a[3] = a0.w, a[4] = a1.x, a[5] = a1.y, a[6] = a1.z, a[7] = a1.w;
            c[0] = c0.x, c[1] = c0.y, c[2] = c0.z, c[3] = c0.w, c[4] = c1.x, c[5] = c1.y, c[6] = c1.z, c[7] = c1.w;
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], c[j], acc[i][j]);
        }
        if (more) stash(b ^ 1);
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int r = m0 + ty * 8 + i;
        if (r >= M) continue;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int c = n0 + tx * 8 + j;
            if (c < N) y[(size_t)r * y_stride + c] = acc[i][j];
        }
    }
}

// And for a decode step's few rows (up to 16): blocks of 16 rows x 16 outputs, one output per thread,
// so that a matrix of 4,096 rows is 256 blocks streaming 16 rows of W each (the 64 x 64 tiles above
// would be 64 blocks, most of whose rows of x are padding).  The same chain per output, the same bits.
#define GS32_BK 64

__global__ void __launch_bounds__(256)
gemm_f32_skinny_kernel(const float* __restrict__ x, int x_stride, const float* __restrict__ w,
                       float* __restrict__ y, int y_stride, int M, int N, int K) {
    __shared__ float xs[2][16][GS32_BK + 1];
    __shared__ float ws[2][16][GS32_BK + 1];
    const int tid = threadIdx.x;
    const int m = tid / 16, n = tid % 16;                     // this thread's output
    const int n0 = blockIdx.x * 16;
    const int lrow = tid / 16, lk = (tid % 16) * 4;           // this thread's piece of a tile: four k of one row
    float4 px, pw;
    auto fetch = [&](int k0) {
        const int k = k0 + lk, wr = n0 + lrow;
        px = (lrow < M && k < K) ? *reinterpret_cast<const float4*>(x + (size_t)lrow * x_stride + k) : make_float4(0.f, 0.f, 0.f, 0.f);
        pw = (wr < N && k < K) ? *reinterpret_cast<const float4*>(w + (size_t)wr * K + k) : make_float4(0.f, 0.f, 0.f, 0.f);
    };
    auto stash = [&](int b) {
        xs[b][lrow][lk] = px.x, xs[b][lrow][lk + 1] = px.y, xs[b][lrow][lk + 2] = px.z, xs[b][lrow][lk + 3] = px.w;
        ws[b][lrow][lk] = pw.x, ws[b][lrow][lk + 1] = pw.y, ws[b][lrow][lk + 2] = pw.z, ws[b][lrow][lk + 3] = pw.w;
    };
    float acc = 0.f;
    fetch(0);
    stash(0);
    __syncthreads();
    int b = 0;
    for (int k0 = 0; k0 < K; k0 += GS32_BK, b ^= 1) {
        const bool more = k0 + GS32_BK < K;
        if (more) fetch(k0 + GS32_BK);
#pragma unroll
        for (int kk = 0; kk < GS32_BK; ++kk) acc = fmaf(xs[b][m][kk], ws[b][n][kk], acc);
        if (more) stash(b ^ 1);
        __syncthreads();
    }
    if (m < M && n0 + n < N) y[(size_t)m * y_stride + n0 + n] = acc;
}

// x: [M, K] rows x_stride apart; w: contiguous [N, K]; y: [M, N] rows y_stride apart.
extern "C" int dl_gemm_f32(const float* x, int x_stride, const float* w, float* y, int y_stride, int M, int N,
                           int K, void* stream) {
    DL_REQUIRE(M >= 0 && N > 0 && K > 0 && x_stride >= K && y_stride >= N, "gemm_f32: bad sizes M=%d N=%d K=%d",
               M, N, K);
    if (M == 0) return DL_OK;
    const bool vec_ok = K % 4 == 0 && x_stride % 4 == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)w % 16) == 0;
    if (M <= 16 && vec_ok) {
        gemm_f32_skinny_kernel<<<(N + 15) / 16, 256, 0, (cudaStream_t)stream>>>(x, x_stride, w, y, y_stride, M, N, K);
        DL_CHECK_LAUNCH("gemm_f32");
        return DL_OK;
    }
    if (M >= 128 && K % 4 == 0 && x_stride % 4 == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)w % 16) == 0) {
        dim3 lgrid((N + GL_BN - 1) / GL_BN, (M + GL_BM - 1) / GL_BM);
        DL_REQUIRE(lgrid.y <= 65535, "gemm_f32: too many rows (%d)", M);
        gemm_f32_large_kernel<<<lgrid, 256, 0, (cudaStream_t)stream>>>(x, x_stride, w, y, y_stride, M, N, K);
        DL_CHECK_LAUNCH("gemm_f32");
        return DL_OK;
    }
    dim3 grid((N + GF_BN - 1) / GF_BN, (M + GF_BM - 1) / GF_BM);
    DL_REQUIRE(grid.y <= 65535, "gemm_f32: too many rows (%d)", M);
    gemm_f32_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(x, x_stride, w, y, y_stride, M, N, K);
    DL_CHECK_LAUNCH("gemm_f32");
    return DL_OK;
}
