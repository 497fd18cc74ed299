// y = x W^T for a handful of rows of x (decode steps): a weight-streaming product.
//
// With M <= 64 rows every projection is bound by the bytes of W, read once.  The reference runs
// these through cuBLAS or one-block-per-output-row GEMV kernels
// (src/DotLLM.Cuda/CudaTransformerModel.cs:317-349, native/kernels/quantized_gemv.cu:13-63).
// Here W is the 16-row operand of mma.sync.m16n8k16 and the tokens are its 8 columns, so the
// tensor cores do the arithmetic while every lane streams 16-byte pieces of W rows straight
// from global memory into registers: within a 32-wide slice of k, lane (g, t) holds k = 8t..8t+7
// of rows g and g+8, and the same slice of token g's activations, which is a consistent
// permutation of k for both operands of two MMAs.  Nothing is staged in shared memory.
//
// A block of 4 warps owns one 16-row tile and a contiguous range of k; its warps take
// 32-wide slices in turn and their partial sums are added in a fixed order.  When a tile's k is
// split over several blocks, each writes its partial to scratch and the last one to arrive adds
// them, again in a fixed order, so the result is deterministic and the same for any number of
// rows of x.  With FUSE_SWIGLU the tile's rows 0-7 are gate rows and rows 8-15 the matching up
// rows, and the epilogue writes silu(gate) * up (native/kernels/swiglu.cu:7-41).
#include "common.cuh"

#define GS_WARPS 4

__device__ __forceinline__ void gs_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 gs_load16(const __nv_bfloat16* p, bool ok) {
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (ok) v = __ldg(reinterpret_cast<const uint4*>(p));
    return v;
}

template <typename TOut> __device__ __forceinline__ void gs_store(TOut* p, float v);
template <> __device__ __forceinline__ void gs_store<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void gs_store<__nv_bfloat16>(__nv_bfloat16* p, float v) {
    *p = __float2bfloat16_rn(v);
}

template <int NT, typename TOut, bool FUSE_SWIGLU>
__global__ void __launch_bounds__(32 * GS_WARPS)
gemm_skinny_kernel(const __nv_bfloat16* __restrict__ x, int x_stride, const __nv_bfloat16* __restrict__ w,
                   TOut* __restrict__ out, int out_stride, int M, int N, int K, int up_offset,
                   int chunks_per_block, float* __restrict__ partials, int* __restrict__ counters) {
    __shared__ float red[GS_WARPS][NT * 4][32];
    __shared__ int is_last;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int tile = blockIdx.x, split = blockIdx.y, ksplit = gridDim.y;

    // rows of W behind fragment rows g and g+8
    int row_lo, row_hi;
    bool ok_lo, ok_hi;
    if (FUSE_SWIGLU) {
        row_lo = tile * 8 + g;                 // gate row i
        row_hi = up_offset + tile * 8 + g;     // up row i
        ok_lo = ok_hi = (tile * 8 + g) < N;
    } else {
        row_lo = tile * 16 + g;
        row_hi = row_lo + 8;
        ok_lo = row_lo < N;
        ok_hi = row_hi < N;
    }
    const __nv_bfloat16* w_lo = w + (size_t)row_lo * K;
    const __nv_bfloat16* w_hi = w + (size_t)row_hi * K;

    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;

    const int n_chunks = (K + 31) / 32;
    const int c_begin = split * chunks_per_block;
    const int c_end = min(n_chunks, c_begin + chunks_per_block);
#pragma unroll 4
    for (int c = c_begin + warp; c < c_end; c += GS_WARPS) {
        const int k = c * 32 + t * 8;
        const bool k_ok = k < K;               // K is a multiple of 8
        const uint4 a_lo = gs_load16(w_lo + k, ok_lo && k_ok);
        const uint4 a_hi = gs_load16(w_hi + k, ok_hi && k_ok);
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            const int tok = j * 8 + g;
            const uint4 b = gs_load16(x + (size_t)tok * x_stride + k, tok < M && k_ok);
            gs_mma(acc[j], a_lo.x, a_hi.x, a_lo.y, a_hi.y, b.x, b.y);
            gs_mma(acc[j], a_lo.z, a_hi.z, a_lo.w, a_hi.w, b.z, b.w);
        }
    }

    // add the block's warps in a fixed order
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) red[warp][j * 4 + e][lane] = acc[j][e];
    __syncthreads();
    if (warp != 0) {
        // warps 1.. only help when the tile is split over blocks (they wait at the barrier below)
    } else {
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float s = red[0][j * 4 + e][lane];
#pragma unroll
                for (int ww = 1; ww < GS_WARPS; ++ww) s += red[ww][j * 4 + e][lane];
                acc[j][e] = s;
            }
    }

    if (ksplit > 1) {
        float* mine = partials + ((size_t)tile * ksplit + split) * (NT * 4 * 32);
        if (warp == 0) {
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) mine[(j * 4 + e) * 32 + lane] = acc[j][e];
            __threadfence();
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            const int seen = atomicAdd(&counters[tile], 1);
            is_last = (seen == ksplit - 1);
            if (is_last) counters[tile] = 0;        // ready for the next launch
        }
        __syncthreads();
        if (!is_last || warp != 0) return;
        __threadfence();
        const float* all = partials + (size_t)tile * ksplit * (NT * 4 * 32);
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float s = 0.f;
                for (int sp = 0; sp < ksplit; ++sp) s += __ldcg(all + (size_t)sp * (NT * 4 * 32) + (j * 4 + e) * 32 + lane);
                acc[j][e] = s;
            }
    } else if (warp != 0) {
        return;
    }

    // epilogue: acc[j] = {(row g, tok 2t), (row g, tok 2t+1), (row g+8, tok 2t), (row g+8, tok 2t+1)}
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const int tok0 = j * 8 + 2 * t;
        if (FUSE_SWIGLU) {
            const int col = tile * 8 + g;
            if (col < N) {
                const float g0 = acc[j][0], g1 = acc[j][1];
                if (tok0 < M) gs_store<TOut>(out + (size_t)tok0 * out_stride + col, g0 * (1.0f / (1.0f + expf(-g0))) * acc[j][2]);
                if (tok0 + 1 < M) gs_store<TOut>(out + (size_t)(tok0 + 1) * out_stride + col, g1 * (1.0f / (1.0f + expf(-g1))) * acc[j][3]);
            }
        } else {
            if (ok_lo) {
                if (tok0 < M) gs_store<TOut>(out + (size_t)tok0 * out_stride + row_lo, acc[j][0]);
                if (tok0 + 1 < M) gs_store<TOut>(out + (size_t)(tok0 + 1) * out_stride + row_lo, acc[j][1]);
            }
            if (ok_hi) {
                if (tok0 < M) gs_store<TOut>(out + (size_t)tok0 * out_stride + row_hi, acc[j][2]);
                if (tok0 + 1 < M) gs_store<TOut>(out + (size_t)(tok0 + 1) * out_stride + row_hi, acc[j][3]);
            }
        }
    }
}

template <int NT, typename TOut, bool FUSE>
static void gs_launch(dim3 grid, cudaStream_t s, const __nv_bfloat16* x, int x_stride, const __nv_bfloat16* w,
                      void* out, int out_stride, int M, int N, int K, int up_offset, int cpb, float* partials,
                      int* counters) {
    gemm_skinny_kernel<NT, TOut, FUSE><<<grid, 32 * GS_WARPS, 0, s>>>(x, x_stride, w, (TOut*)out, out_stride, M, N,
                                                                     K, up_offset, cpb, partials, counters);
}

// Number of k-splits this kernel uses for (tiles, K) on a device with `sms` multiprocessors.
// It depends on the weight's shape only, never on the number of rows of x.
extern "C" int dl_gemm_skinny_splits(int tiles, int K, int sms) {
    const int n_chunks = (K + 31) / 32;
    const int target = sms * 8;                              // blocks wanted in flight
    int ksplit = (target + tiles - 1) / tiles;
    const int max_split = n_chunks / (GS_WARPS * 4) > 1 ? n_chunks / (GS_WARPS * 4) : 1;
    if (ksplit > max_split) ksplit = max_split;
    if (ksplit < 1) ksplit = 1;
    if (ksplit > 16) ksplit = 16;
    return ksplit;
}

// x: bf16 [M, K] rows x_stride apart, M <= 64.  w: bf16, contiguous rows of K.
// fuse_swiglu == 0: w is [N, K], out [M, N].  fuse_swiglu == 1: w is [2N, K] (N gate rows, then N
// up rows), out [M, N] = silu(x Wg^T) * (x Wu^T).
// partials: float32 scratch of at least tiles * ksplit * nt * 128 floats when ksplit > 1
// (nt = number of 8-token groups rounded up to 1, 2, 4 or 8); counters: int32, zero, >= tiles.
extern "C" int dl_gemm_skinny_bf16(const void* x, int x_stride, const void* w, void* out, int out_dtype,
                                   int out_stride, int M, int N, int K, int fuse_swiglu, int ksplit,
                                   float* partials, int* counters, void* stream) {
    DL_REQUIRE(M >= 1 && M <= 64, "gemm_skinny: takes 1 to 64 rows, got %d", M);
    DL_REQUIRE(N > 0 && K > 0 && K % 8 == 0, "gemm_skinny: K=%d must be a positive multiple of 8", K);
    DL_REQUIRE(x_stride % 8 == 0 && x_stride >= K, "gemm_skinny: row stride of x (%d) must be a multiple of 8", x_stride);
    DL_REQUIRE(((uintptr_t)x % 16) == 0 && ((uintptr_t)w % 16) == 0, "gemm_skinny: x and W must be 16-byte aligned");
    DL_REQUIRE(out_stride >= N, "gemm_skinny: out stride shorter than N");
    DL_REQUIRE(out_dtype == DL_F32 || out_dtype == DL_BF16, "gemm_skinny: out dtype %d", out_dtype);
    const int tiles = fuse_swiglu ? (N + 7) / 8 : (N + 15) / 16;
    DL_REQUIRE(ksplit >= 1 && ksplit <= 16, "gemm_skinny: ksplit %d", ksplit);
    DL_REQUIRE(ksplit == 1 || (partials && counters), "gemm_skinny: split k needs scratch");
    const int n_chunks = (K + 31) / 32;
    const int cpb = (n_chunks + ksplit - 1) / ksplit;
    dim3 grid(tiles, ksplit);
    cudaStream_t s = (cudaStream_t)stream;
    const __nv_bfloat16* xb = (const __nv_bfloat16*)x;
    const __nv_bfloat16* wb = (const __nv_bfloat16*)w;
    const int nt = M <= 8 ? 1 : M <= 16 ? 2 : M <= 32 ? 4 : 8;
#define GS_CASE(NTV)                                                                                                \
    if (nt == NTV) {                                                                                                \
        if (fuse_swiglu) {                                                                                          \
            if (out_dtype == DL_F32) gs_launch<NTV, float, true>(grid, s, xb, x_stride, wb, out, out_stride, M, N, K, N, cpb, partials, counters); \
            else gs_launch<NTV, __nv_bfloat16, true>(grid, s, xb, x_stride, wb, out, out_stride, M, N, K, N, cpb, partials, counters);             \
        } else {                                                                                                    \
            if (out_dtype == DL_F32) gs_launch<NTV, float, false>(grid, s, xb, x_stride, wb, out, out_stride, M, N, K, 0, cpb, partials, counters); \
            else gs_launch<NTV, __nv_bfloat16, false>(grid, s, xb, x_stride, wb, out, out_stride, M, N, K, 0, cpb, partials, counters);             \
        }                                                                                                           \
    }
    GS_CASE(1) GS_CASE(2) GS_CASE(4) GS_CASE(8)
#undef GS_CASE
    DL_CHECK_LAUNCH("gemm_skinny");
    return DL_OK;
}

// ---------------------------------------------------------------------------------------------
// The same product for callers that must not allocate (declared in gemm_skinny_static.h).
//
// dl_gemm_skinny_bf16 above takes its split-k scratch from the caller, who normally gets it from
// an allocator.  Some callers have no allocator to ask: code that runs between a framework's
// allocation phases, a host process whose device memory is handed out once at start-up and then
// frozen, a real-time loop that may not take the allocator's lock.  For them the scratch lives in
// this library's own image: a file-scope __device__ array of a fixed, modest size that every GPU
// loading the library holds until the process exits.
//
// The array's name is only a host-side handle for the device object; its device address is asked
// for once per device, with that device current, through cudaGetSymbolAddress.
#include "gemm_skinny_static.h"
#include <mutex>

#define GS_STATIC_PARTIAL_FLOATS (DL_GEMM_SKINNY_STATIC_SCRATCH_BYTES / 4 - DL_GEMM_SKINNY_STATIC_MAX_TILES)

struct GsStaticScratch {
    int counters[DL_GEMM_SKINNY_STATIC_MAX_TILES];
    float partials[GS_STATIC_PARTIAL_FLOATS];
};
static __device__ __align__(256) GsStaticScratch gs_static_scratch;

#define GS_MAX_DEVICES 64
static GsStaticScratch* gs_static_ptr[GS_MAX_DEVICES];      // device address of the array, per device
static std::mutex gs_static_mutex;

// The device address of the scratch on the current device (looked up on the first call there).
static int gs_static_address(GsStaticScratch** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "gemm_skinny_static: cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= GS_MAX_DEVICES) return dl_fail(DL_ERR_UNSUPPORTED, "gemm_skinny_static: device %d out of range", dev);
    std::lock_guard<std::mutex> lock(gs_static_mutex);
    if (gs_static_ptr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, gs_static_scratch);
        if (e != cudaSuccess || p == nullptr)
            return dl_fail(DL_ERR_LAUNCH, "gemm_skinny_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        gs_static_ptr[dev] = static_cast<GsStaticScratch*>(p);
    }
    *out = gs_static_ptr[dev];
    return DL_OK;
}

extern "C" int dl_gemm_skinny_bf16_static(const void* x, int x_stride, const void* w, void* out, int out_dtype,
                                          int out_stride, int M, int N, int K, int fuse_swiglu, void* stream) {
    DL_REQUIRE(M >= 1 && M <= 64 && N > 0 && K > 0, "gemm_skinny_static: bad sizes M=%d N=%d K=%d", M, N, K);
    int sms = 0, dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        return dl_fail(DL_ERR_LAUNCH, "gemm_skinny_static: cannot query the device");
    const int tiles = fuse_swiglu ? (N + 7) / 8 : (N + 15) / 16;
    const int ksplit = dl_gemm_skinny_splits(tiles, K, sms);
    const int nt = M <= 8 ? 1 : M <= 16 ? 2 : M <= 32 ? 4 : 8;
    const size_t need = ksplit > 1 ? (size_t)tiles * ksplit * nt * 128 : 0;
    if (tiles > DL_GEMM_SKINNY_STATIC_MAX_TILES || need > (size_t)GS_STATIC_PARTIAL_FLOATS)
        return dl_fail(DL_ERR_UNSUPPORTED,
                       "gemm_skinny_static: M=%d N=%d K=%d needs %d row tiles and %zu scratch floats; the built-in "
                       "scratch holds %d tiles and %d floats - use dl_gemm_skinny_bf16 with your own scratch",
                       M, N, K, tiles, need, DL_GEMM_SKINNY_STATIC_MAX_TILES, (int)GS_STATIC_PARTIAL_FLOATS);
    GsStaticScratch* scratch = nullptr;
    const int rc = gs_static_address(&scratch);
    if (rc != DL_OK) return rc;
    if (ksplit > 1) {
        // The array keeps whatever the last call left; the arrival counters must start at zero.
        cudaError_t e = cudaMemsetAsync(scratch->counters, 0, sizeof(int) * tiles, (cudaStream_t)stream);
        if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "gemm_skinny_static: memset: %s", cudaGetErrorString(e));
    }
    return dl_gemm_skinny_bf16(x, x_stride, w, out, out_dtype, out_stride, M, N, K, fuse_swiglu, ksplit,
                               scratch->partials, scratch->counters, stream);
}
