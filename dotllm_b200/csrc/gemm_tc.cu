// y = x W^T for many rows of x (prefill): a tcgen05 product with the accumulators in tensor memory.
//
// The reference runs its prefill projections through cuBLAS and gates the feed-forward with a
// separate kernel (src/DotLLM.Cuda/CudaGemm.cs:29-40, native/kernels/swiglu.cu:7-41).  This kernel
// is for the products where fusing pays: with W = [gate; up] the epilogue writes silu(gate) * up, so
// the [T, 2I] intermediate never goes to memory.  It also takes the plain product, and the Q/K/V
// product of a prompt with the position encoding and the cache write in its epilogue: W = [Wq; Wk; Wv],
// the query columns come out rotated, the key columns are rotated and go straight to their cache
// pages, the value columns to theirs (transposed), so that no kernel has to read the product back to
// do it (native/kernels/rope.cu and the cache write are kernels of their own in the reference).
//
// Shape: persistent, one block per multiprocessor, six warps with fixed roles.
//   warp 0   one thread issues the tensor-map copies (TMA, 128-byte swizzle) of x and W tiles into a
//            ring of four stages (x 128 x 64, W 256 x 64 bfloat16 = 48 KB a stage);
//   warp 1   one thread issues tcgen05.mma (M 128, N 256, K 16; four per stage) into one of two
//            accumulators of 256 columns in tensor memory, and commits each stage back to the ring;
//   warps 2-5  the epilogue: each warp reads its 32 lanes (rows) of the finished accumulator with
//            tcgen05.ld, converts (or gates) and stores, while the MMA warp fills the other one.
// A tile is 128 rows of x by 256 rows of W (gated: 128 gate rows and the 128 matching up rows, 128
// output columns).  Tiles are taken in row-of-x-fastest order, so that the blocks running at one
// time share a panel of W in the L2.  Parts of a tile outside the matrices are read as zeros by the
// copy engine and never stored.
//
// Every wait on an mbarrier is bounded (about a second of clock cycles); on expiry the kernel
// records a code in `status`, stops issuing work, waits (bounded) for copies in flight, frees its
// tensor memory and returns.
#include "common.cuh"
#include "tma.cuh"
#include "tcgen05.cuh"
#include <mutex>
#include <type_traits>
#include <unordered_map>

#define GT_BM 128
#define GT_BN 256
#define GT_BK 64
#define GT_STAGES 4
#define GT_THREADS 192
#define GT_A_BYTES (GT_BM * GT_BK * 2)
#define GT_B_BYTES (GT_BN * GT_BK * 2)
#define GT_STAGE_BYTES (GT_A_BYTES + GT_B_BYTES)
#define GT_TMEM_COLS 512

__device__ __forceinline__ uint32_t gt_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Store 32 consecutive outputs of one row, columns col0 .. col0+31, those below n_cols only.
template <typename TOut>
__device__ __forceinline__ void gt_store32(TOut* row_ptr, int col0, int n_cols, const float (&v)[32], bool vec_ok);
template <>
__device__ __forceinline__ void gt_store32<__nv_bfloat16>(__nv_bfloat16* row_ptr, int col0, int n_cols, const float (&v)[32],
                                                          bool vec_ok) {
    if (vec_ok && col0 + 32 <= n_cols) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint4 p;
            p.x = gt_pack(v[8 * i], v[8 * i + 1]);
            p.y = gt_pack(v[8 * i + 2], v[8 * i + 3]);
            p.z = gt_pack(v[8 * i + 4], v[8 * i + 5]);
            p.w = gt_pack(v[8 * i + 6], v[8 * i + 7]);
            *reinterpret_cast<uint4*>(row_ptr + col0 + 8 * i) = p;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (col0 + i < n_cols) row_ptr[col0 + i] = __float2bfloat16_rn(v[i]);
    }
}
template <>
__device__ __forceinline__ void gt_store32<float>(float* row_ptr, int col0, int n_cols, const float (&v)[32], bool vec_ok) {
    if (vec_ok && col0 + 32 <= n_cols) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
            *reinterpret_cast<float4*>(row_ptr + col0 + 4 * i) = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (col0 + i < n_cols) row_ptr[col0 + i] = v[i];
    }
}

enum { GT_PLAIN = 0, GT_GATED = 1, GT_QKV = 2 };

// What the Q/K/V epilogue needs: the columns' split, the rotary tables, where every token (row of x)
// stands in its sequence, and the cache.  Tiles of 256 columns never straddle two of the three ranges
// (the host checks that q_cols and kv_cols are multiples of 256), nor a head (head_dim 64 or 128).
struct GtQkv {
    int q_cols, kv_cols, hd, nkv;
    const float* cos_t;              // [table_rows, hd/2]
    const float* sin_t;
    int table_rows;
    const int32_t* token_pos;        // [M] position of the row's token in its sequence
    const int32_t* token_seq;        // [M] its sequence's row in the block table
    const int32_t* block_table;      // [sequences, bt_stride] page ids
    int bt_stride;
    __nv_bfloat16* k_pool;
    __nv_bfloat16* v_pool;
    int n_pages;
};

// The same roundings as the rope kernels (no contraction), so that the fused and the separate way
// give the same bits.
__device__ __forceinline__ float gt_rot_lo(float x0, float x1, float c, float s) { return __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s)); }
__device__ __forceinline__ float gt_rot_hi(float x0, float x1, float c, float s) { return __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c)); }

// 32 consecutive bfloat16 values to a 16-byte aligned place.
__device__ __forceinline__ void gt_store32_bf16(__nv_bfloat16* dst, const float (&v)[32]) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
        *reinterpret_cast<uint4*>(dst + 8 * i) = make_uint4(gt_pack(v[8 * i], v[8 * i + 1]), gt_pack(v[8 * i + 2], v[8 * i + 3]),
                                                            gt_pack(v[8 * i + 4], v[8 * i + 5]), gt_pack(v[8 * i + 6], v[8 * i + 7]));
}

// The Q/K/V epilogue of one 128 x 256 tile for this thread's row.  `taddr`: the thread's lane of the
// accumulator.  Every lane of the warp runs the tensor-memory loads; stores are for live rows only.
__device__ __forceinline__ void gt_qkv_epilogue(uint32_t taddr, int col_base, int row, bool row_ok, __nv_bfloat16* __restrict__ out,
                                                int out_stride, const GtQkv& qkv) {
    const int hd = qkv.hd, half = hd / 2;
    const int region = col_base < qkv.q_cols ? 0 : (col_base < qkv.q_cols + qkv.kv_cols ? 1 : 2);
    int pos = -1, in_page = 0;
    long long page = -1;
    if (row_ok) {
        pos = qkv.token_pos[row];
        if (pos < 0 || pos >= qkv.table_rows) pos = -1;       // host-validated; never index outside
        if (pos >= 0 && region != 0) {
            page = qkv.block_table[(size_t)qkv.token_seq[row] * qkv.bt_stride + pos / DL_PAGE];
            if (page < 0 || page >= qkv.n_pages) page = -1;
            in_page = pos % DL_PAGE;
        }
    }
    if (region == 2) {
        // values: no rotation; the cache holds them transposed, [dim][token in page] - the lanes of a
        // warp are consecutive tokens, so each store instruction writes a run of one dimension's row
        const int kv0 = (col_base - qkv.q_cols - qkv.kv_cols) / hd;
#pragma unroll 1
        for (int c0 = 0; c0 < GT_BN; c0 += 32) {
            float v[32];
            tc_tmem_load32(taddr + (uint32_t)c0, v);
            if (page >= 0) {
                const int kvh = kv0 + c0 / hd, d0 = c0 % hd;
                __nv_bfloat16* dst = qkv.v_pool + dl_v_offset((int)page, qkv.nkv, kvh, d0, hd) + in_page;
#pragma unroll
                for (int i = 0; i < 32; ++i) dst[(size_t)i * DL_PAGE] = __float2bfloat16_rn(v[i]);
            }
        }
        return;
    }
    // queries and keys: dims c .. c+31 of the low half of a head pair with the same dims of the high half
#pragma unroll 1
    for (int h0 = 0; h0 < GT_BN; h0 += hd) {
#pragma unroll 1
        for (int c = 0; c < half; c += 32) {
            float lo[32], hi[32];
            tc_tmem_load32(taddr + (uint32_t)(h0 + c), lo);
            tc_tmem_load32(taddr + (uint32_t)(h0 + half + c), hi);
            // no lane leaves the loop early: the loads above are the whole warp's
            const float* cs = qkv.cos_t + (size_t)(pos < 0 ? 0 : pos) * half + c;
            const float* sn = qkv.sin_t + (size_t)(pos < 0 ? 0 : pos) * half + c;
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
                const float4 c4 = *reinterpret_cast<const float4*>(cs + i), s4 = *reinterpret_cast<const float4*>(sn + i);
                const float cc[4] = {c4.x, c4.y, c4.z, c4.w}, ss[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    // the product is rounded to bfloat16 before it is rotated, as the separate kernels see it
                    const float x0 = __bfloat162float(__float2bfloat16_rn(lo[i + e])), x1 = __bfloat162float(__float2bfloat16_rn(hi[i + e]));
                    lo[i + e] = gt_rot_lo(x0, x1, cc[e], ss[e]);
                    hi[i + e] = gt_rot_hi(x0, x1, cc[e], ss[e]);
                }
            }
            __nv_bfloat16* dst = nullptr;
            if (region == 0) {
                if (pos >= 0) dst = out + (size_t)row * out_stride + col_base + h0;
            } else if (page >= 0) {
                dst = qkv.k_pool + dl_k_offset((int)page, qkv.nkv, (col_base - qkv.q_cols + h0) / hd, in_page, hd);
            }
            if (dst != nullptr) {
                gt_store32_bf16(dst + c, lo);
                gt_store32_bf16(dst + half + c, hi);
            }
        }
    }
}

// MODE GT_GATED: W is [2N, K], gate rows then up rows; a tile's accumulator holds 128 gate columns then
// the 128 matching up columns, and the output tile is 128 columns wide.  GT_QKV: see GtQkv.
template <typename TOut, int MODE>
__global__ void __launch_bounds__(GT_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w, TOut* __restrict__ out,
               int out_stride, int M, int N, int K, int vec_ok, const GtQkv qkv, int* __restrict__ status) {
    constexpr bool GATED = MODE == GT_GATED;
    extern __shared__ unsigned char gt_smem_raw[];
    // the swizzled tiles must start on 1024-byte boundaries
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)gt_smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ uint64_t full_bar[GT_STAGES], empty_bar[GT_STAGES], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_base_holder;
    __shared__ volatile int gave_up;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int OUT_BN = GATED ? GT_BN / 2 : GT_BN;
    const int tiles_m = (M + GT_BM - 1) / GT_BM;
    const int tiles_n = (N + OUT_BN - 1) / OUT_BN;
    const int n_tiles = tiles_m * tiles_n;
    const int k_blocks = (K + GT_BK - 1) / GT_BK;

    if (threadIdx.x == 0) {
        gave_up = 0;
        for (int s = 0; s < GT_STAGES; ++s) {
            tc_mbar_init(&full_bar[s], 1);
            tc_mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            tc_mbar_init(&acc_full[b], 1);
            tc_mbar_init(&acc_empty[b], 4);                   // one arrival per epilogue warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {                                          // the MMA warp owns the tensor memory
        tc_tmem_alloc(&tmem_base_holder, GT_TMEM_COLS);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_holder;

    if (warp == 0) {
        // ------------------------------------------------------------ copies
        if (lane == 0) {
            int it = 0;
            bool stop = false;
            for (int tile = blockIdx.x; tile < n_tiles && !stop; tile += gridDim.x) {
                const int tm = tile % tiles_m, tn = tile / tiles_m;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % GT_STAGES;
                    if (it >= GT_STAGES && !tc_mbar_wait(&empty_bar[s], ((it / GT_STAGES) - 1) & 1, &gave_up)) {
                        if (!gave_up) atomicExch(status, 21);
                        gave_up = 1;
                        stop = true;
                        break;
                    }
                    unsigned char* a = tiles + (size_t)s * GT_STAGE_BYTES;
                    unsigned char* b = a + GT_A_BYTES;
                    tc_mbar_expect(&full_bar[s], GT_STAGE_BYTES);
                    dl_tma_load_2d(a, &tmap_x, kb * GT_BK, tm * GT_BM, &full_bar[s]);
                    if (GATED) {
                        dl_tma_load_2d(b, &tmap_w, kb * GT_BK, tn * OUT_BN, &full_bar[s]);
                        dl_tma_load_2d(b + GT_B_BYTES / 2, &tmap_w, kb * GT_BK, N + tn * OUT_BN, &full_bar[s]);
                    } else {
                        dl_tma_load_2d(b, &tmap_w, kb * GT_BK, tn * GT_BN, &full_bar[s]);
                    }
                }
            }
            if (stop) {
                // copies already issued must land before the block's shared memory is released
                for (int i = max(0, it - GT_STAGES); i < it; ++i) {
                    const long long t0 = clock64();
                    while (!tc_mbar_try(&full_bar[i % GT_STAGES], (i / GT_STAGES) & 1) && clock64() - t0 < TC_WAIT_CYCLES) {}
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ tensor-core issue
        if (lane == 0) {
            // instruction descriptor: float32 accumulate, bfloat16 A and B, both K-major, N 256, M 128
            const uint32_t idesc = tc_idesc_bf16(GT_BM, GT_BN);
            int it = 0, local = 0;
            bool stop = false;
            for (int tile = blockIdx.x; tile < n_tiles && !stop; tile += gridDim.x, ++local) {
                const int buf = local & 1;
                if (local >= 2 && !tc_mbar_wait(&acc_empty[buf], ((local >> 1) - 1) & 1, &gave_up)) {
                    if (!gave_up) atomicExch(status, 22);
                    gave_up = 1;
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(buf * GT_BN);
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % GT_STAGES;
                    if (!tc_mbar_wait(&full_bar[s], (it / GT_STAGES) & 1, &gave_up)) {
                        if (!gave_up) atomicExch(status, 23);
                        gave_up = 1;
                        stop = true;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_addr = tc_smem(tiles + (size_t)s * GT_STAGE_BYTES);
                    const uint64_t a_desc = tc_operand_desc(a_addr), b_desc = tc_operand_desc(a_addr + GT_A_BYTES);
#pragma unroll
                    for (int k = 0; k < GT_BK / 16; ++k)        // 16 k = 32 bytes further along the swizzled rows
                        tc_mma(d_tmem, a_desc + (uint64_t)(k * 2), b_desc + (uint64_t)(k * 2), idesc, (kb | k) != 0 ? 1u : 0u);
                    tc_commit(&empty_bar[s]);                    // the stage is free once these MMAs have read it
                }
                if (!stop) tc_commit(&acc_full[buf]);
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue: warp w reads lanes 32 (w % 4) ..
        const int quarter = warp & 3;
        int local = 0;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++local) {
            const int tm = tile % tiles_m, tn = tile / tiles_m;
            const int buf = local & 1;
            // the decision is the warp's: tcgen05.ld below needs all 32 lanes
            const bool ready = tc_mbar_wait(&acc_full[buf], (local >> 1) & 1, &gave_up);
            if (!__all_sync(0xffffffffu, ready)) {
                if (lane == 0 && !gave_up) atomicExch(status, 24);
                gave_up = 1;
                break;
            }
            tc_fence_after();
            const int row = tm * GT_BM + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * GT_BN);
            TOut* row_ptr = out + (size_t)row * out_stride;
            const int col_base = tn * OUT_BN;
            if (MODE == GT_QKV) {
                if (std::is_same<TOut, __nv_bfloat16>::value)
                    gt_qkv_epilogue(taddr, col_base, row, row < M, reinterpret_cast<__nv_bfloat16*>(out), out_stride, qkv);
            } else {
#pragma unroll 1
                for (int c0 = 0; c0 < OUT_BN; c0 += 32) {
                    float v[32];
                    tc_tmem_load32(taddr + (uint32_t)c0, v);    // every lane of the warp takes part
                    if (GATED) {
                        float u[32];
                        tc_tmem_load32(taddr + (uint32_t)(GT_BN / 2 + c0), u);
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = v[i] * (1.0f / (1.0f + expf(-v[i]))) * u[i];
                    }
                    if (row < M && col_base + c0 < N) gt_store32<TOut>(row_ptr, col_base + c0, N, v, vec_ok != 0);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) tc_mbar_arrive(&acc_empty[buf]);
        }
    }
    tc_fence_before();
    __syncthreads();                                         // nobody leaves while copies or MMAs may be in flight
    if (warp == 1) {
        tc_fence_after();
        tc_tmem_free(tmem_base, GT_TMEM_COLS);
    }
}

struct GtMapKey {
    const void* base;
    long long rows, cols, pitch;
    int box_rows;
    bool operator==(const GtMapKey& o) const {
        return base == o.base && rows == o.rows && cols == o.cols && pitch == o.pitch && box_rows == o.box_rows;
    }
};
struct GtMapKeyHash {
    size_t operator()(const GtMapKey& k) const {
        return std::hash<const void*>()(k.base) ^ ((size_t)k.rows * 1000003u) ^ ((size_t)k.cols * 10007u) ^ ((size_t)k.pitch * 31u) ^
               (size_t)k.box_rows;
    }
};

// Tensor maps cost a driver call to encode; they are kept per (matrix, shape, box).
static int gt_tensor_map(CUtensorMap* out, const void* base, long long rows, long long cols, long long pitch_bytes, int box_rows) {
    static std::unordered_map<GtMapKey, CUtensorMap, GtMapKeyHash> maps;
    static std::mutex maps_mutex;
    std::lock_guard<std::mutex> lock(maps_mutex);
    const GtMapKey key{base, rows, cols, pitch_bytes, box_rows};
    auto it = maps.find(key);
    if (it == maps.end()) {
        CUtensorMap fresh;
        if (dl_tmap_encode_2d_bf16(&fresh, base, (uint64_t)rows, (uint64_t)cols, (uint64_t)pitch_bytes, box_rows, GT_BK,
                                   DL_TMAP_SWIZZLE_128B) != 0)
            return DL_ERR_LAUNCH;
        if (maps.size() > 4096) maps.clear();
        it = maps.emplace(key, fresh).first;
    }
    *out = it->second;
    return DL_OK;
}

template <typename TOut, int MODE>
static int gt_launch(cudaStream_t s, const void* x, int x_stride, const void* w, void* out, int out_stride, int M, int N, int K,
                     int blocks, int* status, const GtQkv& qkv = GtQkv{}) {
    constexpr bool GATED = MODE == GT_GATED;
    const size_t smem = (size_t)GT_STAGES * GT_STAGE_BYTES + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<TOut, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "gemm_tc: shared memory %zu: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    CUtensorMap tmap_x, tmap_w;
    int rc = gt_tensor_map(&tmap_x, x, M, K, (long long)x_stride * 2, GT_BM);
    if (rc != DL_OK) return rc;
    rc = gt_tensor_map(&tmap_w, w, GATED ? 2ll * N : N, K, (long long)K * 2, GATED ? GT_BN / 2 : GT_BN);
    if (rc != DL_OK) return rc;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        return dl_fail(DL_ERR_LAUNCH, "gemm_tc: cannot query the device");
    const int out_bn = GATED ? GT_BN / 2 : GT_BN;
    const long long n_tiles = (long long)((M + GT_BM - 1) / GT_BM) * ((N + out_bn - 1) / out_bn);
    if (blocks <= 0 || blocks > sms) blocks = sms;
    if (blocks > n_tiles) blocks = (int)n_tiles;
    const int elem = (int)sizeof(TOut);
    const int vec_ok = (((uintptr_t)out % 16) == 0 && ((size_t)out_stride * elem) % 16 == 0) ? 1 : 0;
    gemm_tc_kernel<TOut, MODE><<<blocks, GT_THREADS, smem, s>>>(tmap_x, tmap_w, (TOut*)out, out_stride, M, N, K, vec_ok, qkv, status);
    DL_CHECK_LAUNCH("gemm_tc");
    return DL_OK;
}

// x: bf16 [M, K], rows x_stride elements apart.  w: bf16, contiguous rows of K.
// flags bit 0 (gated) clear: w is [N, K], out [M, N].  Set: w is [2N, K] (N gate rows, then N up
// rows), out [M, N] = silu(x Wg^T) * (x Wu^T), bfloat16 only.
// out_dtype: 0 = float32, 1 = bfloat16.  blocks: persistent blocks (<= 0: one per multiprocessor).
// status: int32, set non-zero if a wait expired.
extern "C" int dl_gemm_tc_bf16(const void* x, int x_stride, const void* w, void* out, int out_dtype, int out_stride, int M,
                               int N, int K, int flags, int blocks, int* status, void* stream) {
    DL_REQUIRE(M >= 1 && N >= 1 && K >= 8 && K % 8 == 0, "gemm_tc: M=%d N=%d K=%d (K must be a positive multiple of 8)", M, N, K);
    DL_REQUIRE(x_stride >= K && x_stride % 8 == 0, "gemm_tc: row stride of x (%d) must be a multiple of 8 and at least K", x_stride);
    DL_REQUIRE(((uintptr_t)x % 16) == 0 && ((uintptr_t)w % 16) == 0, "gemm_tc: x and W must be 16-byte aligned");
    DL_REQUIRE(out_stride >= N, "gemm_tc: out stride shorter than N");
    DL_REQUIRE(out_dtype == DL_F32 || out_dtype == DL_BF16, "gemm_tc: out dtype %d", out_dtype);
    DL_REQUIRE((flags & ~1) == 0, "gemm_tc: unknown flags %d", flags);
    DL_REQUIRE(status != nullptr, "gemm_tc: needs a status word");
    DL_REQUIRE((long long)M * out_stride < (1ll << 40), "gemm_tc: output too large");
    cudaStream_t s = (cudaStream_t)stream;
    if (flags & 1) {
        DL_REQUIRE(out_dtype == DL_BF16, "gemm_tc: the gated product writes bfloat16");
        return gt_launch<__nv_bfloat16, GT_GATED>(s, x, x_stride, w, out, out_stride, M, N, K, blocks, status);
    }
    if (out_dtype == DL_F32) return gt_launch<float, GT_PLAIN>(s, x, x_stride, w, out, out_stride, M, N, K, blocks, status);
    return gt_launch<__nv_bfloat16, GT_PLAIN>(s, x, x_stride, w, out, out_stride, M, N, K, blocks, status);
}

// The Q/K/V product of a prompt with the rotation and the cache write in its epilogue.
// x: bf16 [M, K]; w: bf16 [q_cols + 2 kv_cols, K] (query rows, key rows, value rows), contiguous.
// q_out: bf16 [M, q_cols] rows q_stride apart: the rotated queries.  The rotated keys and the values go to
// the pages of the cache (k_pool [pages, nkv, 64, hd], v_pool [pages, nkv, hd, 64]) that block_table
// [sequences, bt_stride] names for token_seq[row] at position token_pos[row].  cos_t, sin_t: float32
// [table_rows, hd/2] (a full-width rotation, pairs d and d + hd/2).  head_dim 64 or 128; q_cols and
// kv_cols multiples of 256.  Same bits as the plain product followed by dl_rope_cache_write.
extern "C" int dl_gemm_tc_qkv_bf16(const void* x, int x_stride, const void* w, void* q_out, int q_stride, int M, int K, int q_cols,
                                   int kv_cols, int hd, int nkv, const float* cos_t, const float* sin_t, int table_rows,
                                   const int32_t* token_pos, const int32_t* token_seq, const int32_t* block_table, int bt_stride,
                                   void* k_pool, void* v_pool, int n_pages, int blocks, int* status, void* stream) {
    DL_REQUIRE(M >= 1 && K >= 8 && K % 8 == 0, "gemm_tc_qkv: M=%d K=%d (K must be a positive multiple of 8)", M, K);
    DL_REQUIRE(hd == 64 || hd == 128, "gemm_tc_qkv: head_dim %d (takes 64 and 128)", hd);
    DL_REQUIRE(q_cols > 0 && kv_cols > 0 && q_cols % GT_BN == 0 && kv_cols % GT_BN == 0 && kv_cols == nkv * hd,
               "gemm_tc_qkv: %d query and %d key columns must be multiples of %d (and the key columns nkv * head_dim)", q_cols,
               kv_cols, GT_BN);
    DL_REQUIRE(x_stride >= K && x_stride % 8 == 0 && q_stride >= q_cols && q_stride % 8 == 0, "gemm_tc_qkv: row strides");
    DL_REQUIRE(((uintptr_t)x % 16) == 0 && ((uintptr_t)w % 16) == 0 && ((uintptr_t)q_out % 16) == 0 && ((uintptr_t)k_pool % 16) == 0 &&
                   ((uintptr_t)v_pool % 16) == 0 && ((uintptr_t)cos_t % 16) == 0 && ((uintptr_t)sin_t % 16) == 0,
               "gemm_tc_qkv: x, W, q, the pools and the tables must be 16-byte aligned");
    DL_REQUIRE(cos_t && sin_t && table_rows > 0 && token_pos && token_seq && block_table && bt_stride >= 1 && n_pages > 0,
               "gemm_tc_qkv: needs tables, positions, a block table and a cache");
    DL_REQUIRE(status != nullptr, "gemm_tc_qkv: needs a status word");
    GtQkv qkv{q_cols, kv_cols, hd, nkv, cos_t, sin_t, table_rows, token_pos, token_seq, block_table, bt_stride,
              (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, n_pages};
    return gt_launch<__nv_bfloat16, GT_QKV>((cudaStream_t)stream, x, x_stride, w, q_out, q_stride, M, q_cols + 2 * kv_cols, K, blocks,
                                            status, qkv);
}
