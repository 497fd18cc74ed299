// y = x W^T for 17 to 128 rows of x (decode steps of many sequences): a weight-streaming product
// on the fifth-generation tensor cores.
//
// With up to 128 rows every projection of a decode step is still bound by the bytes of W, read once
// (at 128 rows a bfloat16 weight byte meets 128 FLOP; the machine's ridge is near 250).  The reference
// runs these products through cuBLAS (src/DotLLM.Cuda/CudaTransformerModel.cs:317-349,
// src/DotLLM.Cuda/CudaGemm.cs:29-40), whose tiles are too few for 148 multiprocessors at these row
// counts.  Here the product is swapped: 128 rows of W are the M of tcgen05.mma and the tokens (padded
// to a multiple of 16) its N, so the accumulator in tensor memory is [128 outputs][tokens] and W is
// the operand that streams.
//
// Shape: persistent, warp-specialised, stream-K.  The work is the list of (tile of W rows, 64-wide
// chunk of k) units in tile-major order, cut into contiguous shares, one per block: equal shares so
// that every multiprocessor streams the same number of bytes, or, where the tiles divide among at
// least three quarters of the multiprocessors in whole tiles or equal parts of a tile, shares cut
// there (a cut tile costs a trip through global memory at the end of the kernel).  The cut depends on the
// matrix and the device only, never on the rows of x.  A unit is one box of W [128][64] (plain), or
// two (gated, W = [gate; up]: 128 gate rows and the 128 matching up rows; two MMAs fill two column
// ranges of the accumulator and the epilogue writes silu(gate) * up, native/kernels/swiglu.cu:7-41,
// lane by lane with no exchange between threads), and one box of x [tokens][64].
//   warp 0   one thread issues the tensor-map copies (TMA, 128-byte swizzle, no multicast) into a ring
//            of stages, two units back to back so that neighbouring 128-byte pieces of a row of W
//            reach the memory together; with resident weights the first ring of W boxes is issued
//            before the kernel waits for its predecessor on the stream;
//   warp 1   one thread issues tcgen05.mma (M 128, N tokens, K 16; four per box) into one of two
//            accumulator buffers in tensor memory and commits each stage back to the ring;
//   warp 2   row statistics when x is a stream times a gain (see below);
//   warps 4-19  the epilogue: four groups of four warps that take turns at slices of 8 tokens.  A
//            warp reads its 32 lanes (outputs) of a finished accumulator with tcgen05.ld.  The work
//            per token is a short chain of dependent instructions, so what makes the epilogue fast
//            is the number of warps it is spread over (one group: 8 us for a gated tile of 64
//            tokens; four groups: under 3).  A tile that lies wholly inside one share is finished at once.  A tile cut
//            between shares is written as float32 parts; the block that arrives last adds the parts
//            in share order, so the result has the same bits on every launch.  When that happens at
//            the end of a block's share (the usual case) the ring is idle, and the other blocks' parts
//            are fetched into it by bulk copies while the block's own part stays in tensor memory.
//
// The two fusions of the add + RMSNorm between products (native/kernels/fused_add_rmsnorm.cu:9-72 is
// a kernel of its own in the reference) are those of the product for up to 16 rows: with `gain` a
// float32 product adds into the residual stream, writes stream * gain as bfloat16 and the sum of
// squares of every row per 128 columns; with `sumsq_in` the statistics warp adds those sums in
// order and every output row is multiplied by rsqrt(sum / n + eps).
//
// Every wait on an mbarrier is bounded (about a second of clock cycles); on expiry the kernel records
// a code in `status`, stops issuing work, waits (bounded) for copies in flight, frees its tensor
// memory and returns.  Decisions that the epilogue threads must take together are taken with a
// reducing named barrier, so no thread is left waiting at a barrier that others have abandoned.
#include "common.cuh"
#include "tma.cuh"
#include "tcgen05.cuh"
#include <type_traits>

#define GD_BM 128                              // rows of W per box: the MMA's M
#define GD_BK 64                               // k per chunk: 128 bytes, the swizzle's width
#define GD_A_BYTES (GD_BM * GD_BK * 2)
#define GD_MAX_STAGES 12
#define GD_MAX_ROWS 128
#define GD_SUM_STRIDE 128                      // floats between the sums of two 128-column parts
#define GD_SMEM_BUDGET (216 * 1024)
#ifndef GD_EPI_GROUPS
#define GD_EPI_GROUPS 4                       // groups of four epilogue warps; a group covers the 128 lanes
#endif
#define GD_EPI_THREADS (128 * GD_EPI_GROUPS)
#define GD_THREADS (128 + GD_EPI_THREADS)      // warps 0-3: copies, MMA issue, row statistics, idle
#define GD_CHUNK_BYTES (32 * GD_BM * 4)        // 32 accumulator columns of a part: [8][128 lanes][4] floats

enum { GD_PLAIN = 0, GD_GATED = 1 };

struct GdFuse {
    const float* gain;          // set: out is the float32 residual stream, out += x W^T in place, and ...
    __nv_bfloat16* scaled;      // ... scaled[m][n] = bf16(out[m][n] * gain[n]), rows scaled_stride apart,
    int scaled_stride;
    float* sumsq_out;           // ... sumsq_out[(n / 128) * 128 + m] = sum over those 128 columns of out[m][n]^2
    const float* sumsq_in;      // set: output row m is multiplied by rsqrt(sum_p sumsq_in[p * 128 + m] * inv_n + eps)
    int n_parts;
    float inv_n, eps;
};

struct GdWork {
    void* out;
    int out_stride;
    int M, Mpad, N, K;
    int cpt, total, share;      // chunks per tile, units in all, units per block
    int stages, stage_bytes;
    GdFuse fuse;
};

template <typename TOut> __device__ __forceinline__ void gd_store(TOut* p, float v);
template <> __device__ __forceinline__ void gd_store<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void gd_store<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// All epilogue threads meet; true if `ok` held for every one of them.
__device__ __forceinline__ bool gd_epilogue_all(bool ok) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %1, 0;\n\tbar.red.and.pred q, 1, %2, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
        : "=r"(r)
        : "r"(ok ? 1u : 0u), "n"(GD_EPI_THREADS)
        : "memory");
    return r != 0;
}
__device__ __forceinline__ void gd_epilogue_sync() { asm volatile("bar.sync 1, %0;" ::"n"(GD_EPI_THREADS) : "memory"); }

// The epilogue works on 8 tokens (accumulator columns) at a time, in short loops: a block runs its
// epilogue once or twice per launch, so code unrolled over 32 or 64 tokens would be executed cold,
// one instruction-cache miss after another (measured: 11 us for 32 tokens of the add-into-stream
// form, unrolled).
//
// 8 tokens c .. c+7 of output column n, held by this thread: scale, gate, add into the stream, store.
// `u` is read only when GATED.  `ss_row`: this warp's row of the per-token sums of squares in shared
// memory (add-into-stream only); `h_in`: the stream's present values of these tokens (gd_stream8).
// Loads, arithmetic and stores are kept in separate stages so that
// the 8 tokens' chains overlap (a store between two tokens' loads would order them).
template <typename TOut, bool GATED>
__device__ __forceinline__ void gd_finish8(const float (&v)[8], const float (&u)[8], int c, int n, bool n_ok, TOut* __restrict__ out,
                                           int out_stride, int M, const float* __restrict__ row_scale, const GdFuse& fuse,
                                           float gain_n, float* __restrict__ ss_row, int lane, const float (&h_in)[8]) {
    float val[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) val[i] = row_scale != nullptr ? row_scale[min(c + i, GD_MAX_ROWS - 1)] : 1.0f;
    if (!GATED && std::is_same<TOut, float>::value && fuse.gain != nullptr) {
        float* __restrict__ stream = reinterpret_cast<float*>(out);
        __nv_bfloat16* __restrict__ scaled = fuse.scaled;
        float h[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float prod = row_scale != nullptr ? v[i] * val[i] : v[i];
            h[i] = (n_ok && c + i < M) ? h_in[i] + prod : 0.f;    // h_in: the stream's values, asked for ahead of time
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (n_ok && c + i < M) {
                stream[(size_t)(c + i) * out_stride + n] = h[i];
                scaled[(size_t)(c + i) * fuse.scaled_stride + n] = __float2bfloat16_rn(h[i] * gain_n);
            }
        }
        // sums of squares over the warp's 32 columns, the 8 tokens' butterflies side by side
#pragma unroll
        for (int i = 0; i < 8; ++i) h[i] = h[i] * h[i];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
#pragma unroll
            for (int i = 0; i < 8; ++i) h[i] += __shfl_xor_sync(0xffffffffu, h[i], o);   // both partners add the same two numbers
        }
        if (lane == 0) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (c + i < M) ss_row[c + i] = h[i];
        }
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float g = row_scale != nullptr ? v[i] * val[i] : v[i];
            if (GATED) {
                const float up = row_scale != nullptr ? u[i] * val[i] : u[i];
                // bfloat16 keeps 8 bits: the fast exponential and reciprocal (errors of a few float32 ulps) change
                // no output bit that the exact ones would not; a float32 result gets the exact functions
                if (std::is_same<TOut, float>::value) g = g * (1.0f / (1.0f + expf(-g))) * up;
                else g = g * __fdividef(1.0f, 1.0f + __expf(-g)) * up;    // no branches: the 8 tokens' chains interleave
            }
            val[i] = g;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (c + i < M && n_ok) gd_store<TOut>(out + (size_t)(c + i) * out_stride + n, val[i]);
    }
}

// The residual stream's values of tokens c .. c+7 at column n (zeros beyond the matrix).
__device__ __forceinline__ void gd_stream8(float (&h)[8], const float* __restrict__ stream, int out_stride, int c, int n, bool n_ok,
                                           int M) {
#pragma unroll
    for (int i = 0; i < 8; ++i) h[i] = (n_ok && c + i < M) ? __ldcg(stream + (size_t)(c + i) * out_stride + n) : 0.f;
}

// A part in global or shared memory holds 32 accumulator columns as [8][128 lanes][4] floats: a
// thread's four consecutive columns are one float4, and a warp's float4s are contiguous.  These add
// columns 8q .. 8q+7 of such a chunk.
__device__ __forceinline__ void gd_add8_global(float (&v)[8], const float* chunk, int q, int lane128) {
    const float4 a = __ldcg(reinterpret_cast<const float4*>(chunk) + (2 * q) * GD_BM + lane128);
    const float4 b = __ldcg(reinterpret_cast<const float4*>(chunk) + (2 * q + 1) * GD_BM + lane128);
    v[0] += a.x, v[1] += a.y, v[2] += a.z, v[3] += a.w, v[4] += b.x, v[5] += b.y, v[6] += b.z, v[7] += b.w;
}
__device__ __forceinline__ void gd_add8_shared(float (&v)[8], const unsigned char* chunk, int q, int lane128) {
    const float4 a = *(reinterpret_cast<const float4*>(chunk) + (2 * q) * GD_BM + lane128);
    const float4 b = *(reinterpret_cast<const float4*>(chunk) + (2 * q + 1) * GD_BM + lane128);
    v[0] += a.x, v[1] += a.y, v[2] += a.z, v[3] += a.w, v[4] += b.x, v[5] += b.y, v[6] += b.z, v[7] += b.w;
}

template <typename TOut, int MODE>
__global__ void __launch_bounds__(GD_THREADS, 1)
gemm_decode_tc_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x, const GdWork work,
                      int early_weights, float* __restrict__ partials, int* __restrict__ counters, int* __restrict__ status) {
    constexpr bool GATED = MODE == GD_GATED;
    constexpr int BOXES = MODE == GD_PLAIN ? 1 : 2;          // boxes of W per unit
    constexpr int PARTS = GATED ? 2 : 1;                     // accumulator ranges one finished chunk needs
    extern __shared__ unsigned char gd_smem_raw[];
    // the swizzled tiles must start on 1024-byte boundaries
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)gd_smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ uint64_t full_bar[GD_MAX_STAGES], empty_bar[GD_MAX_STAGES], acc_full[2], acc_empty[2], scale_bar, merge_bar[2];
    __shared__ uint32_t tmem_base_holder;
    __shared__ volatile int gave_up;
    __shared__ int last_flag;
    __shared__ float row_scale_smem[GD_MAX_ROWS];
    __shared__ float ss_part[4][GD_MAX_ROWS];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int Mpad = work.Mpad, cpt = work.cpt, stages = work.stages;
    const int Mcol = (Mpad + 31) & ~31;                     // columns between two ranges: tcgen05.ld reads 32 at a time
    const int buf_cols = BOXES * Mcol;                      // accumulator columns of one buffer
    uint32_t tmem_cols = 32;
    while ((int)tmem_cols < 2 * buf_cols) tmem_cols <<= 1;
    const int begin = min(work.total, (int)blockIdx.x * work.share), end = min(work.total, ((int)blockIdx.x + 1) * work.share);

    if (threadIdx.x == 0) {
        gave_up = 0;
        for (int s = 0; s < stages; ++s) {
            tc_mbar_init(&full_bar[s], 1);
            tc_mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            tc_mbar_init(&acc_full[b], 1);
            tc_mbar_init(&acc_empty[b], 4 * GD_EPI_GROUPS);  // one arrival per epilogue warp
            tc_mbar_init(&merge_bar[b], 1);
        }
        tc_mbar_init(&scale_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tc_tmem_alloc(&tmem_base_holder, tmem_cols);      // the MMA warp owns the tensor memory
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    dl_launch_dependents();
    const uint32_t tmem_base = tmem_base_holder;

    if (warp == 0) {
        // ------------------------------------------------------------ copies
        if (lane == 0) {
            const int n_mine = end - begin;
            const uint32_t stage_bytes = (uint32_t)work.stage_bytes;
            const uint64_t policy = dl_stream_policy();     // W is read once a step: first out of the L2
            auto load_w = [&](int unit, int s) {
                const int tile = unit / cpt, kc = unit - tile * cpt;
                unsigned char* a = tiles + (size_t)s * stage_bytes;
                const int row0 = tile * GD_BM;
                dl_tma_load_2d_hint(a, &tmap_w, kc * GD_BK, row0, &full_bar[s], policy);
                if (GATED) dl_tma_load_2d_hint(a + GD_A_BYTES, &tmap_w, kc * GD_BK, row0 + work.N, &full_bar[s], policy);
            };
            auto load_x = [&](int unit, int s) {
                const int kc = unit % cpt;
                unsigned char* b = tiles + (size_t)s * stage_bytes + BOXES * GD_A_BYTES;
                dl_tma_load_2d(b, &tmap_x, kc * GD_BK, 0, &full_bar[s]);
            };
            // While the kernel before this one finishes, the ring fills with weights (the caller
            // vouches that nothing pending writes them); x is that kernel's output and waits.
            const int pre = early_weights ? min(stages, n_mine) : 0;
            for (int i = 0; i < pre; ++i) {
                tc_mbar_expect(&full_bar[i], stage_bytes);   // a box is always written whole: parts outside a matrix arrive as zeros
                load_w(begin + i, i);
            }
            dl_grid_dependency_wait();
            for (int i = 0; i < pre; ++i) load_x(begin + i, i);
            int it = pre;
            bool stop = false;
            const int group = stages >= 4 ? 2 : 1;
            while (it < n_mine && !stop) {
                // wait until `group` stages are free, then issue their copies back to back
                const int n_now = min(group, n_mine - it);
                for (int j = 0; j < n_now; ++j) {
                    const int i2 = it + j, s = i2 % stages;
                    if (i2 >= stages && !tc_mbar_wait(&empty_bar[s], ((i2 / stages) - 1) & 1, &gave_up)) {
                        if (!gave_up) atomicExch(status, 31);
                        gave_up = 1;
                        stop = true;
                        break;
                    }
                }
                if (stop) break;
                for (int j = 0; j < n_now; ++j) {
                    const int s = (it + j) % stages;
                    tc_mbar_expect(&full_bar[s], stage_bytes);
                    load_w(begin + it + j, s);
                }
                for (int j = 0; j < n_now; ++j) load_x(begin + it + j, (it + j) % stages);
                it += n_now;
            }
            if (stop) {
                // copies already issued must land before the block's shared memory is released
                for (int i = max(0, it - stages); i < it; ++i) {
                    const long long t0 = clock64();
                    while (!tc_mbar_try(&full_bar[i % stages], (i / stages) & 1) && clock64() - t0 < TC_WAIT_CYCLES) {}
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ tensor-core issue
        if (lane == 0) {
            const uint32_t idesc = tc_idesc_bf16(GD_BM, Mpad);
            int it = 0, seg = 0;
            bool stop = false;
            for (int cur = begin; cur < end && !stop; ++seg) {
                const int tile = cur / cpt;
                const int seg_end = min(end, (tile + 1) * cpt);
                const int buf = seg & 1;
                if (seg >= 2 && !tc_mbar_wait(&acc_empty[buf], ((seg >> 1) - 1) & 1, &gave_up)) {
                    if (!gave_up) atomicExch(status, 32);
                    gave_up = 1;
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(buf * buf_cols);
                for (int u = cur; u < seg_end; ++u, ++it) {
                    const int s = it % stages;
                    if (!tc_mbar_wait(&full_bar[s], (it / stages) & 1, &gave_up)) {
                        if (!gave_up) atomicExch(status, 33);
                        gave_up = 1;
                        stop = true;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_addr = tc_smem(tiles + (size_t)s * work.stage_bytes);
                    const uint64_t a_desc = tc_operand_desc(a_addr);
                    const uint64_t b_desc = tc_operand_desc(a_addr + BOXES * GD_A_BYTES);
#pragma unroll
                    for (int k = 0; k < GD_BK / 16; ++k) {      // 16 k = 32 bytes further along the swizzled rows
                        const uint32_t acc = (u > cur || k > 0) ? 1u : 0u;
                        tc_mma(d_tmem, a_desc + (uint64_t)(k * 2), b_desc + (uint64_t)(k * 2), idesc, acc);
                        if (BOXES == 2)
                            tc_mma(d_tmem + (uint32_t)Mcol, tc_operand_desc(a_addr + GD_A_BYTES) + (uint64_t)(k * 2),
                                   b_desc + (uint64_t)(k * 2), idesc, acc);
                    }
                    tc_commit(&empty_bar[s]);                // the stage is free once these MMAs have read it
                }
                if (!stop) tc_commit(&acc_full[buf]);
                cur = seg_end;
            }
        }
    } else if (warp == 2) {
        // ------------------------------------------------------------ row statistics
        if (work.fuse.sumsq_in != nullptr) {
            dl_grid_dependency_wait();                       // the sums come from the kernel before this one
            for (int m = lane; m < work.M; m += 32) {
                float acc = 0.f;
                for (int p0 = 0; p0 < work.fuse.n_parts; p0 += 8) {
                    float v[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        v[i] = p0 + i < work.fuse.n_parts ? __ldcg(work.fuse.sumsq_in + (size_t)(p0 + i) * GD_SUM_STRIDE + m) : 0.f;
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc += v[i];  // part order: fixed
                }
                row_scale_smem[m] = rsqrtf(acc * work.fuse.inv_n + work.fuse.eps);
            }
            __threadfence_block();
            __syncwarp();
            if (lane == 0) tc_mbar_arrive(&scale_bar);
        }
    } else if (warp >= 4) {
        // ------------------------------------------------------------ epilogue: warp w owns lanes 32 (w % 4) ..
        dl_grid_dependency_wait();       // out, partials and counters may still be in use by the kernel before this one
        const int quarter = warp & 3, group = (warp - 4) >> 2;          // groups take turns at 8-token slices
        const int lane128 = quarter * 32 + lane;
        const bool leader = threadIdx.x == GD_THREADS - GD_EPI_THREADS;
        TOut* out = reinterpret_cast<TOut*>(work.out);
        const int M = work.M, N = work.N, share = work.share;
        const float* row_scale = nullptr;
        const bool adds = !GATED && std::is_same<TOut, float>::value && work.fuse.gain != nullptr;
        const size_t part_floats = (size_t)buf_cols * GD_BM;
        const int n_chunks = (M + 31) / 32;                  // 32-token chunks that hold tokens
        const uint32_t ring_bytes = (uint32_t)(stages * work.stage_bytes);
        int seg = 0;
        bool dead = false;
        for (int cur = begin; cur < end && !dead; ++seg) {
            const int tile = cur / cpt;
            const int seg_end = min(end, (tile + 1) * cpt);
            const int buf = seg & 1;
            const bool last_seg = seg_end == end;
            bool ok = tc_mbar_wait(&acc_full[buf], (seg >> 1) & 1, &gave_up);
            if (ok && work.fuse.sumsq_in != nullptr && row_scale == nullptr) ok = tc_mbar_wait(&scale_bar, 0, &gave_up);
            if (!gd_epilogue_all(ok)) {
                if (!ok && !gave_up) atomicExch(status, 34);
                gave_up = 1;
                break;
            }
            if (work.fuse.sumsq_in != nullptr) row_scale = row_scale_smem;
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * buf_cols);
            const bool whole = (cur == tile * cpt) && (seg_end == (tile + 1) * cpt);
            int g_lo = 0, g_hi = 0;
            bool finish = whole, bulk = false;
            int n_buf = 1;
            uint32_t item_bytes = 0;
            if (!whole) {
                // a block's first tile may be shared with the block before, its last with the block after
                const int which = (tile == begin / cpt) ? 0 : 1;
                float* mine = partials + ((size_t)blockIdx.x * 2 + which) * part_floats;
#pragma unroll 1
                for (int c = 8 * group; c < buf_cols; c += 8 * GD_EPI_GROUPS) {
                    float v[8];
                    tc_tmem_load8(taddr + (uint32_t)c, v);
                    float4* dst = reinterpret_cast<float4*>(mine) + (size_t)(c >> 2) * GD_BM + lane128;
                    dst[0] = make_float4(v[0], v[1], v[2], v[3]);
                    dst[GD_BM] = make_float4(v[4], v[5], v[6], v[7]);
                }
                if (!last_seg) {                             // the last segment keeps its accumulator: nothing follows it
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) tc_mbar_arrive(&acc_empty[buf]);
                }
                g_lo = (tile * cpt) / share, g_hi = ((tile + 1) * cpt - 1) / share;
                __threadfence();
                gd_epilogue_sync();                          // every thread's part is written
                if (leader) {
                    // One read-modify-write that releases this block's part and acquires the parts of the
                    // blocks counted before.
                    int seen;
                    asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(seen) : "l"(counters + tile) : "memory");
                    const int last = (seen == g_hi - g_lo) ? 1 : 0;
                    if (last) counters[tile] = 0;            // ready for the next product or launch
                    last_flag = last;
                }
                gd_epilogue_sync();
                finish = last_flag != 0;
                // At the end of the share the ring is idle (every copy has landed and every MMA has read
                // its stage): the other blocks' parts come in by bulk copies, up to two chunks ahead.
                item_bytes = (uint32_t)((g_hi - g_lo) * PARTS) * GD_CHUNK_BYTES;
                n_buf = item_bytes * 2 <= ring_bytes ? 2 : 1;
                bulk = finish && last_seg && item_bytes <= ring_bytes;
            }
            if (finish) {
                const int n_items = n_chunks;               // an item: 32 tokens
                auto issue = [&](int item) {                 // leader only: fetch what item `item` needs of the other blocks' parts
                    const int c0 = item * 32;
                    const int b = item % n_buf;
                    unsigned char* dst = tiles + (size_t)b * item_bytes;
                    tc_mbar_expect(&merge_bar[b], item_bytes);
                    for (int gg = g_lo; gg <= g_hi; ++gg) {
                        if (gg == (int)blockIdx.x) continue;
                        const int wh = (tile == (gg * share) / cpt) ? 0 : 1;
                        const float* theirs = partials + ((size_t)gg * 2 + wh) * part_floats;
#pragma unroll
                        for (int p = 0; p < PARTS; ++p) {
                            dl_bulk_load(dst, theirs + (size_t)(p * Mcol + c0) * GD_BM, GD_CHUNK_BYTES, &merge_bar[b]);
                            dst += GD_CHUNK_BYTES;
                        }
                    }
                };
                if (bulk && leader) {
                    tc_fence_async_smem();
                    for (int i = 0; i < min(n_buf, n_items); ++i) issue(i);
                }
#pragma unroll 1
                for (int item = 0; item < n_items; ++item) {
                    const int c0 = item * 32;
                    const int n = tile * GD_BM + lane128;
                    const bool n_ok = n < N;
                    const float gain_n = (adds && n_ok) ? __ldg(work.fuse.gain + n) : 0.f;
                    const int col = c0;                      // first accumulator column of the chunk (gate's when gated)
                    // The stream's values of this group's slices are asked for now: they arrive while the
                    // merge data does (only this tile's finisher ever writes them).
                    constexpr int SLICES = (4 + GD_EPI_GROUPS - 1) / GD_EPI_GROUPS;
                    float h_pre[SLICES][8];
#pragma unroll
                    for (int j = 0; j < SLICES; ++j) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) h_pre[j][i] = 0.f;
                        if (adds && group + j * GD_EPI_GROUPS < 4)
                            gd_stream8(h_pre[j], reinterpret_cast<const float*>(work.out), work.out_stride,
                                       c0 + 8 * (group + j * GD_EPI_GROUPS), n, n_ok, M);
                    }
                    const unsigned char* src = nullptr;
                    if (!whole && bulk) {
                        // a block merges this way once at most (at its last segment): use k of a buffer is phase k
                        const bool landed = tc_mbar_wait(&merge_bar[item % n_buf], (uint32_t)((item / n_buf) & 1), &gave_up);
                        if (!gd_epilogue_all(landed)) {
                            if (!landed && !gave_up) atomicExch(status, 35);
                            gave_up = 1;
                            dead = true;
                            break;
                        }
                        src = tiles + (size_t)(item % n_buf) * item_bytes;
                    }
#pragma unroll
                    for (int j = 0; j < SLICES; ++j) {       // 8 tokens at a time
                        const int q = group + j * GD_EPI_GROUPS;
                        const int c = c0 + 8 * q;
                        if (q >= 4 || c >= M) break;
                        float v[8], u[8];
                        if (whole) {
                            tc_tmem_load8(taddr + (uint32_t)(col + 8 * q), v);
                            if (GATED) tc_tmem_load8(taddr + (uint32_t)(Mcol + col + 8 * q), u);
                        } else {
#pragma unroll
                            for (int i = 0; i < 8; ++i) v[i] = 0.f, u[i] = 0.f;
                            const unsigned char* theirs_s = src;
#pragma unroll 1
                            for (int gg = g_lo; gg <= g_hi; ++gg) {      // share order: fixed
                                if (bulk && gg == (int)blockIdx.x) {     // this block's own part is still in tensor memory
                                    float t[8];
                                    tc_tmem_load8(taddr + (uint32_t)(col + 8 * q), t);
#pragma unroll
                                    for (int i = 0; i < 8; ++i) v[i] += t[i];
                                    if (GATED) {
                                        tc_tmem_load8(taddr + (uint32_t)(Mcol + col + 8 * q), t);
#pragma unroll
                                        for (int i = 0; i < 8; ++i) u[i] += t[i];
                                    }
                                } else if (bulk) {
                                    gd_add8_shared(v, theirs_s, q, lane128);
                                    if (GATED) gd_add8_shared(u, theirs_s + GD_CHUNK_BYTES, q, lane128);
                                    theirs_s += PARTS * GD_CHUNK_BYTES;
                                } else {
                                    const int wh = (tile == (gg * share) / cpt) ? 0 : 1;
                                    const float* theirs = partials + ((size_t)gg * 2 + wh) * part_floats;
                                    gd_add8_global(v, theirs + (size_t)col * GD_BM, q, lane128);
                                    if (GATED) gd_add8_global(u, theirs + (size_t)(Mcol + col) * GD_BM, q, lane128);
                                }
                            }
                        }
                        gd_finish8<TOut, GATED>(v, u, c, n, n_ok, out, work.out_stride, M, row_scale, work.fuse, gain_n,
                                                ss_part[quarter], lane, h_pre[j]);
                    }
                    if (bulk) {
                        // Every thread's reads of the buffer have completed (their values went into the stores
                        // above) before it passes this barrier, so the copy that refills the buffer comes after them.
                        gd_epilogue_sync();
                        if (leader && item + n_buf < n_items) {
                            tc_fence_async_smem();
                            issue(item + n_buf);
                        }
                    }
                    if (adds && c0 + 32 >= M) {
                        // the 128 columns' sum of squares per row: the four warps' 32-column sums, added in warp order
                        gd_epilogue_sync();
                        const int m = lane128;
                        if (m < M && group == 0)
                            work.fuse.sumsq_out[(size_t)tile * GD_SUM_STRIDE + m] =
                                ((ss_part[0][m] + ss_part[1][m]) + ss_part[2][m]) + ss_part[3][m];
                        gd_epilogue_sync();
                    }
                }
            }
            if (whole && !dead) {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) tc_mbar_arrive(&acc_empty[buf]);
            }
            if (!whole && !dead) gd_epilogue_sync();         // last_flag is read by all before anyone writes it again
            cur = seg_end;
        }
    }
    tc_fence_before();
    __syncthreads();                                         // nobody leaves while copies or MMAs may be in flight
    if (warp == 1) {
        tc_fence_after();
        tc_tmem_free(tmem_base, tmem_cols);
    }
}

// How the work of an (N, K) matrix is cut: the kind of unit, tiles (128 outputs),
// chunks per tile, blocks, units per block.  Depends on the matrix and the device only, never on M.
struct GdPlan {
    int mode, tiles, cpt, total, blocks, share;
};

static GdPlan gd_plan(int N, int K, int gated, int sms) {
    GdPlan p;
    p.mode = gated ? GD_GATED : GD_PLAIN;
    p.tiles = (N + GD_BM - 1) / GD_BM;
    p.cpt = (K + GD_BK - 1) / GD_BK;
    p.total = p.tiles * p.cpt;
    p.blocks = (p.total + 3) / 4;                            // at least about four units a block
    if (p.blocks > sms) p.blocks = sms;
    if (p.blocks < 1) p.blocks = 1;
    p.share = (p.total + p.blocks - 1) / p.blocks;
    // Cuts cost: a cut tile goes through global memory and is finished by whoever arrives last.  When
    // the tiles divide among the multiprocessors in whole tiles or in equal parts of a tile, and at
    // least three quarters of the multiprocessors get work that way, cut there and nowhere else.
    if (p.tiles <= sms && p.total >= 4 * p.tiles) {
        const int parts = sms / p.tiles;
        if (p.cpt % parts == 0 && 4 * p.tiles * parts >= 3 * sms && p.cpt / parts >= 4) p.share = p.cpt / parts;
    }
    p.blocks = (p.total + p.share - 1) / p.share;            // no block without work
    return p;
}

static int gd_mpad(int M) { return (M + 15) / 16 * 16; }
static int gd_buf_cols(int M, int mode) { return (mode == GD_PLAIN ? 1 : 2) * ((gd_mpad(M) + 31) / 32 * 32); }

// Scratch the product needs: float32 partial sums and int32 arrival counters (zero before the first
// launch; every launch leaves them zero).
extern "C" int dl_gemm_decode_tc_scratch(int M, int N, int K, int gated, int sms, long long* partial_floats, int* n_counters) {
    const GdPlan p = gd_plan(N, K, gated, sms);
    *partial_floats = (long long)p.blocks * 2 * gd_buf_cols(M, p.mode) * GD_BM;
    *n_counters = p.tiles;
    return DL_OK;
}

template <typename TOut, int MODE>
static int gd_launch(const GdPlan& p, cudaStream_t s, const void* x, int x_stride, const void* w, void* out, int out_stride, int M,
                     int N, int K, int early, float* partials, int* counters, int* status, const GdFuse& fuse) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_decode_tc_kernel<TOut, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             GD_SMEM_BUDGET);
        if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "gemm_decode_tc: shared memory %d: %s", GD_SMEM_BUDGET, cudaGetErrorString(e));
        configured = true;
    }
    const int Mpad = gd_mpad(M);
    const int stage_bytes = (MODE == GD_PLAIN ? 1 : 2) * GD_A_BYTES + Mpad * GD_BK * 2;
    int stages = (GD_SMEM_BUDGET - 1024) / stage_bytes;
    if (stages > GD_MAX_STAGES) stages = GD_MAX_STAGES;
    CUtensorMap tmap_w, tmap_x;
    if (dl_tmap_cached_2d_bf16(&tmap_w, w, MODE == GD_GATED ? 2ull * N : (unsigned long long)N, K, (unsigned long long)K * 2, GD_BM,
                               GD_BK, DL_TMAP_SWIZZLE_128B) != 0)
        return DL_ERR_LAUNCH;
    if (dl_tmap_cached_2d_bf16(&tmap_x, x, M, K, (unsigned long long)x_stride * 2, Mpad, GD_BK, DL_TMAP_SWIZZLE_128B) != 0)
        return DL_ERR_LAUNCH;
    const GdWork work{out, out_stride, M, Mpad, N, K, p.cpt, p.total, p.share, stages, stage_bytes, fuse};
    const size_t smem = (size_t)stages * stage_bytes + 1024;
    cudaError_t le = dl_launch_dependent(gemm_decode_tc_kernel<TOut, MODE>, dim3(p.blocks), dim3(GD_THREADS), smem, s, tmap_w, tmap_x,
                                         work, early, partials, counters, status);
    if (le != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "gemm_decode_tc: %s", cudaGetErrorString(le));
    return DL_OK;
}

// x: bf16 [M, K] rows x_stride apart, 1 <= M <= 128.  w: bf16, contiguous rows of K.
// flags bit 0 (gated) clear: w is [N, K], out [M, N].  Set: w is [2N, K] (N gate rows, then N up
// rows), out [M, N] = silu(x Wg^T) * (x Wu^T).
// flags bit 1 (resident weights): the caller vouches that nothing still pending on the stream
// writes w, so the kernel may start reading w before the kernel launched before it has finished.
// gain / scaled / sumsq_out and sumsq_in / n_parts / inv_n / eps: the fusions described at the top
// (all null: a plain product); sums are laid out [part of 128 columns][128] floats.
// partials / counters: scratch of the sizes dl_gemm_decode_tc_scratch gives; status: int32, set
// non-zero if a wait expired.
extern "C" int dl_gemm_decode_tc_bf16(const void* x, int x_stride, const void* w, void* out, int out_dtype, int out_stride, int M,
                                      int N, int K, int flags, const float* gain, void* scaled, int scaled_stride,
                                      float* sumsq_out, const float* sumsq_in, int n_parts, float inv_n, float eps,
                                      float* partials, long long partial_floats, int* counters, int n_counters, int* status,
                                      void* stream) {
    const int gated = flags & 1, early = (flags >> 1) & 1;
    DL_REQUIRE((flags & ~3) == 0, "gemm_decode_tc: unknown flags %d", flags);
    DL_REQUIRE(M >= 1 && M <= GD_MAX_ROWS, "gemm_decode_tc: takes 1 to %d rows, got %d", GD_MAX_ROWS, M);
    DL_REQUIRE(N > 0 && K > 0 && K % 8 == 0, "gemm_decode_tc: K=%d must be a positive multiple of 8", K);
    DL_REQUIRE(x_stride % 8 == 0 && x_stride >= K, "gemm_decode_tc: row stride of x (%d) must be a multiple of 8", x_stride);
    DL_REQUIRE(((uintptr_t)x % 16) == 0 && ((uintptr_t)w % 16) == 0, "gemm_decode_tc: x and W must be 16-byte aligned");
    DL_REQUIRE(out_stride >= N, "gemm_decode_tc: out stride shorter than N");
    DL_REQUIRE(out_dtype == DL_F32 || out_dtype == DL_BF16, "gemm_decode_tc: out dtype %d", out_dtype);
    DL_REQUIRE(status != nullptr && partials != nullptr && counters != nullptr, "gemm_decode_tc: needs scratch and a status word");
    DL_REQUIRE(((uintptr_t)partials % 16) == 0, "gemm_decode_tc: the partial sums must be 16-byte aligned");
    GdFuse fuse{};
    if (gain != nullptr) {
        DL_REQUIRE(out_dtype == DL_F32 && !gated, "gemm_decode_tc: adding into the stream needs a plain float32 product");
        DL_REQUIRE(scaled != nullptr && sumsq_out != nullptr && scaled_stride >= N, "gemm_decode_tc: the scaled copy and the sums need a place");
        fuse.gain = gain, fuse.scaled = (__nv_bfloat16*)scaled, fuse.scaled_stride = scaled_stride, fuse.sumsq_out = sumsq_out;
    }
    if (sumsq_in != nullptr) {
        DL_REQUIRE(n_parts > 0 && inv_n > 0.f && eps >= 0.f, "gemm_decode_tc: row factors need parts, a width and an eps");
        fuse.sumsq_in = sumsq_in, fuse.n_parts = n_parts, fuse.inv_n = inv_n, fuse.eps = eps;
    }
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        return dl_fail(DL_ERR_LAUNCH, "gemm_decode_tc: cannot query the device");
    const GdPlan p = gd_plan(N, K, gated, sms);
    DL_REQUIRE(partial_floats >= (long long)p.blocks * 2 * gd_buf_cols(M, p.mode) * GD_BM && n_counters >= p.tiles,
               "gemm_decode_tc: scratch too small (%lld floats, %d counters)", partial_floats, n_counters);
    cudaStream_t s = (cudaStream_t)stream;
#define GD_CASE(MODEV)                                                                                                            \
    if (p.mode == MODEV) {                                                                                                        \
        if (out_dtype == DL_F32)                                                                                                  \
            return gd_launch<float, MODEV>(p, s, x, x_stride, w, out, out_stride, M, N, K, early, partials, counters, status, fuse); \
        return gd_launch<__nv_bfloat16, MODEV>(p, s, x, x_stride, w, out, out_stride, M, N, K, early, partials, counters, status, fuse); \
    }
    GD_CASE(GD_PLAIN) GD_CASE(GD_GATED)
#undef GD_CASE
    return dl_fail(DL_ERR_UNSUPPORTED, "gemm_decode_tc: mode %d", p.mode);
}
