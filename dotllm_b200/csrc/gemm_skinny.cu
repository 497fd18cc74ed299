// y = x W^T for a handful of rows of x (decode steps): a weight-streaming product.
//
// With M <= 16 rows every projection is bound by the bytes of W, read once.  The reference runs
// these through cuBLAS or one-block-per-output-row GEMV kernels
// (src/DotLLM.Cuda/CudaTransformerModel.cs:317-349, native/kernels/quantized_gemv.cu:13-63).
// Here W is the 16-row operand of mma.sync.m16n8k16 and the tokens are its 8 columns: within a
// 32-wide slice of k, lane (g, t) holds k = 8t..8t+7 of rows g and g+8 and the same slice of token
// g's activations, which is a consistent permutation of k for both operands of two MMAs.
//
// Shape: persistent, warp-specialised, stream-K.  The work is the list of (16-row tile, 256-wide
// chunk of k) pairs in tile-major order, cut into equal contiguous shares, one per consumer warp of
// the whole grid, so every warp streams the same number of bytes whatever N and K are.  One producer
// warp per block (lane c serving consumer warp c) copies chunks as tiled boxes of a tensor map over W
// (cp.async.bulk.tensor.2d, 16 rows by 256 k) into a private ring of shared-memory stages for each
// consumer warp, signalling an mbarrier per stage; copies run ahead of the arithmetic by the depth
// of the ring.  A consumer never synchronises with another warp of
// its block.  A tile that lies wholly inside one share is finished by that warp; a tile cut between
// shares is summed, in share order, by whichever of its warps arrives last, so the result is
// deterministic and does not depend on the number of rows of x.  With FUSE_SWIGLU a tile's rows
// 0-7 are gate rows and rows 8-15 the matching up rows, and the epilogue writes silu(gate) * up
// (native/kernels/swiglu.cu:7-41).
//
//
// Two optional fusions take the add + RMSNorm between two products of a decode step into the products
// themselves (the reference's fused_add_rmsnorm, native/kernels/fused_add_rmsnorm.cu:9-72, is a kernel
// of its own).  A float32 product with `gain` set adds its result into the float32 residual stream it
// is given as `out`, writes the sum times the norm's gain as bfloat16 (`scaled`) and the sum of squares
// of every 16-column tile and row (`sumsq_out`).  The product that follows takes `scaled` as its x
// and `sumsq_in`: a warp of its own adds the tiles' sums in tile order, and every output row is
// multiplied by rsqrt(sum / n + eps) in the epilogue - x W^T of the normalised row, since the
// normalisation is one factor per row.  All of it in float32 and in a fixed order.
//
// Every wait on an mbarrier is bounded (about a second of clock cycles); on expiry the kernel records
// a code in `status` and returns after waiting (bounded) for copies in flight.
#include "common.cuh"
#include "tma.cuh"
#include <mutex>
#include <type_traits>
#include <unordered_map>

#ifndef GS_CONSUMERS
#define GS_CONSUMERS 6
#endif
#ifndef GS_SLOTS
#define GS_SLOTS 4                         // ring stages per consumer warp
#endif
#define GS_BK 256                          // k per chunk
#define GS_STAGE_ELEMS (16 * GS_BK)         // a stage is the dense box the copy engine writes: [16 rows][256 k]
#define GS_THREADS (32 * (GS_CONSUMERS + 2))   // consumers, the producer warp, the row-statistics warp
#define GS_WAIT_CYCLES (1ll << 31)
#define GS_MAX_ROWS 16

__device__ __forceinline__ void gs_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t gs_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void gs_mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(gs_smem(bar)), "r"(count));
}
__device__ __forceinline__ void gs_mbar_expect(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(gs_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void gs_mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(gs_smem(bar)) : "memory");
}
__device__ __forceinline__ bool gs_mbar_try(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(gs_smem(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool gs_mbar_wait(uint64_t* bar, uint32_t parity, volatile int* gave_up) {
    if (gs_mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
    while (!gs_mbar_try(bar, parity)) {
        if (*gave_up || clock64() - t0 > GS_WAIT_CYCLES) return false;
    }
    return true;
}
__device__ __forceinline__ uint4 gs_lds128(uint32_t addr) {     // 16 bytes from a shared-space byte address
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}

template <typename TOut> __device__ __forceinline__ void gs_store(TOut* p, float v);
template <> __device__ __forceinline__ void gs_store<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void gs_store<__nv_bfloat16>(__nv_bfloat16* p, float v) {
    *p = __float2bfloat16_rn(v);
}

// The optional fusions of a launch (all pointers null: a plain product).
struct GsFuse {
    const float* gain;          // set: out is the float32 residual stream, out += x W^T in place, and ...
    __nv_bfloat16* scaled;      // ... scaled[m][n] = bf16(out[m][n] * gain[n]), rows scaled_stride apart,
    int scaled_stride;
    float* sumsq_out;           // ... sumsq_out[tile * 16 + m] = sum over the tile's 16 columns of out[m][n]^2
    const float* sumsq_in;      // set: output row m is multiplied by rsqrt(sum_p sumsq_in[p * 16 + m] * inv_n + eps)
    int n_parts;
    float inv_n, eps;
};

// acc[j] = {(row g, tok 2t), (row g, tok 2t+1), (row g+8, tok 2t), (row g+8, tok 2t+1)} of 8-token group j
// `row_scale`: null, or the factor of every output row (token).  `fuse.gain` (float32 plain products
// only): add into `out` and leave the scaled copy and the tile's sums of squares for the next product.
template <int NT, typename TOut, bool FUSE_SWIGLU>
__device__ __forceinline__ void gs_epilogue(const float (&acc_in)[NT][4], TOut* out, int out_stride, int tile, int M,
                                            int N, int g, int t, const float* row_scale, const GsFuse& fuse,
                                            const float (&stream_in)[NT][4], const float (&gain_in)[2]) {
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const int tok0 = j * 8 + 2 * t;
        float acc[4] = {acc_in[j][0], acc_in[j][1], acc_in[j][2], acc_in[j][3]};
        if (row_scale != nullptr) {
            const float s0 = row_scale[tok0], s1 = row_scale[tok0 + 1];
            acc[0] *= s0, acc[1] *= s1, acc[2] *= s0, acc[3] *= s1;
        }
        if (FUSE_SWIGLU) {
            const int col = tile * 8 + g;
            if (col < N) {
                const float g0 = acc[0], g1 = acc[1];
                if (tok0 < M) gs_store<TOut>(out + (size_t)tok0 * out_stride + col, g0 * (1.0f / (1.0f + expf(-g0))) * acc[2]);
                if (tok0 + 1 < M) gs_store<TOut>(out + (size_t)(tok0 + 1) * out_stride + col, g1 * (1.0f / (1.0f + expf(-g1))) * acc[3]);
            }
        } else if (std::is_same<TOut, float>::value && fuse.gain != nullptr) {
            float* stream = reinterpret_cast<float*>(out);
            float ss[2] = {0.f, 0.f};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int row = tile * 16 + g + (e >> 1) * 8, tok = tok0 + (e & 1);
                if (row < N && tok < M) {
                    const float h = stream_in[j][e] + acc[e];
                    stream[(size_t)tok * out_stride + row] = h;
                    fuse.scaled[(size_t)tok * fuse.scaled_stride + row] = __float2bfloat16_rn(h * gain_in[e >> 1]);
                    ss[e & 1] = fmaf(h, h, ss[e & 1]);
                }
            }
            // the tile's 16 columns of a token lie in the 8 lanes that share t: add them in a fixed order
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                ss[e] += __shfl_xor_sync(0xffffffffu, ss[e], 4);
                ss[e] += __shfl_xor_sync(0xffffffffu, ss[e], 8);
                ss[e] += __shfl_xor_sync(0xffffffffu, ss[e], 16);
                if (g == 0 && tok0 + e < M) fuse.sumsq_out[(size_t)tile * 16 + tok0 + e] = ss[e];
            }
        } else {
            const int row_lo = tile * 16 + g, row_hi = row_lo + 8;
            if (row_lo < N) {
                if (tok0 < M) gs_store<TOut>(out + (size_t)tok0 * out_stride + row_lo, acc[0]);
                if (tok0 + 1 < M) gs_store<TOut>(out + (size_t)(tok0 + 1) * out_stride + row_lo, acc[1]);
            }
            if (row_hi < N) {
                if (tok0 < M) gs_store<TOut>(out + (size_t)tok0 * out_stride + row_hi, acc[2]);
                if (tok0 + 1 < M) gs_store<TOut>(out + (size_t)(tok0 + 1) * out_stride + row_hi, acc[3]);
            }
        }
    }
}

// Built with -DGS_TIMELINE (DOTLLM_NVCC_EXTRA), every warp stamps the global nanosecond timer at six
// points of a launch into gs_timeline, which dl_gemm_skinny_timeline copies out
// (`python -m dotllm_b200.kernels.microbench gemm_skinny --timeline` prints the spread over the grid).
#ifdef GS_TIMELINE
__device__ long long gs_timeline[6][2048];       // [event][block * (GS_CONSUMERS + 2) + warp]
__device__ __forceinline__ long long gs_now() {
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define GS_STAMP(ev)                                                                                                     \
    do {                                                                                                                 \
        const int slot__ = blockIdx.x * (GS_CONSUMERS + 2) + (threadIdx.x >> 5);                                          \
        if ((threadIdx.x & 31) == 0 && slot__ < 2048) gs_timeline[ev][slot__] = gs_now();                                 \
    } while (0)
extern "C" int dl_gemm_skinny_timeline(long long* out) {
    return cudaMemcpyFromSymbol(out, gs_timeline, sizeof(gs_timeline)) == cudaSuccess ? DL_OK : DL_ERR_LAUNCH;
}
#else
#define GS_STAMP(ev)
#endif

// The product of a launch: its operands and how its chunks are cut (see GsPlan below).
struct GsWork {
    const __nv_bfloat16* x;
    int x_stride;
    void* out;
    int out_stride;
    int M, N, K, up_offset, cpt, total_chunks, share;
    GsFuse fuse;
};

// The rings of a block: a private ring of GS_SLOTS stages per consumer warp.
struct GsRings {
    __nv_bfloat16* stage_mem;                               // [consumer][slot][16][GS_BK]
    uint64_t (*full_bar)[GS_SLOTS];
    uint64_t (*empty_bar)[GS_SLOTS];
    volatile int* gave_up;
    int* status;
    uint64_t* scale_bar;                                    // completes when row_scale is written
    const float* row_scale;                                 // [16] factors of the output rows (sumsq_in)
};

// Producer lane `lane` (< GS_CONSUMERS) feeds consumer warp `lane`: it walks that warp's share chunk
// by chunk, waits for the ring slot to be free, and issues one tiled copy (two for gate + up) per
// chunk.  `cnt` counts the chunks of this ring.  False: gave up.
template <bool FUSE_SWIGLU>
__device__ __forceinline__ bool gs_produce(const CUtensorMap* tmap, const GsWork& w, const GsRings& r, int lane, int& cnt) {
    const int gw = blockIdx.x * GS_CONSUMERS + lane;
    int cur = min(w.total_chunks, gw * w.share);
    const int end = min(w.total_chunks, (gw + 1) * w.share);
    const uint64_t policy = dl_stream_policy();             // W is read once a step: first out of the L2
    for (; cur < end; ++cur, ++cnt) {
        const int slot = cnt % GS_SLOTS;
        if (cnt >= GS_SLOTS && !gs_mbar_wait(&r.empty_bar[lane][slot], ((cnt / GS_SLOTS) - 1) & 1, r.gave_up)) {
            if (!*r.gave_up) atomicExch(r.status, 1);
            *r.gave_up = 1;
            return false;
        }
        const int tile = cur / w.cpt, kc = cur - tile * w.cpt;
        __nv_bfloat16* dst = r.stage_mem + (size_t)(lane * GS_SLOTS + slot) * GS_STAGE_ELEMS;
        // a box is always written whole: parts outside the matrix arrive as zeros
        gs_mbar_expect(&r.full_bar[lane][slot], GS_STAGE_ELEMS * 2);
        if (FUSE_SWIGLU) {
            dl_tma_load_2d_hint(dst, tmap, kc * GS_BK, tile * 8, &r.full_bar[lane][slot], policy);
            dl_tma_load_2d_hint(dst + 8 * GS_BK, tmap, kc * GS_BK, w.up_offset + tile * 8, &r.full_bar[lane][slot], policy);
        } else {
            dl_tma_load_2d_hint(dst, tmap, kc * GS_BK, tile * 16, &r.full_bar[lane][slot], policy);
        }
    }
    return true;
}

// After giving up: copies already issued must land before the block's shared memory is released.
__device__ __forceinline__ void gs_drain(const GsRings& r, int lane, int cnt) {
    for (int i = max(0, cnt - GS_SLOTS); i < cnt; ++i) {
        const long long t0 = clock64();
        while (!gs_mbar_try(&r.full_bar[lane][i % GS_SLOTS], (i / GS_SLOTS) & 1) && clock64() - t0 < GS_WAIT_CYCLES) {}
    }
}

// Consumer warp `warp` works through its share of the product.  `cnt` counts the chunks of its ring;
// `dead` is set when a wait expired.
template <int NT, typename TOut, bool FUSE_SWIGLU>
__device__ __forceinline__ void gs_consume(const GsWork& w, const GsRings& r, float* __restrict__ partials,
                                           int* __restrict__ counters, int warp, int lane, int& cnt, bool& dead) {
    const int g = lane >> 2, t = lane & 3;
    const int gw = blockIdx.x * GS_CONSUMERS + warp;
    const int begin = min(w.total_chunks, gw * w.share), end = min(w.total_chunks, (gw + 1) * w.share);
    const int cpt = w.cpt, share = w.share, M = w.M, N = w.N, K = w.K;
    const __nv_bfloat16* x = w.x;
    TOut* out = reinterpret_cast<TOut*>(w.out);
    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;
    const float* row_scale = nullptr;                    // set once the statistics warp has written the factors
    // The stream's values and the gains of the tile at hand, asked for when the tile begins so that the
    // epilogue does not wait for them (only this tile's finishing warp ever writes them).
    float stream_in[NT][4], gain_in[2] = {0.f, 0.f};
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) stream_in[j][e] = 0.f;
    int stream_tile = -1;
    int seg_begin = begin;                               // first chunk of the current tile's segment
    for (int cur = begin; cur < end; ++cur, ++cnt) {
        const int slot = cnt % GS_SLOTS;
        const int tile = cur / cpt, kc = cur - tile * cpt;
        const int k0 = kc * GS_BK;
        if (std::is_same<TOut, float>::value && !FUSE_SWIGLU && w.fuse.gain != nullptr && tile != stream_tile) {
            stream_tile = tile;
            const float* stream = reinterpret_cast<const float*>(w.out);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int row = tile * 16 + g + 8 * h;
                gain_in[h] = row < N ? __ldg(w.fuse.gain + row) : 0.f;
#pragma unroll
                for (int j = 0; j < NT; ++j)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int tok = j * 8 + 2 * t + e;
                        stream_in[j][2 * h + e] = (row < N && tok < M) ? __ldcg(stream + (size_t)tok * w.out_stride + row) : 0.f;
                    }
            }
        }
        // activations of this chunk, asked for before waiting on the weights
        uint4 xf[GS_BK / 32][NT];
#pragma unroll
        for (int s = 0; s < GS_BK / 32; ++s)
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const int tok = j * 8 + g, k = k0 + 32 * s + 8 * t;
                xf[s][j] = make_uint4(0u, 0u, 0u, 0u);
                if (tok < M && k < K) xf[s][j] = __ldg(reinterpret_cast<const uint4*>(x + (size_t)tok * w.x_stride + k));
            }
        if (!dead && !gs_mbar_wait(&r.full_bar[warp][slot], (cnt / GS_SLOTS) & 1, r.gave_up)) {
            if (!*r.gave_up) atomicExch(r.status, 3);
            *r.gave_up = 1;
            dead = true;
        }
        if (cur == begin) GS_STAMP(2);                        // the first chunk of the share has landed
        if (!dead) {
            // this lane's byte address in shared space; the loads below are constant offsets away.
            // Rows beyond the matrix and k beyond K arrived as zeros, so nothing needs guarding.
            const uint32_t st = gs_smem(r.stage_mem + (size_t)(warp * GS_SLOTS + slot) * GS_STAGE_ELEMS) +
                                (uint32_t)(g * GS_BK + 8 * t) * 2u;
#pragma unroll
            for (int s = 0; s < GS_BK / 32; ++s) {
                const uint4 a_lo = gs_lds128(st + (uint32_t)(32 * s * 2));
                const uint4 a_hi = gs_lds128(st + (uint32_t)((8 * GS_BK + 32 * s) * 2));
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    gs_mma(acc[j], a_lo.x, a_hi.x, a_lo.y, a_hi.y, xf[s][j].x, xf[s][j].y);
                    gs_mma(acc[j], a_lo.z, a_hi.z, a_lo.w, a_hi.w, xf[s][j].z, xf[s][j].w);
                }
            }
            // The slot may be released only after every MMA fed from it has been issued (an MMA issues
            // when its operands have arrived from shared memory; a released slot is overwritten by the
            // next copy at once).  The MMAs are not volatile, so pin their results here: the compiler
            // cannot sink them below this point.
#pragma unroll
            for (int j = 0; j < NT; ++j) asm volatile("" : "+f"(acc[j][0]), "+f"(acc[j][1]), "+f"(acc[j][2]), "+f"(acc[j][3]));
            // ... and the reads themselves must be done before the copy engine may overwrite the stage:
            // without this fence a slot that was refilled at once showed rows of the new chunk to the old reads.
            __threadfence_block();
            __syncwarp();
            if (lane == 0) gs_mbar_arrive(&r.empty_bar[warp][slot]);
        }
        if (cur == end - 1) GS_STAMP(3);                      // the last chunk of the share is consumed
        if (kc == cpt - 1 || cur == end - 1) {
            // ---- the segment [seg_begin, cur] of this tile is done
            const bool whole = (seg_begin == tile * cpt) && (kc == cpt - 1);
            if (w.fuse.sumsq_in != nullptr && row_scale == nullptr && !dead) {
                // the factors of the rows: written by the statistics warp long before the first tile ends
                if (!gs_mbar_wait(r.scale_bar, 0, r.gave_up)) {
                    if (!*r.gave_up) atomicExch(r.status, 5);
                    *r.gave_up = 1;
                    dead = true;
                } else {
                    row_scale = r.row_scale;
                }
            }
            if (whole) {
                gs_epilogue<NT, TOut, FUSE_SWIGLU>(acc, out, w.out_stride, tile, M, N, g, t, row_scale, w.fuse, stream_in, gain_in);
            } else {
                // a warp's first tile may be shared with the share before, its last with the share after
                const int which = (tile == begin / cpt) ? 0 : 1;
                float* mine = partials + ((size_t)gw * 2 + which) * (NT * 4 * 32);
#pragma unroll
                for (int j = 0; j < NT; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) mine[(j * 4 + e) * 32 + lane] = acc[j][e];
                __syncwarp();
                const int g_lo = (tile * cpt) / share, g_hi = ((tile + 1) * cpt - 1) / share;
                int last = 0;
                if (lane == 0) {
                    // One read-modify-write that releases this warp's part (the lanes' stores are ordered
                    // before it by the __syncwarp above) and acquires the parts of the warps counted before.
                    int seen;
                    asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(seen) : "l"(counters + tile) : "memory");
                    last = (seen == g_hi - g_lo) ? 1 : 0;
                    if (last) counters[tile] = 0;        // ready for the next product or launch
                }
                last = __shfl_sync(0xffffffffu, last, 0);
                __syncwarp();                            // the other lanes' reads below come after lane 0's acquire
                if (last) {
#pragma unroll
                    for (int j = 0; j < NT; ++j)
#pragma unroll
                        for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;
                    for (int gg = g_lo; gg <= g_hi; ++gg) {          // share order: fixed
                        const int wh = (tile == (gg * share) / cpt) ? 0 : 1;
                        const float* theirs = partials + ((size_t)gg * 2 + wh) * (NT * 4 * 32);
#pragma unroll
                        for (int j = 0; j < NT; ++j)
#pragma unroll
                            for (int e = 0; e < 4; ++e) acc[j][e] += __ldcg(theirs + (j * 4 + e) * 32 + lane);
                    }
                    gs_epilogue<NT, TOut, FUSE_SWIGLU>(acc, out, w.out_stride, tile, M, N, g, t, row_scale, w.fuse, stream_in, gain_in);
                }
            }
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;
            seg_begin = cur + 1;
        }
    }
}

#define GS_INIT_RINGS()                                                                                  \
    extern __shared__ __align__(128) unsigned char gs_smem_raw[];                                        \
    __shared__ uint64_t full_bar[GS_CONSUMERS][GS_SLOTS], empty_bar[GS_CONSUMERS][GS_SLOTS];             \
    __shared__ volatile int gave_up;                                                                     \
    __shared__ uint64_t scale_bar;                                                                       \
    __shared__ float row_scale_smem[GS_MAX_ROWS];                                                        \
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;                                          \
    if (threadIdx.x == 0) {                                                                              \
        gave_up = 0;                                                                                     \
        gs_mbar_init(&scale_bar, 1);                                                                     \
        for (int c = 0; c < GS_CONSUMERS; ++c)                                                           \
            for (int s = 0; s < GS_SLOTS; ++s) {                                                         \
                gs_mbar_init(&full_bar[c][s], 1);                                                        \
                gs_mbar_init(&empty_bar[c][s], 1);                                                       \
            }                                                                                            \
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");                               \
    }                                                                                                    \
    __syncthreads();                                                                                     \
    dl_launch_dependents();                                                                              \
    const GsRings rings{reinterpret_cast<__nv_bfloat16*>(gs_smem_raw), full_bar, empty_bar, &gave_up, status, &scale_bar,  \
                        row_scale_smem}

template <int NT, typename TOut, bool FUSE_SWIGLU>
__global__ void __launch_bounds__(GS_THREADS, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmap, const GsWork work, int early_weights,
                   float* __restrict__ partials, int* __restrict__ counters, int* __restrict__ status) {
    GS_STAMP(0);                                              // block started
    GS_INIT_RINGS();
    GS_STAMP(1);                                              // barriers ready
    if (warp == GS_CONSUMERS) {
        // ------------------------------------------------------------ producer warp
        // When the caller vouches that no pending work writes the weights (early_weights), the
        // producer does not wait for the kernel before this one: while that kernel finishes, the
        // rings fill.
        if (!early_weights) dl_grid_dependency_wait();
        if (lane < GS_CONSUMERS) {
            int cnt = 0;
            if (!gs_produce<FUSE_SWIGLU>(&tmap, work, rings, lane, cnt)) gs_drain(rings, lane, cnt);
        }
    } else if (warp == GS_CONSUMERS + 1) {
        // ------------------------------------------------------------ row-statistics warp
        if (work.fuse.sumsq_in != nullptr) {
            dl_grid_dependency_wait();   // the sums come from the kernel before this one
            // A warp-wide float4 load covers 8 parts x 16 rows: lane -> (rows 4q .. 4q+3, part l/4 of
            // every 8).  All loads of a batch are in flight together; a lane adds its parts in part
            // order, then the 8 lanes of a row group are added in a fixed order: the same bits on
            // every launch.
            const int q = lane & 3, sub = lane >> 2;
            const float4* in = reinterpret_cast<const float4*>(work.fuse.sumsq_in) + q;
            float4 acc4 = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int p0 = 0; p0 < work.fuse.n_parts; p0 += 8 * 16) {
                float4 v[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int p = p0 + 8 * i + sub;
                    v[i] = p < work.fuse.n_parts ? __ldcg(in + (size_t)p * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
                for (int i = 0; i < 16; ++i) acc4.x += v[i].x, acc4.y += v[i].y, acc4.z += v[i].z, acc4.w += v[i].w;
            }
#pragma unroll
            for (int o = 4; o < 32; o <<= 1) {
                // both partners add (lower lane's value) + (higher lane's value)
                const float4 other = make_float4(__shfl_xor_sync(0xffffffffu, acc4.x, o), __shfl_xor_sync(0xffffffffu, acc4.y, o),
                                                 __shfl_xor_sync(0xffffffffu, acc4.z, o), __shfl_xor_sync(0xffffffffu, acc4.w, o));
                const bool low = (lane & o) == 0;
                acc4.x = low ? acc4.x + other.x : other.x + acc4.x;
                acc4.y = low ? acc4.y + other.y : other.y + acc4.y;
                acc4.z = low ? acc4.z + other.z : other.z + acc4.z;
                acc4.w = low ? acc4.w + other.w : other.w + acc4.w;
            }
            if (lane < 4) {
                row_scale_smem[4 * lane + 0] = rsqrtf(acc4.x * work.fuse.inv_n + work.fuse.eps);
                row_scale_smem[4 * lane + 1] = rsqrtf(acc4.y * work.fuse.inv_n + work.fuse.eps);
                row_scale_smem[4 * lane + 2] = rsqrtf(acc4.z * work.fuse.inv_n + work.fuse.eps);
                row_scale_smem[4 * lane + 3] = rsqrtf(acc4.w * work.fuse.inv_n + work.fuse.eps);
            }
            __threadfence_block();
            __syncwarp();
            if (lane == 0) gs_mbar_arrive(&scale_bar);
        }
    } else {
        // ------------------------------------------------------------ consumer warp
        dl_grid_dependency_wait();       // x comes from the kernel before this one; out, partials and counters may be in use by it
        int cnt = 0;
        bool dead = false;
        gs_consume<NT, TOut, FUSE_SWIGLU>(work, rings, partials, counters, warp, lane, cnt, dead);
        GS_STAMP(4);                                          // share done, hand-over of cut tiles included
    }
    __syncthreads();                                         // nobody leaves while copies may still land
    GS_STAMP(5);
}

// How the work of an (N, K) matrix is cut: tiles of 16 rows (8 gate + 8 up when gated), chunks per
// tile, blocks, chunks per consumer warp.  Depends on the matrix and the device only, never on M.
struct GsPlan {
    int tiles, cpt, total, blocks, share;
};

static GsPlan gs_plan(int N, int K, int fuse_swiglu, int sms) {
    GsPlan p;
    p.tiles = fuse_swiglu ? (N + 7) / 8 : (N + 15) / 16;
    p.cpt = (K + GS_BK - 1) / GS_BK;
    p.total = p.tiles * p.cpt;
    const int per_block = GS_CONSUMERS * 4;                  // at least about four chunks per warp
    p.blocks = (p.total + per_block - 1) / per_block;
    if (p.blocks > sms) p.blocks = sms;
    if (p.blocks < 1) p.blocks = 1;
    const int warps = p.blocks * GS_CONSUMERS;
    p.share = (p.total + warps - 1) / warps;
    return p;
}

// Scratch the product needs: float32 partial sums and int32 arrival counters (zero before the first
// launch; every launch leaves them zero).
extern "C" int dl_gemm_skinny_scratch(int M, int N, int K, int fuse_swiglu, int sms, int* partial_floats,
                                      int* n_counters) {
    const GsPlan p = gs_plan(N, K, fuse_swiglu, sms);
    const int nt = M <= 8 ? 1 : 2;
    *partial_floats = p.blocks * GS_CONSUMERS * 2 * nt * 4 * 32;
    *n_counters = p.tiles;
    return DL_OK;
}

// Tensor map of W: rows of K bfloat16, boxes of 16 rows (8 for gate + up) by 256 columns.  Encoding
// costs a driver call, so maps are kept per (matrix, shape).
struct GsMapKey {
    const void* w;
    int rows, k, box;
    bool operator==(const GsMapKey& o) const { return w == o.w && rows == o.rows && k == o.k && box == o.box; }
};
struct GsMapKeyHash {
    size_t operator()(const GsMapKey& k) const {
        return std::hash<const void*>()(k.w) ^ ((size_t)k.rows * 1000003u) ^ ((size_t)k.k * 10007u) ^ (size_t)k.box;
    }
};

static int gs_weight_map(CUtensorMap* out, const void* w, int N, int K, bool gated) {
    static std::unordered_map<GsMapKey, CUtensorMap, GsMapKeyHash> maps;
    static std::mutex maps_mutex;
    const int rows = gated ? 2 * N : N, box = gated ? 8 : 16;
    std::lock_guard<std::mutex> lock(maps_mutex);
    const GsMapKey key{w, rows, K, box};
    auto it = maps.find(key);
    if (it == maps.end()) {
        CUtensorMap fresh;
        if (dl_tmap_encode_2d_bf16(&fresh, w, (uint64_t)rows, (uint64_t)K, (uint64_t)K * 2, box, GS_BK, DL_TMAP_SWIZZLE_NONE) != 0)
            return DL_ERR_LAUNCH;
        if (maps.size() > 4096) maps.clear();
        it = maps.emplace(key, fresh).first;
    }
    *out = it->second;
    return DL_OK;
}

template <int NT, typename TOut, bool FUSE>
static int gs_launch(const GsPlan& p, cudaStream_t s, const __nv_bfloat16* x, int x_stride, const __nv_bfloat16* w,
                     void* out, int out_stride, int M, int N, int K, int up_offset, int early_weights, float* partials,
                     int* counters, int* status, const GsFuse& fuse) {
    const size_t smem = (size_t)GS_CONSUMERS * GS_SLOTS * GS_STAGE_ELEMS * 2;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_skinny_kernel<NT, TOut, FUSE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "gemm_skinny: shared memory %zu: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    CUtensorMap tmap;
    const int rc = gs_weight_map(&tmap, w, N, K, FUSE);
    if (rc != DL_OK) return rc;
    const GsWork work{x, x_stride, out, out_stride, M, N, K, up_offset, p.cpt, p.total, p.share, fuse};
    cudaError_t le = dl_launch_dependent(gemm_skinny_kernel<NT, TOut, FUSE>, dim3(p.blocks), dim3(GS_THREADS), smem, s, tmap, work,
                                         early_weights, partials, counters, status);
    if (le != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "gemm_skinny: %s", cudaGetErrorString(le));
    return DL_OK;
}

// x: bf16 [M, K] rows x_stride apart, M <= 16.  w: bf16, contiguous rows of K.
// flags bit 0 (gated) clear: w is [N, K], out [M, N].  Set: w is [2N, K] (N gate rows, then N up
// rows), out [M, N] = silu(x Wg^T) * (x Wu^T).
// flags bit 1 (resident weights): the caller vouches that nothing still pending on the stream
// writes w, so the kernel may start reading w before the kernel launched before it has finished.
// partials / counters: scratch of the sizes dl_gemm_skinny_scratch gives; status: int32, set
// non-zero if a wait expired.
static int gs_run(const void* x, int x_stride, const void* w, void* out, int out_dtype, int out_stride, int M, int N, int K,
                  int flags, float* partials, int partial_floats, int* counters, int n_counters, int* status, void* stream,
                  const GsFuse& fuse) {
    const int fuse_swiglu = flags & 1, early = (flags >> 1) & 1;
    DL_REQUIRE((flags & ~3) == 0, "gemm_skinny: unknown flags %d", flags);
    DL_REQUIRE(M >= 1 && M <= GS_MAX_ROWS, "gemm_skinny: takes 1 to %d rows, got %d", GS_MAX_ROWS, M);
    DL_REQUIRE(N > 0 && K > 0 && K % 8 == 0, "gemm_skinny: K=%d must be a positive multiple of 8", K);
    DL_REQUIRE(x_stride % 8 == 0 && x_stride >= K, "gemm_skinny: row stride of x (%d) must be a multiple of 8", x_stride);
    DL_REQUIRE(((uintptr_t)x % 16) == 0 && ((uintptr_t)w % 16) == 0, "gemm_skinny: x and W must be 16-byte aligned");
    DL_REQUIRE(out_stride >= N, "gemm_skinny: out stride shorter than N");
    DL_REQUIRE(out_dtype == DL_F32 || out_dtype == DL_BF16, "gemm_skinny: out dtype %d", out_dtype);
    DL_REQUIRE(status != nullptr && partials != nullptr && counters != nullptr, "gemm_skinny: needs scratch and a status word");
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        return dl_fail(DL_ERR_LAUNCH, "gemm_skinny: cannot query the device");
    const GsPlan p = gs_plan(N, K, fuse_swiglu, sms);
    const int nt = M <= 8 ? 1 : 2;
    DL_REQUIRE(partial_floats >= p.blocks * GS_CONSUMERS * 2 * nt * 4 * 32 && n_counters >= p.tiles,
               "gemm_skinny: scratch too small (%d floats, %d counters)", partial_floats, n_counters);
    cudaStream_t s = (cudaStream_t)stream;
    const __nv_bfloat16* xb = (const __nv_bfloat16*)x;
    const __nv_bfloat16* wb = (const __nv_bfloat16*)w;
#define GS_CASE(NTV)                                                                                                   \
    if (nt == NTV) {                                                                                                   \
        if (fuse_swiglu) {                                                                                             \
            if (out_dtype == DL_F32) return gs_launch<NTV, float, true>(p, s, xb, x_stride, wb, out, out_stride, M, N, K, N, early, partials, counters, status, fuse); \
            return gs_launch<NTV, __nv_bfloat16, true>(p, s, xb, x_stride, wb, out, out_stride, M, N, K, N, early, partials, counters, status, fuse);                \
        }                                                                                                              \
        if (out_dtype == DL_F32) return gs_launch<NTV, float, false>(p, s, xb, x_stride, wb, out, out_stride, M, N, K, 0, early, partials, counters, status, fuse);    \
        return gs_launch<NTV, __nv_bfloat16, false>(p, s, xb, x_stride, wb, out, out_stride, M, N, K, 0, early, partials, counters, status, fuse);                   \
    }
    GS_CASE(1) GS_CASE(2)
#undef GS_CASE
    return dl_fail(DL_ERR_UNSUPPORTED, "gemm_skinny: %d rows", M);
}

extern "C" int dl_gemm_skinny_bf16(const void* x, int x_stride, const void* w, void* out, int out_dtype,
                                   int out_stride, int M, int N, int K, int flags, float* partials,
                                   int partial_floats, int* counters, int n_counters, int* status, void* stream) {
    return gs_run(x, x_stride, w, out, out_dtype, out_stride, M, N, K, flags, partials, partial_floats, counters, n_counters,
                  status, stream, GsFuse{});
}

// The same with the fusions of an add + RMSNorm between two products (either, both or neither):
// gain set (float32 [N]; out must be float32 and the product plain): out is the float32 residual
//   stream and is added to in place; scaled bf16 [M, N] (rows scaled_stride apart) receives
//   out * gain, sumsq_out float32 [ceil(N / 16) * 16] the sum of squares per 16-column tile and row.
// sumsq_in set (float32 [n_parts * 16], as a product before this one left it): every output row m
//   is multiplied by rsqrt(sum_p sumsq_in[p * 16 + m] / n + eps), n = 1 / inv_n the width of x's norm.
extern "C" int dl_gemm_skinny_fused_bf16(const void* x, int x_stride, const void* w, void* out, int out_dtype,
                                         int out_stride, int M, int N, int K, int flags, const float* gain, void* scaled,
                                         int scaled_stride, float* sumsq_out, const float* sumsq_in, int n_parts, float inv_n,
                                         float eps, float* partials, int partial_floats, int* counters, int n_counters,
                                         int* status, void* stream) {
    GsFuse fuse{};
    if (gain != nullptr) {
        DL_REQUIRE(out_dtype == DL_F32 && (flags & 1) == 0, "gemm_skinny: adding into the stream needs a plain float32 product");
        DL_REQUIRE(scaled != nullptr && sumsq_out != nullptr && scaled_stride >= N, "gemm_skinny: the scaled copy and the sums need a place");
        fuse.gain = gain, fuse.scaled = (__nv_bfloat16*)scaled, fuse.scaled_stride = scaled_stride, fuse.sumsq_out = sumsq_out;
    }
    if (sumsq_in != nullptr) {
        DL_REQUIRE(n_parts > 0 && inv_n > 0.f && eps >= 0.f, "gemm_skinny: row factors need parts, a width and an eps");
        fuse.sumsq_in = sumsq_in, fuse.n_parts = n_parts, fuse.inv_n = inv_n, fuse.eps = eps;
    }
    return gs_run(x, x_stride, w, out, out_dtype, out_stride, M, N, K, flags, partials, partial_floats, counters, n_counters,
                  status, stream, fuse);
}

// ---------------------------------------------------------------------------------------------
// The same product for callers that must not allocate (declared in gemm_skinny_static.h).
//
// dl_gemm_skinny_bf16 above takes its scratch from the caller, who normally gets it from an
// allocator.  Some callers have no allocator to ask: code that runs between a framework's
// allocation phases, a host process whose device memory is handed out once at start-up and then
// frozen, a real-time loop that may not take the allocator's lock.  For them the scratch lives in
// this library's own image: a file-scope __device__ array of a fixed, modest size that every GPU
// loading the library holds until the process exits.
//
// The array's name is only a host-side handle for the device object; its device address is asked
// for once per device, with that device current, through cudaGetSymbolAddress.
#include "gemm_skinny_static.h"

#define GS_STATIC_PARTIAL_FLOATS ((DL_GEMM_SKINNY_STATIC_SCRATCH_BYTES - 256) / 4 - DL_GEMM_SKINNY_STATIC_MAX_TILES)

struct GsStaticScratch {
    int status;
    int pad[63];
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
    DL_REQUIRE(M >= 1 && M <= GS_MAX_ROWS && N > 0 && K > 0, "gemm_skinny_static: bad sizes M=%d N=%d K=%d (1 to %d rows)", M, N,
               K, GS_MAX_ROWS);
    int sms = 0, dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        return dl_fail(DL_ERR_LAUNCH, "gemm_skinny_static: cannot query the device");
    int need_floats = 0, need_counters = 0;
    dl_gemm_skinny_scratch(M, N, K, fuse_swiglu, sms, &need_floats, &need_counters);
    if (need_counters > DL_GEMM_SKINNY_STATIC_MAX_TILES || need_floats > (int)GS_STATIC_PARTIAL_FLOATS)
        return dl_fail(DL_ERR_UNSUPPORTED,
                       "gemm_skinny_static: M=%d N=%d K=%d needs %d row tiles and %d scratch floats; the built-in "
                       "scratch holds %d tiles and %d floats - use dl_gemm_skinny_bf16 with your own scratch",
                       M, N, K, need_counters, need_floats, DL_GEMM_SKINNY_STATIC_MAX_TILES, (int)GS_STATIC_PARTIAL_FLOATS);
    GsStaticScratch* scratch = nullptr;
    const int rc = gs_static_address(&scratch);
    if (rc != DL_OK) return rc;
    // The array keeps whatever the last call left; the arrival counters must start at zero.
    cudaError_t e = cudaMemsetAsync(scratch->counters, 0, sizeof(int) * need_counters, (cudaStream_t)stream);
    if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "gemm_skinny_static: memset: %s", cudaGetErrorString(e));
    return dl_gemm_skinny_bf16(x, x_stride, w, out, out_dtype, out_stride, M, N, K, fuse_swiglu ? 1 : 0, scratch->partials,
                               need_floats, scratch->counters, need_counters, &scratch->status, stream);
}

// The give-up word of the static calls on the current device: copies it to *code (0: every wait so
// far was served) and clears it.  Waits for `stream` to drain, so that it speaks for every static
// call queued there before it; allocates nothing.
extern "C" int dl_gemm_skinny_static_status(int* code, void* stream) {
    DL_REQUIRE(code != nullptr, "gemm_skinny_static_status: needs a place for the code");
    GsStaticScratch* scratch = nullptr;
    const int rc = gs_static_address(&scratch);
    if (rc != DL_OK) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e = cudaMemcpyAsync(code, &scratch->status, sizeof(int), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e == cudaSuccess && *code != 0) e = cudaMemsetAsync(&scratch->status, 0, sizeof(int), s);
    if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "gemm_skinny_static_status: %s", cudaGetErrorString(e));
    return DL_OK;
}
