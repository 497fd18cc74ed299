// Decode attention: one new token per sequence over its paged bfloat16 cache, split over keys.
//
// Role of the reference's attention_f16 with seq_q == 1 (native/kernels/attention.cu:19-197): scores
// scaled by 1/sqrt(hd), softmax with the running maximum subtracted, weighted sum of values, query
// head h reading KV head h / group.  A decode step is bound by the bytes of K and V, so each
// (sequence, KV head) is cut into runs of pages that separate blocks stream, and all query heads
// of the group share every key and value that is loaded: the group's heads are the rows of
// mma.sync.m16n8k16 tiles (rows beyond the group are zero).
//
// Data path: a cache page of one KV head is two contiguous pieces (K [64][hd], V [hd][64]).  One
// producer thread copies them with cp.async.bulk (the bulk-copy engine) into a ring of shared-memory
// stages, signalling an mbarrier per stage; the copies run ahead of the arithmetic by the depth of
// the ring and cost no registers.  Four consumer warps work in two pairs: a pair takes every second
// page, each warp of the pair one half (32 keys) of it.
//
// Arithmetic: lane (g, t) reads 16-byte pieces of K rows: dims 8t..8t+7 of a 32-dim slice are a
// consistent permutation of k for Q and K in two MMAs; the 8 key columns of score tile j are keys
// 8(g/2) + 2j + (g&1) of the 32, so that after four tiles the lane holds scores of keys 8t..8t+7 -
// exactly the k-permutation that pairs with a 16-byte piece of a transposed V row.  Softmax is
// float32 with exact expf.  Warps of a block, then the blocks of a (sequence, KV head), are merged
// in a fixed order; the last block to finish does the merge and writes bfloat16.
//
// Every wait on an mbarrier is bounded (about a second of clock cycles); on expiry the kernel
// records a code in `status`, stops issuing copies, waits (bounded) for copies in flight, and
// returns.  The host reads `status` at its next synchronisation point.
#include "common.cuh"

#define AD_CONSUMERS 4
#define AD_THREADS (32 * (AD_CONSUMERS + 1))
#define AD_STAGES 3
#define AD_WAIT_CYCLES (1ll << 31)

__device__ __forceinline__ void ad_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t ad_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ uint32_t ad_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void ad_mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(ad_smem(bar)), "r"(count));
}
__device__ __forceinline__ void ad_mbar_expect(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(ad_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ad_mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(ad_smem(bar)) : "memory");
}
__device__ __forceinline__ bool ad_mbar_try(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(ad_smem(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: false when the barrier did not complete in time (or another thread gave up).
__device__ __forceinline__ bool ad_mbar_wait(uint64_t* bar, uint32_t parity, volatile int* gave_up) {
    if (ad_mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
    while (!ad_mbar_try(bar, parity)) {
        if (*gave_up || clock64() - t0 > AD_WAIT_CYCLES) return false;
    }
    return true;
}
__device__ __forceinline__ void ad_bulk_copy(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(ad_smem(dst)),
                 "l"(src), "r"(bytes), "r"(ad_smem(bar))
                 : "memory");
}

// Zero the bf16 elements of a 16-byte piece (keys first..first+7) outside [lo, hi).
__device__ __forceinline__ uint4 ad_keep_keys(uint4 v, int first, int lo, int hi) {
    uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int k0 = first + 2 * i;
        const bool a = k0 >= lo && k0 < hi, b = k0 + 1 >= lo && k0 + 1 < hi;
        if (!a && !b) w[i] = 0u;
        else if (!a) w[i] &= 0xffff0000u;
        else if (!b) w[i] &= 0x0000ffffu;
    }
    return v;
}

template <int HD>
__global__ void __launch_bounds__(AD_THREADS)
attention_decode_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, __nv_bfloat16* __restrict__ out,
                        int out_stride, const __nv_bfloat16* __restrict__ k_pool,
                        const __nv_bfloat16* __restrict__ v_pool, int n_pages,
                        const int32_t* __restrict__ seq_len, const int32_t* __restrict__ block_table,
                        int bt_stride, int nh, int nkv, float scale, int window, int keys_per_split,
                        float* __restrict__ part_o, float* __restrict__ part_ml, int* __restrict__ counters,
                        int* __restrict__ status) {
    constexpr int DC = HD / 32;          // 32-dim slices of a head
    constexpr int DT = HD / 8;           // 8-dim output tiles
    constexpr int PAGE_ELEMS = DL_PAGE * HD;
    constexpr uint32_t PAGE_BYTES = PAGE_ELEMS * 2;
    // stages: [K page | V page]; after the loop the same memory holds the warps' partial outputs
    extern __shared__ __align__(128) unsigned char ad_smem_raw[];
    __nv_bfloat16* stage_mem = reinterpret_cast<__nv_bfloat16*>(ad_smem_raw);
    float (*sm_o)[16][HD + 4] = reinterpret_cast<float (*)[16][HD + 4]>(ad_smem_raw);
    __shared__ uint64_t full_bar[AD_STAGES], empty_bar[AD_STAGES];
    __shared__ float sm_m[AD_CONSUMERS][16], sm_l[AD_CONSUMERS][16];
    __shared__ int is_last;
    __shared__ volatile int gave_up;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int group = nh / nkv;
    const int len = seq_len[b];                          // keys 0..len-1; the query sits at len-1
    const int first = (window > 0 && len - window > 0) ? len - window : 0;
    const int origin = (first / DL_PAGE) * DL_PAGE;      // runs start at the first visible key's page
    const int n_splits = (len - origin + keys_per_split - 1) / keys_per_split;
    if (split >= n_splits) return;
    const int run_begin = origin + split * keys_per_split;
    const int run_end = min(len, run_begin + keys_per_split);
    const int page0 = run_begin / DL_PAGE;
    const int run_pages = (run_end - run_begin + DL_PAGE - 1) / DL_PAGE;
    const int32_t* pages = block_table + (size_t)b * bt_stride;

    if (threadIdx.x == 0) {
        gave_up = 0;
        for (int s = 0; s < AD_STAGES; ++s) {
            ad_mbar_init(&full_bar[s], 1);
            ad_mbar_init(&empty_bar[s], 2);              // the two warps of a pair release a stage
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    float o[DT][4];
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;

    if (warp == AD_CONSUMERS) {
        // ------------------------------------------------------------ producer (one thread)
        if (lane == 0) {
            int issued = 0;
            for (int i = 0; i < run_pages; ++i) {
                const int s = i % AD_STAGES;
                const int page = pages[page0 + i];
                if (page < 0 || page >= n_pages) { gave_up = 1; atomicExch(status, 2); break; }   // host-validated
                if (i >= AD_STAGES && !ad_mbar_wait(&empty_bar[s], ((i / AD_STAGES) - 1) & 1, &gave_up)) {
                    gave_up = 1;
                    atomicExch(status, 1);
                    break;
                }
                __nv_bfloat16* dst = stage_mem + (size_t)s * 2 * PAGE_ELEMS;
                ad_mbar_expect(&full_bar[s], 2 * PAGE_BYTES);
                ad_bulk_copy(dst, k_pool + dl_k_offset(page, nkv, kvh, 0, HD), PAGE_BYTES, &full_bar[s]);
                ad_bulk_copy(dst + PAGE_ELEMS, v_pool + dl_v_offset(page, nkv, kvh, 0, HD), PAGE_BYTES, &full_bar[s]);
                issued = i + 1;
            }
            if (gave_up) {
                // copies already issued must land before the block's shared memory is released
                for (int i = max(0, issued - AD_STAGES); i < issued; ++i) {
                    const long long t0 = clock64();
                    while (!ad_mbar_try(&full_bar[i % AD_STAGES], (i / AD_STAGES) & 1) && clock64() - t0 < AD_WAIT_CYCLES) {}
                }
            }
        }
    } else {
        // ------------------------------------------------------------ consumers
        const int pair = warp >> 1, half = warp & 1;
        // Q rows g and g+8 of the group (zero beyond the group)
        uint4 qf_lo[DC], qf_hi[DC];
        {
            const __nv_bfloat16* qb = q + (size_t)b * q_stride + (size_t)kvh * group * HD;
#pragma unroll
            for (int c = 0; c < DC; ++c) {
                qf_lo[c] = make_uint4(0u, 0u, 0u, 0u);
                qf_hi[c] = make_uint4(0u, 0u, 0u, 0u);
                if (g < group) qf_lo[c] = *reinterpret_cast<const uint4*>(qb + (size_t)g * HD + c * 32 + t * 8);
                if (g + 8 < group) qf_hi[c] = *reinterpret_cast<const uint4*>(qb + (size_t)(g + 8) * HD + c * 32 + t * 8);
            }
        }
#pragma unroll
        for (int i = 0; i < DT; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) o[i][e] = 0.f;

        for (int i = pair; i < run_pages; i += 2) {
            const int s = i % AD_STAGES;
            if (!ad_mbar_wait(&full_bar[s], (i / AD_STAGES) & 1, &gave_up)) {
                gave_up = 1;
                atomicExch(status, 3);
                break;
            }
            const int base = run_begin + i * DL_PAGE + 32 * half;     // first key of this warp's 32
            if (base < run_end) {
                const __nv_bfloat16* kp = stage_mem + (size_t)s * 2 * PAGE_ELEMS + (size_t)(32 * half) * HD;
                const __nv_bfloat16* vp = stage_mem + (size_t)s * 2 * PAGE_ELEMS + PAGE_ELEMS + 32 * half;

                // ---- S = Q K^T for 32 keys
                float sc[4][4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int key = 8 * (g >> 1) + 2 * j + (g & 1);
#pragma unroll
                    for (int e = 0; e < 4; ++e) sc[j][e] = 0.f;
#pragma unroll
                    for (int c = 0; c < DC; ++c) {
                        const uint4 kf = *reinterpret_cast<const uint4*>(kp + (size_t)key * HD + c * 32 + t * 8);
                        ad_mma(sc[j], qf_lo[c].x, qf_hi[c].x, qf_lo[c].y, qf_hi[c].y, kf.x, kf.y);
                        ad_mma(sc[j], qf_lo[c].z, qf_hi[c].z, qf_lo[c].w, qf_hi[c].w, kf.z, kf.w);
                    }
                }
                // ---- mask, online softmax (lane holds keys base + 8t + 2j + {0,1} of rows g and g+8)
                float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
                for (int j = 0; j < 4; ++j)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int key = base + 8 * t + 2 * j + e;
                        const bool ok = key >= first && key < len;
                        sc[j][e] = ok ? sc[j][e] * scale : -INFINITY;
                        sc[j][2 + e] = ok ? sc[j][2 + e] * scale : -INFINITY;
                        mx_lo = fmaxf(mx_lo, sc[j][e]);
                        mx_hi = fmaxf(mx_hi, sc[j][2 + e]);
                    }
                mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
                mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
                mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
                mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
                const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
                // 32 keys may be wholly masked by the window: the state stays untouched then
                const float c_lo = (mn_lo == -INFINITY) ? 1.f : expf(m_lo - mn_lo);
                const float c_hi = (mn_hi == -INFINITY) ? 1.f : expf(m_hi - mn_hi);
                float ps_lo = 0.f, ps_hi = 0.f;
                uint32_t pa[4][2];                               // [tile][row half] packed bf16 pairs
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float p0 = (sc[j][0] == -INFINITY) ? 0.f : expf(sc[j][0] - mn_lo);
                    const float p1 = (sc[j][1] == -INFINITY) ? 0.f : expf(sc[j][1] - mn_lo);
                    const float p2 = (sc[j][2] == -INFINITY) ? 0.f : expf(sc[j][2] - mn_hi);
                    const float p3 = (sc[j][3] == -INFINITY) ? 0.f : expf(sc[j][3] - mn_hi);
                    ps_lo += p0 + p1;
                    ps_hi += p2 + p3;
                    pa[j][0] = ad_pack(p0, p1);
                    pa[j][1] = ad_pack(p2, p3);
                }
                l_lo = l_lo * c_lo + ps_lo;
                l_hi = l_hi * c_hi + ps_hi;
                m_lo = mn_lo;
                m_hi = mn_hi;

                // ---- O = O * corr + P V.  Keys outside [first, len) may hold anything (even NaN).
                const bool ragged = (base + 32 > len) || (base < first);
#pragma unroll
                for (int i2 = 0; i2 < DT; ++i2) {
                    o[i2][0] *= c_lo;
                    o[i2][1] *= c_lo;
                    o[i2][2] *= c_hi;
                    o[i2][3] *= c_hi;
                    uint4 v = *reinterpret_cast<const uint4*>(vp + (size_t)(8 * i2 + g) * DL_PAGE + 8 * t);
                    if (ragged) v = ad_keep_keys(v, base + 8 * t, first, len);
                    ad_mma(o[i2], pa[0][0], pa[0][1], pa[1][0], pa[1][1], v.x, v.y);
                    ad_mma(o[i2], pa[2][0], pa[2][1], pa[3][0], pa[3][1], v.z, v.w);
                }
            }
            __syncwarp();
            if (lane == 0) ad_mbar_arrive(&empty_bar[s]);
        }
        l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
        l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
        l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
        l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    }

    // ---- merge the block's warps (fixed order).  The stages are free now: all copies were consumed.
    __syncthreads();
    if (gave_up) return;
    if (warp < AD_CONSUMERS) {
#pragma unroll
        for (int i = 0; i < DT; ++i) {
            sm_o[warp][g][8 * i + 2 * t] = o[i][0];
            sm_o[warp][g][8 * i + 2 * t + 1] = o[i][1];
            sm_o[warp][g + 8][8 * i + 2 * t] = o[i][2];
            sm_o[warp][g + 8][8 * i + 2 * t + 1] = o[i][3];
        }
        if (t == 0) {
            sm_m[warp][g] = m_lo;
            sm_l[warp][g] = l_lo;
            sm_m[warp][g + 8] = m_hi;
            sm_l[warp][g + 8] = l_hi;
        }
    }
    __syncthreads();

    const size_t part_row = ((size_t)(b * nkv + kvh) * gridDim.x + split) * group;
    for (int idx = threadIdx.x; idx < group * HD; idx += AD_THREADS) {
        const int r = idx / HD, d = idx - r * HD;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < AD_CONSUMERS; ++w) m = fmaxf(m, sm_m[w][r]);
        float acc = 0.f, l = 0.f;
#pragma unroll
        for (int w = 0; w < AD_CONSUMERS; ++w) {
            const float f = (sm_m[w][r] == -INFINITY) ? 0.f : expf(sm_m[w][r] - m);
            acc += sm_o[w][r][d] * f;
            l += sm_l[w][r] * f;
        }
        if (n_splits == 1) {
            out[(size_t)b * out_stride + (size_t)(kvh * group + r) * HD + d] = __float2bfloat16_rn(acc / l);
        } else {
            part_o[(part_row + r) * HD + d] = acc;
            if (d == 0) {
                part_ml[(part_row + r) * 2] = m;
                part_ml[(part_row + r) * 2 + 1] = l;
            }
        }
    }
    if (n_splits == 1) return;

    // ---- the last block of this (sequence, KV head) merges the runs (fixed order)
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        int* counter = counters + b * nkv + kvh;
        const int seen = atomicAdd(counter, 1);
        is_last = (seen == n_splits - 1);
        if (is_last) *counter = 0;                       // ready for the next launch
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    const size_t row0 = ((size_t)(b * nkv + kvh) * gridDim.x) * group;
    for (int idx = threadIdx.x; idx < group * HD; idx += AD_THREADS) {
        const int r = idx / HD, d = idx - r * HD;
        float m = -INFINITY;
        for (int sp = 0; sp < n_splits; ++sp) m = fmaxf(m, __ldcg(part_ml + (row0 + (size_t)sp * group + r) * 2));
        float acc = 0.f, l = 0.f;
        for (int sp = 0; sp < n_splits; ++sp) {
            const size_t row = row0 + (size_t)sp * group + r;
            const float ms = __ldcg(part_ml + row * 2);
            const float f = (ms == -INFINITY) ? 0.f : expf(ms - m);
            acc += __ldcg(part_o + row * HD + d) * f;
            l += __ldcg(part_ml + row * 2 + 1) * f;
        }
        out[(size_t)b * out_stride + (size_t)(kvh * group + r) * HD + d] = __float2bfloat16_rn(acc / l);
    }
}

template <int HD>
static int ad_launch(dim3 grid, cudaStream_t s, const void* q, int q_stride, void* out, int out_stride,
                     const void* k_pool, const void* v_pool, int n_pages, const int32_t* seq_len,
                     const int32_t* block_table, int bt_stride, int nh, int nkv, float scale, int window,
                     int keys_per_split, float* part_o, float* part_ml, int* counters, int* status) {
    const size_t stage_bytes = (size_t)AD_STAGES * 2 * DL_PAGE * HD * 2;
    const size_t merge_bytes = (size_t)AD_CONSUMERS * 16 * (HD + 4) * sizeof(float);
    const size_t smem = stage_bytes > merge_bytes ? stage_bytes : merge_bytes;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "attention_decode: shared memory %zu: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    attention_decode_kernel<HD><<<grid, AD_THREADS, smem, s>>>(
        (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)k_pool,
        (const __nv_bfloat16*)v_pool, n_pages, seq_len, block_table, bt_stride, nh, nkv, scale, window, keys_per_split,
        part_o, part_ml, counters, status);
    DL_CHECK_LAUNCH("attention_decode");
    return DL_OK;
}

// q: bf16 [B, nh*hd] rows q_stride apart (one token per sequence); out likewise.
// seq_len[b]: keys of sequence b including the new token.  max_splits = grid size over runs,
// at least ceil(longest visible span / keys_per_split).
// part_o: float32 [B, nkv, max_splits, group, hd]; part_ml: float32 [B, nkv, max_splits, group, 2];
// counters: int32 zeros [B * nkv] (left zero); status: int32, set non-zero if a wait expired.
extern "C" int dl_attention_decode_bf16(const void* q, int q_stride, void* out, int out_stride, const void* k_pool,
                                        const void* v_pool, int n_pages, const int32_t* seq_len,
                                        const int32_t* block_table, int bt_stride, int n_seqs, int nh, int nkv,
                                        int hd, float scale, int window, int keys_per_split, int max_splits,
                                        float* part_o, float* part_ml, int* counters, int* status, void* stream) {
    DL_REQUIRE(n_seqs >= 0 && nh > 0 && nkv > 0 && nh % nkv == 0, "attention_decode: bad head counts");
    DL_REQUIRE(nh / nkv <= 16, "attention_decode: groups of more than 16 query heads are not supported (%d)", nh / nkv);
    DL_REQUIRE(keys_per_split >= DL_PAGE && keys_per_split % DL_PAGE == 0, "attention_decode: keys_per_split %d must be a multiple of %d", keys_per_split, DL_PAGE);
    DL_REQUIRE(max_splits >= 1 && (max_splits == 1 || (part_o && part_ml && counters)), "attention_decode: split runs need scratch");
    DL_REQUIRE(status != nullptr, "attention_decode: needs a status word");
    DL_REQUIRE(q_stride % 8 == 0 && ((uintptr_t)q % 16) == 0 && ((uintptr_t)k_pool % 16) == 0 && ((uintptr_t)v_pool % 16) == 0,
               "attention_decode: q and the pools must be 16-byte aligned");
    DL_REQUIRE(n_seqs <= 65535 && nkv <= 65535, "attention_decode: grid too large");
    if (n_seqs == 0) return DL_OK;
    dim3 grid(max_splits, nkv, n_seqs);
    cudaStream_t s = (cudaStream_t)stream;
#define AD_CASE(HDV)                                                                                                  \
    if (hd == HDV)                                                                                                    \
        return ad_launch<HDV>(grid, s, q, q_stride, out, out_stride, k_pool, v_pool, n_pages, seq_len, block_table,   \
                              bt_stride, nh, nkv, scale, window, keys_per_split, part_o, part_ml, counters, status);
    AD_CASE(32) AD_CASE(64) AD_CASE(96) AD_CASE(128)
#undef AD_CASE
    return dl_fail(DL_ERR_UNSUPPORTED, "attention_decode: head_dim %d (takes 32, 64, 96, 128)", hd);
}
