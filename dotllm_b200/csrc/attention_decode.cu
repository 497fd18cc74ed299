// Decode attention: one new token per sequence over its paged bfloat16 cache, split over keys.
//
// Role of the reference's attention_f16 with seq_q == 1 (native/kernels/attention.cu:19-197): scores
// scaled by 1/sqrt(hd), softmax with the running maximum subtracted, weighted sum of values, query
// head h reading KV head h / group.  A decode step is bound by the bytes of K and V, so each
// (sequence, KV head) is cut into runs of pages, and all query heads of the group share every key
// and value that is loaded: the group's heads are the rows of mma.sync.m16n8k16 tiles (rows beyond
// the group are zero).
//
// Shape: persistent and warp-specialised.  One block per multiprocessor walks the runs
// it % gridDim.x == blockIdx.x.  A cache page of one KV head is two contiguous pieces (K [64][hd],
// V [hd][64]); one producer thread copies them with cp.async.bulk (the bulk-copy engine) into a ring
// of shared-memory stages, signalling an mbarrier per stage, and runs ahead of the arithmetic by the
// depth of the ring, across run boundaries, at no cost in registers.  Consumer warp w takes pages
// w, w + C, ... of the stream; at the end of a run the warps merge their partial results in shared
// memory and the block writes either the output or the run's partial (max, sum, weighted values).
// A second small kernel merges the runs of a (sequence, head) in a fixed order.
//
// Arithmetic: lane (g, t) reads 16-byte pieces of K rows: dims 8t..8t+7 of a 32-dim slice are a
// consistent permutation of k for Q and K in two MMAs; the 8 key columns of score tile j are keys
// 8(g/2) + 2j + (g&1) of a 32-key half page, so that after four tiles the lane holds scores of keys
// 8t..8t+7 - exactly the k-permutation that pairs with a 16-byte piece of a transposed V row.
// Softmax is float32 in base 2: scores are scaled by log2(e)/sqrt(hd) and exponentials are
// ex2.approx (2 ulp), far below the bfloat16 rounding of the weights that follows.
//
// Every wait on an mbarrier is bounded (about a second of clock cycles); on expiry the kernel
// records a code in `status`, stops issuing copies, waits (bounded) for copies in flight, and
// returns.  The host reads `status` at its next synchronisation point.
#include "common.cuh"

// One ring stage per consumer warp: warp w owns stage w and sees every phase of its barriers in
// order.  (A warp that shared stages with others could fall two phases behind a barrier and
// mistake an old completion for the one it waits for: mbarrier waits tell phases apart by parity only.)
#define AD_MAX_STAGES 6                        // consumer warps = stages, as many as fit in shared memory
#define AD_THREADS (32 * (AD_MAX_STAGES + 1))  // the last warp is the producer
#define AD_WAIT_CYCLES (1ll << 31)

__device__ __forceinline__ void ad_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
    // not volatile: independent accumulators must be free to interleave
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float ad_ex2(float x) {            // 2^x, 2 ulp; ex2(-inf) = 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
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
__device__ __forceinline__ void ad_consumer_sync(int n_consumers) {
    asm volatile("bar.sync 1, %0;" ::"r"(32 * n_consumers) : "memory");
}

// 16 bytes from a shared-space byte address (a 32-bit register, constant offsets fold into the load)
__device__ __forceinline__ uint4 ad_lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}

// One (sequence, KV head, run of pages) and where its pages are.
struct AdItem {
    int b, kvh, split, n_splits, len, first, run_begin, page0, n_pages;
};

__device__ __forceinline__ AdItem ad_item(int it, int max_splits, int nkv, const int32_t* seq_len, int window,
                                          int keys_per_split) {
    AdItem w;
    w.split = it % max_splits;
    const int pair = it / max_splits;
    w.kvh = pair % nkv;
    w.b = pair / nkv;
    w.len = seq_len[w.b];                                  // keys 0..len-1; the query sits at len-1
    w.first = (window > 0 && w.len - window > 0) ? w.len - window : 0;
    const int origin = (w.first / DL_PAGE) * DL_PAGE;      // runs start at the first visible key's page
    w.n_splits = (w.len - origin + keys_per_split - 1) / keys_per_split;
    w.run_begin = origin + w.split * keys_per_split;
    const int run_end = min(w.len, w.run_begin + keys_per_split);
    w.page0 = w.run_begin / DL_PAGE;
    w.n_pages = w.split < w.n_splits ? (run_end - w.run_begin + DL_PAGE - 1) / DL_PAGE : 0;
    return w;
}

// WIDE: the group has more than 8 query heads, so fragment rows 8..15 carry data too.
template <int HD, bool WIDE>
__global__ void __launch_bounds__(AD_THREADS, 1)
attention_decode_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, __nv_bfloat16* __restrict__ out,
                        int out_stride, const __nv_bfloat16* __restrict__ k_pool,
                        const __nv_bfloat16* __restrict__ v_pool, int n_pages,
                        const int32_t* __restrict__ seq_len, const int32_t* __restrict__ block_table,
                        int bt_stride, int n_items, int max_splits, int nh, int nkv, float scale, int window,
                        int keys_per_split, int n_stages, float* __restrict__ part_o,
                        float* __restrict__ part_ml, int* __restrict__ status) {
    constexpr int DC = HD / 32;          // 32-dim slices of a head
    constexpr int DT = HD / 8;           // 8-dim output tiles
    constexpr int PAGE_ELEMS = DL_PAGE * HD;
    constexpr uint32_t PAGE_BYTES = PAGE_ELEMS * 2;
    extern __shared__ __align__(128) unsigned char ad_smem_raw[];
    __nv_bfloat16* stage_mem = reinterpret_cast<__nv_bfloat16*>(ad_smem_raw);      // [stage][K page | V page]
    const int group = nh / nkv;
    // after the stages: each consumer warp's partial output [group][HD + 4]
    float* merge_o = reinterpret_cast<float*>(ad_smem_raw + (size_t)n_stages * 2 * PAGE_BYTES);
    __shared__ uint64_t full_bar[AD_MAX_STAGES], empty_bar[AD_MAX_STAGES];
    __shared__ float sm_m[AD_MAX_STAGES][16], sm_l[AD_MAX_STAGES][16];
    __shared__ volatile int gave_up;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    // The kernel checks its own shared-memory layout: if the launch gave it less dynamic shared
    // memory than the stages and merge buffers need, it records status 11 and touches nothing.
    uint32_t smem_bytes;
    asm("mov.u32 %0, %dynamic_smem_size;" : "=r"(smem_bytes));
    const uint32_t smem_lo = ad_smem(ad_smem_raw), smem_hi = smem_lo + smem_bytes;
    if ((size_t)n_stages * 2 * PAGE_BYTES + (size_t)n_stages * group * (HD + 4) * 4 > smem_bytes) {
        if (threadIdx.x == 0) atomicExch(status, 11);
        return;
    }

    if (threadIdx.x == 0) {
        gave_up = 0;
        for (int s = 0; s < n_stages; ++s) {
            ad_mbar_init(&full_bar[s], 1);
            ad_mbar_init(&empty_bar[s], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == AD_MAX_STAGES) {
        // ------------------------------------------------------------ producer
        // The warp reads 32 page ids at a time (one coalesced load); lane 0 issues the copies.
        int n = 0;                                           // pages issued so far, over all runs
        bool stop = false;
        for (int it = blockIdx.x; it < n_items && !stop; it += gridDim.x) {
            const AdItem w = ad_item(it, max_splits, nkv, seq_len, window, keys_per_split);
            const int32_t* pages = block_table + (size_t)w.b * bt_stride + w.page0;
            for (int i0 = 0; i0 < w.n_pages && !stop; i0 += 32) {
                const int mine = (i0 + lane < w.n_pages) ? pages[i0 + lane] : 0;
                const int count = min(32, w.n_pages - i0);
                for (int j = 0; j < count; ++j, ++n) {
                    const int page = __shfl_sync(0xffffffffu, mine, j);
                    int bad = 0;
                    if (lane == 0) {
                        const int s = n % n_stages;
                        if (page < 0 || page >= n_pages) {   // host-validated
                            bad = 2;
                        } else if (n >= n_stages && !ad_mbar_wait(&empty_bar[s], ((n / n_stages) - 1) & 1, &gave_up)) {
                            bad = 1;
                        } else {
                            __nv_bfloat16* dst = stage_mem + (size_t)s * 2 * PAGE_ELEMS;
                            ad_mbar_expect(&full_bar[s], 2 * PAGE_BYTES);
                            ad_bulk_copy(dst, k_pool + dl_k_offset(page, nkv, w.kvh, 0, HD), PAGE_BYTES, &full_bar[s]);
                            ad_bulk_copy(dst + PAGE_ELEMS, v_pool + dl_v_offset(page, nkv, w.kvh, 0, HD), PAGE_BYTES, &full_bar[s]);
                        }
                    }
                    bad = __shfl_sync(0xffffffffu, bad, 0);
                    if (bad) {
                        if (lane == 0) { gave_up = 1; atomicExch(status, bad); }
                        stop = true;
                        break;
                    }
                }
            }
        }
        if (stop && lane == 0) {
            // copies already issued must land before the block's shared memory is released
            for (int i = max(0, n - n_stages); i < n; ++i) {
                const long long t0 = clock64();
                while (!ad_mbar_try(&full_bar[i % n_stages], (i / n_stages) & 1) && clock64() - t0 < AD_WAIT_CYCLES) {}
            }
        }
    } else if (warp < n_stages) {
        // ------------------------------------------------------------ consumers (warp w owns stage w)
        float* my_o = merge_o + (size_t)warp * group * (HD + 4);
        const float scale2 = scale * 1.4426950408889634f;    // scores in units of log2
        int n0 = 0;                                          // pages of the runs before this one
        for (int it = blockIdx.x; it < n_items; it += gridDim.x) {
            const AdItem w = ad_item(it, max_splits, nkv, seq_len, window, keys_per_split);
            if (w.n_pages == 0) continue;                    // the same for every warp of the block
            // Q rows g and g+8 of the group (zero beyond the group)
            uint4 qf_lo[DC], qf_hi[DC];
            {
                const __nv_bfloat16* qb = q + (size_t)w.b * q_stride + (size_t)w.kvh * group * HD;
#pragma unroll
                for (int c = 0; c < DC; ++c) {
                    qf_lo[c] = make_uint4(0u, 0u, 0u, 0u);
                    qf_hi[c] = make_uint4(0u, 0u, 0u, 0u);
                    if (g < group) qf_lo[c] = *reinterpret_cast<const uint4*>(qb + (size_t)g * HD + c * 32 + t * 8);
                    if (WIDE && g + 8 < group) qf_hi[c] = *reinterpret_cast<const uint4*>(qb + (size_t)(g + 8) * HD + c * 32 + t * 8);
                }
            }
            float o[DT][4];
#pragma unroll
            for (int i = 0; i < DT; ++i)
#pragma unroll
                for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
            float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;   // maxima in units of log2

            const int i_first = ((warp - n0) % n_stages + n_stages) % n_stages;   // first i with (n0 + i) % n_stages == warp
            for (int i = i_first; i < w.n_pages; i += n_stages) {
                const int n = n0 + i;
                const int s = warp;
                if (!ad_mbar_wait(&full_bar[s], (n / n_stages) & 1, &gave_up)) {
                    if (!gave_up) atomicExch(status, 3);
                    gave_up = 1;
                    continue;                                 // keep walking so that every barrier below is reached
                }
                const int base = w.run_begin + i * DL_PAGE;  // first key of the page
                __nv_bfloat16* kp = stage_mem + (size_t)s * 2 * PAGE_ELEMS;
                __nv_bfloat16* vp = kp + PAGE_ELEMS;
                const bool ragged = (base + DL_PAGE > w.len) || (base < w.first);
                if (ragged) {
                    // Keys outside [first, len) may hold anything (even NaN): make their values exact
                    // zeros in the stage once, so that the product below needs no special case.
                    for (int idx = lane; idx < HD * DL_PAGE; idx += 32) {
                        const int key = base + (idx & (DL_PAGE - 1));
                        if (key < w.first || key >= w.len) vp[idx] = __float2bfloat16_rn(0.f);
                    }
                    __syncwarp();
                }
                // this lane's byte addresses in shared space; every load below is a constant offset away
                const uint32_t k_addr = ad_smem(kp) + (uint32_t)((8 * (g >> 1) + (g & 1)) * HD + t * 8) * 2u;
                const uint32_t v_addr = ad_smem(vp) + (uint32_t)(g * DL_PAGE + t * 8) * 2u;
                // the furthest loads are (38 rows of K + 96 dims) and (15 dim tiles of V + 32 keys) away
                const bool inside = k_addr >= smem_lo && k_addr + (uint32_t)((38 * HD + (DC - 1) * 32) * 2 + 16) <= smem_hi &&
                                    v_addr >= smem_lo && v_addr + (uint32_t)((8 * (DT - 1) * DL_PAGE + 32) * 2 + 16) <= smem_hi &&
                                    ((k_addr | v_addr) & 15u) == 0;
                if (__any_sync(0xffffffffu, !inside)) {       // never read outside the block's shared memory
                    if (lane == 0) atomicExch(status, 10);
                    gave_up = 1;
                    __syncwarp();
                    if (lane == 0) ad_mbar_arrive(&empty_bar[s]);
                    continue;
                }

                // ---- S = Q K^T for 64 keys: two halves of four 8-key tiles, dim slice outermost so
                // that consecutive MMAs go to eight different accumulators
                float sc[2][4][4];
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int j = 0; j < 4; ++j)
#pragma unroll
                        for (int e = 0; e < 4; ++e) sc[h][j][e] = 0.f;
#pragma unroll
                for (int c = 0; c < DC; ++c) {
                    uint4 kf[2][4];
#pragma unroll
                    for (int h = 0; h < 2; ++h)
#pragma unroll
                        for (int j = 0; j < 4; ++j)     // key 32h + 8(g/2) + 2j + (g&1), dims 32c + 8t ..
                            kf[h][j] = ad_lds128(k_addr + (uint32_t)(((32 * h + 2 * j) * HD + c * 32) * 2));
#pragma unroll
                    for (int h = 0; h < 2; ++h)
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            ad_mma(sc[h][j], qf_lo[c].x, qf_hi[c].x, qf_lo[c].y, qf_hi[c].y, kf[h][j].x, kf[h][j].y);
#pragma unroll
                    for (int h = 0; h < 2; ++h)
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            ad_mma(sc[h][j], qf_lo[c].z, qf_hi[c].z, qf_lo[c].w, qf_hi[c].w, kf[h][j].z, kf[h][j].w);
                }
                // ---- mask (ragged pages only; lane holds keys base + 32h + 8t + 2j + {0,1}) and row maximum
                if (ragged) {
#pragma unroll
                    for (int h = 0; h < 2; ++h)
#pragma unroll
                        for (int j = 0; j < 4; ++j)
#pragma unroll
                            for (int e = 0; e < 2; ++e) {
                                const int key = base + 32 * h + 8 * t + 2 * j + e;
                                if (key < w.first || key >= w.len) {
                                    sc[h][j][e] = -INFINITY;
                                    sc[h][j][2 + e] = -INFINITY;
                                }
                            }
                }
                float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        mx_lo = fmaxf(mx_lo, fmaxf(sc[h][j][0], sc[h][j][1]));
                        if (WIDE) mx_hi = fmaxf(mx_hi, fmaxf(sc[h][j][2], sc[h][j][3]));
                    }
                mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
                mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
                // scale > 0, so the maximum of the scaled scores is the scaled maximum
                const float mn_lo = fmaxf(m_lo, mx_lo * scale2);
                // a page may be wholly masked by the window: the state stays untouched then
                const bool dead_lo = mn_lo == -INFINITY;
                const float c_lo = dead_lo ? 1.f : ad_ex2(m_lo - mn_lo);
                const float sub_lo = dead_lo ? 0.f : mn_lo;
                float mn_hi = -INFINITY, c_hi = 1.f, sub_hi = 0.f;
                if (WIDE) {
                    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
                    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
                    mn_hi = fmaxf(m_hi, mx_hi * scale2);
                    const bool dead_hi = mn_hi == -INFINITY;
                    c_hi = dead_hi ? 1.f : ad_ex2(m_hi - mn_hi);
                    sub_hi = dead_hi ? 0.f : mn_hi;
                }
                // ---- p = 2^(s * scale2 - max): one FFMA and one ex2 per score; ex2(-inf) = 0
                float ps_lo = 0.f, ps_hi = 0.f;
                uint32_t pa[2][4][2];                        // [half][tile][row half] packed bf16 pairs
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float p0 = ad_ex2(fmaf(sc[h][j][0], scale2, -sub_lo));
                        const float p1 = ad_ex2(fmaf(sc[h][j][1], scale2, -sub_lo));
                        ps_lo += p0 + p1;
                        pa[h][j][0] = ad_pack(p0, p1);
                        pa[h][j][1] = 0u;
                        if (WIDE) {
                            const float p2 = ad_ex2(fmaf(sc[h][j][2], scale2, -sub_hi));
                            const float p3 = ad_ex2(fmaf(sc[h][j][3], scale2, -sub_hi));
                            ps_hi += p2 + p3;
                            pa[h][j][1] = ad_pack(p2, p3);
                        }
                    }
                l_lo = l_lo * c_lo + ps_lo;
                m_lo = mn_lo;
                if (WIDE) {
                    l_hi = l_hi * c_hi + ps_hi;
                    m_hi = mn_hi;
                }
                // ---- O = O * corr + P V.  The rescale is skipped while no row's maximum moves.
                const bool rescale = __any_sync(0xffffffffu, c_lo != 1.f || (WIDE && c_hi != 1.f));
                if (rescale) {
#pragma unroll
                    for (int i2 = 0; i2 < DT; ++i2) {
                        o[i2][0] *= c_lo;
                        o[i2][1] *= c_lo;
                        if (WIDE) {
                            o[i2][2] *= c_hi;
                            o[i2][3] *= c_hi;
                        }
                    }
                }
#pragma unroll
                for (int h = 0; h < 2; ++h) {
#pragma unroll
                    for (int i2 = 0; i2 < DT; ++i2) {
                        // dim 8 i2 + g, keys 32h + 8t ..
                        const uint4 v = ad_lds128(v_addr + (uint32_t)((8 * i2 * DL_PAGE + 32 * h) * 2));
                        ad_mma(o[i2], pa[h][0][0], pa[h][0][1], pa[h][1][0], pa[h][1][1], v.x, v.y);
                        ad_mma(o[i2], pa[h][2][0], pa[h][2][1], pa[h][3][0], pa[h][3][1], v.z, v.w);
                    }
                }
                __syncwarp();
                if (lane == 0) ad_mbar_arrive(&empty_bar[s]);
            }
            n0 += w.n_pages;

            // ---- merge the block's warps (fixed order) and hand the run's result on
            l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
            l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
            if (WIDE) {
                l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
                l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
            }
#pragma unroll
            for (int i = 0; i < DT; ++i) {
                if (g < group) {
                    my_o[g * (HD + 4) + 8 * i + 2 * t] = o[i][0];
                    my_o[g * (HD + 4) + 8 * i + 2 * t + 1] = o[i][1];
                }
                if (WIDE && g + 8 < group) {
                    my_o[(g + 8) * (HD + 4) + 8 * i + 2 * t] = o[i][2];
                    my_o[(g + 8) * (HD + 4) + 8 * i + 2 * t + 1] = o[i][3];
                }
            }
            if (t == 0) {
                sm_m[warp][g] = m_lo;
                sm_l[warp][g] = l_lo;
                sm_m[warp][g + 8] = WIDE ? m_hi : -INFINITY;
                sm_l[warp][g + 8] = WIDE ? l_hi : 0.f;
            }
            ad_consumer_sync(n_stages);

            const int tid = threadIdx.x;                     // 0 .. 32*n_stages-1
            const size_t part_row = ((size_t)(w.b * nkv + w.kvh) * max_splits + w.split) * group;
            for (int idx = tid; idx < group * HD; idx += 32 * n_stages) {
                const int r = idx / HD, d = idx - r * HD;
                float m = -INFINITY;
                for (int cw = 0; cw < n_stages; ++cw) m = fmaxf(m, sm_m[cw][r]);
                float acc = 0.f, l = 0.f;
                for (int cw = 0; cw < n_stages; ++cw) {
                    const float f = (sm_m[cw][r] == -INFINITY) ? 0.f : ad_ex2(sm_m[cw][r] - m);
                    acc += merge_o[((size_t)cw * group + r) * (HD + 4) + d] * f;
                    l += sm_l[cw][r] * f;
                }
                if (w.n_splits == 1) {
                    out[(size_t)w.b * out_stride + (size_t)(w.kvh * group + r) * HD + d] = __float2bfloat16_rn(acc / l);
                } else {
                    part_o[(part_row + r) * HD + d] = acc;
                    if (d == 0) {
                        part_ml[(part_row + r) * 2] = m;
                        part_ml[(part_row + r) * 2 + 1] = l;
                    }
                }
            }
            ad_consumer_sync(n_stages);                              // the merge buffers are free for the next run
        }
    }
    __syncthreads();                                         // nobody leaves while copies may still land
}

// Merge the runs of every (sequence, head) that was cut into more than one, in run order.
// One block per (sequence, KV head); thread -> (head of the group, dim).
__global__ void __launch_bounds__(256)
attention_decode_combine_kernel(__nv_bfloat16* __restrict__ out, int out_stride, const int32_t* __restrict__ seq_len,
                                int nh, int nkv, int hd, int window, int keys_per_split, int max_splits,
                                const float* __restrict__ part_o, const float* __restrict__ part_ml) {
    const int kvh = blockIdx.x, b = blockIdx.y;
    const int group = nh / nkv;
    const int len = seq_len[b];
    const int first = (window > 0 && len - window > 0) ? len - window : 0;
    const int origin = (first / DL_PAGE) * DL_PAGE;
    const int n_splits = (len - origin + keys_per_split - 1) / keys_per_split;
    if (n_splits <= 1) return;                               // the main kernel wrote the output itself
    const size_t row0 = ((size_t)(b * nkv + kvh) * max_splits) * group;
    for (int idx = threadIdx.x; idx < group * hd; idx += blockDim.x) {
        const int r = idx / hd, d = idx - r * hd;
        float m = -INFINITY;
        for (int sp = 0; sp < n_splits; ++sp) m = fmaxf(m, part_ml[(row0 + (size_t)sp * group + r) * 2]);
        float acc = 0.f, l = 0.f;
        for (int sp = 0; sp < n_splits; ++sp) {
            const size_t row = row0 + (size_t)sp * group + r;
            const float ms = part_ml[row * 2];
            const float f = (ms == -INFINITY) ? 0.f : ad_ex2(ms - m);
            acc += part_o[row * hd + d] * f;
            l += part_ml[row * 2 + 1] * f;
        }
        out[(size_t)b * out_stride + (size_t)(kvh * group + r) * hd + d] = __float2bfloat16_rn(acc / l);
    }
}

template <int HD, bool WIDE>
static int ad_launch(cudaStream_t s, const void* q, int q_stride, void* out, int out_stride, const void* k_pool,
                     const void* v_pool, int n_pages, const int32_t* seq_len, const int32_t* block_table,
                     int bt_stride, int n_seqs, int max_splits, int nh, int nkv, float scale, int window,
                     int keys_per_split, float* part_o, float* part_ml, int* status) {
    const int group = nh / nkv;
    int dev = 0, sms = 0, max_smem = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    const size_t stage = (size_t)2 * DL_PAGE * HD * 2;
    const size_t merge_per = (size_t)group * (HD + 4) * sizeof(float);     // one consumer warp's partial output
    int n_stages = AD_MAX_STAGES;
    while (n_stages > 2 && n_stages * (stage + merge_per) + 2048 > (size_t)max_smem) --n_stages;
    const size_t smem = n_stages * (stage + merge_per);
    if (smem + 2048 > (size_t)max_smem)
        return dl_fail(DL_ERR_UNSUPPORTED, "attention_decode: head_dim %d with %d heads per group needs %zu bytes of shared memory", HD, group, smem);
    static int configured = 0;
    if (configured < (int)smem) {
        cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<HD, WIDE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "attention_decode: shared memory %zu: %s", smem, cudaGetErrorString(e));
        configured = (int)smem;
    }
    const int n_items = n_seqs * nkv * max_splits;
    const int blocks = n_items < sms ? n_items : sms;
    attention_decode_kernel<HD, WIDE><<<blocks, AD_THREADS, smem, s>>>(
        (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)k_pool,
        (const __nv_bfloat16*)v_pool, n_pages, seq_len, block_table, bt_stride, n_items, max_splits, nh, nkv, scale,
        window, keys_per_split, n_stages, part_o, part_ml, status);
    DL_CHECK_LAUNCH("attention_decode");
    if (max_splits > 1) {
        attention_decode_combine_kernel<<<dim3(nkv, n_seqs), 256, 0, s>>>((__nv_bfloat16*)out, out_stride, seq_len, nh, nkv,
                                                                        HD, window, keys_per_split, max_splits, part_o,
                                                                        part_ml);
        DL_CHECK_LAUNCH("attention_decode_combine");
    }
    return DL_OK;
}

// q: bf16 [B, nh*hd] rows q_stride apart (one token per sequence); out likewise.
// seq_len[b]: keys of sequence b including the new token.  max_splits: runs a (sequence, KV head) may
// be cut into, at least ceil(longest visible span / keys_per_split).
// part_o: float32 [B, nkv, max_splits, group, hd]; part_ml: float32 [B, nkv, max_splits, group, 2]
// (scratch, needed when max_splits > 1); status: int32, set non-zero if a wait expired.
extern "C" int dl_attention_decode_bf16(const void* q, int q_stride, void* out, int out_stride, const void* k_pool,
                                        const void* v_pool, int n_pages, const int32_t* seq_len,
                                        const int32_t* block_table, int bt_stride, int n_seqs, int nh, int nkv,
                                        int hd, float scale, int window, int keys_per_split, int max_splits,
                                        float* part_o, float* part_ml, int* status, void* stream) {
    DL_REQUIRE(n_seqs >= 0 && nh > 0 && nkv > 0 && nh % nkv == 0, "attention_decode: bad head counts");
    DL_REQUIRE(nh / nkv <= 16, "attention_decode: groups of more than 16 query heads are not supported (%d)", nh / nkv);
    DL_REQUIRE(scale > 0.f, "attention_decode: the score scale must be positive");
    DL_REQUIRE(keys_per_split >= DL_PAGE && keys_per_split % DL_PAGE == 0, "attention_decode: keys_per_split %d must be a multiple of %d", keys_per_split, DL_PAGE);
    DL_REQUIRE(max_splits >= 1 && (max_splits == 1 || (part_o && part_ml)), "attention_decode: split runs need scratch");
    DL_REQUIRE(status != nullptr, "attention_decode: needs a status word");
    DL_REQUIRE(q_stride % 8 == 0 && ((uintptr_t)q % 16) == 0 && ((uintptr_t)k_pool % 16) == 0 && ((uintptr_t)v_pool % 16) == 0,
               "attention_decode: q and the pools must be 16-byte aligned");
    DL_REQUIRE((long long)n_seqs * nkv * max_splits < (1ll << 30) && n_seqs <= 65535, "attention_decode: too many runs");
    if (n_seqs == 0) return DL_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const bool wide = nh / nkv > 8;
#define AD_CASE(HDV)                                                                                                   \
    if (hd == HDV) {                                                                                                   \
        if (wide)                                                                                                      \
            return ad_launch<HDV, true>(s, q, q_stride, out, out_stride, k_pool, v_pool, n_pages, seq_len, block_table, \
                                        bt_stride, n_seqs, max_splits, nh, nkv, scale, window, keys_per_split, part_o, \
                                        part_ml, status);                                                              \
        return ad_launch<HDV, false>(s, q, q_stride, out, out_stride, k_pool, v_pool, n_pages, seq_len, block_table,   \
                                     bt_stride, n_seqs, max_splits, nh, nkv, scale, window, keys_per_split, part_o,    \
                                     part_ml, status);                                                                 \
    }
    AD_CASE(32) AD_CASE(64) AD_CASE(96) AD_CASE(128)
#undef AD_CASE
    return dl_fail(DL_ERR_UNSUPPORTED, "attention_decode: head_dim %d (takes 32, 64, 96, 128)", hd);
}
