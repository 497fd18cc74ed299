// Decode attention: one new token per sequence over its paged bfloat16 cache, split over keys.
//
// Role of the reference's attention_f16 with seq_q == 1 (native/kernels/attention.cu:19-197): scores
// scaled by 1/sqrt(hd), softmax with the running maximum subtracted, weighted sum of values, query
// head h reading KV head h / group.  A decode step is bound by the bytes of K and V, so each
// (sequence, KV head) is cut into runs of pages, and all query heads of the group share every key
// and value that is loaded: the group's heads are the rows of mma.sync.m16n8k16 tiles (rows beyond
// the group are zero).
//
// Shape: persistent, warp-specialised, stream-K.  The step's work is the list of all visible cache
// pages ordered by (sequence, KV head, page); it is cut into equal contiguous shares, one per block
// (one block per multiprocessor), whatever the lengths of the sequences are - the kernel computes
// the cut itself from the lengths on the device, so a captured launch serves any lengths.  A share
// is a few segments, each a run of pages of one (sequence, KV head).  A cache page of one KV head
// is two contiguous pieces (K [64][hd], V [hd][64]); one producer thread copies them with
// cp.async.bulk (the bulk-copy engine) into a ring of shared-memory stages, signalling an mbarrier
// per stage, and runs ahead of the arithmetic by the depth of the ring, across segment boundaries,
// at no cost in registers.  Consumer warp w takes pages w, w + C, ... of the stream; at the end of a
// segment the warps merge their partial results in shared memory and the block writes either the
// output (the segment was the whole pair) or the segment's partial (max, sum, weighted values) and
// counts itself in; the block that brings a pair's last missing segment merges the pair's segments in
// block order and writes the output (no second kernel, and the same bits whoever arrives last).
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

// The ring has `depth` stages per consumer warp: page n of a block's stream goes to stage n % (warps *
// depth) and to warp n % warps, so warp w owns stages w, w + warps, ... and sees every phase of their
// barriers in order.  (A warp that shared stages with others could fall two phases behind a barrier and
// mistake an old completion for the one it waits for: mbarrier waits tell phases apart by parity only.)
// A stage is asked for again only when its warp has used it up, so the bytes a multiprocessor has in
// flight are the ring's: with the 32 KB pages of head size 128 six stages fill the shared memory; the
// smaller pages of smaller heads take a deeper ring, or the copies' latency bounds the kernel
// (head size 64, depth 1: 96 KB in flight, 2.9 TB/s over the whole GPU).
#ifndef AD_MAX_STAGES
#define AD_MAX_STAGES 6                        // consumer warps, as many as fit in shared memory
#endif
#define AD_MAX_DEPTH 4                         // ring stages per consumer warp, at most
#define AD_MAX_RING (AD_MAX_STAGES * AD_MAX_DEPTH)
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
// The pages are read once per step and together exceed the L2: they are brought in to be evicted
// first, so that what the step reads again (queries, tables, partial results, the kernels' code) stays.
__device__ __forceinline__ uint64_t ad_stream_policy() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ void ad_bulk_copy(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(ad_smem(dst)),
                 "l"(src), "r"(bytes), "r"(ad_smem(bar)), "l"(policy)
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

// Pages of a sequence that its newest token sees (from the page of the first visible key).  A length
// of 0 marks a row that holds nothing (an idle row of a captured step wider than its batch): it has
// no pages, so no block walks it, nothing is read or written for it and its output row stays as it was.
__device__ __forceinline__ int ad_first_key(int len, int window) { return (window > 0 && len - window > 0) ? len - window : 0; }
__device__ __forceinline__ int ad_pages_of(int len, int window) {
    if (len <= 0) return 0;
    return (len - 1) / DL_PAGE - ad_first_key(len, window) / DL_PAGE + 1;
}

// The work of a step is the list of all visible pages, ordered by (sequence, KV head, page), cut into
// equal contiguous shares, one per block.  AdCut is that cut, computed by every warp for itself.
struct AdCut {
    int total, share;        // pages in the step, pages per block
};

__device__ __forceinline__ AdCut ad_cut(const int32_t* seq_len, int n_seqs, int nkv, int window, int n_blocks, int lane) {
    int sum = 0;
    for (int b0 = 0; b0 < n_seqs; b0 += 32)
        if (b0 + lane < n_seqs) sum += ad_pages_of(seq_len[b0 + lane], window);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    AdCut c;
    c.total = sum * nkv;
    c.share = max(1, (c.total + n_blocks - 1) / n_blocks);
    return c;
}

// The sequence that holds page r of the list (r < total), and the pages of the list before it.
__device__ __forceinline__ void ad_locate(const int32_t* seq_len, int n_seqs, int nkv, int window, int r, int lane,
                                          int* b_out, int* before_out) {
    int before = 0, b = n_seqs, b_before = 0;
    for (int b0 = 0; b0 < n_seqs; b0 += 32) {
        const int np = (b0 + lane < n_seqs) ? ad_pages_of(seq_len[b0 + lane], window) * nkv : 0;
        int incl = np;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int up = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += up;
        }
        const unsigned hit = __ballot_sync(0xffffffffu, before + incl > r);
        if (hit) {
            const int src = __ffs(hit) - 1;
            b = b0 + src;
            b_before = before + __shfl_sync(0xffffffffu, incl - np, src);
            break;
        }
        before += __shfl_sync(0xffffffffu, incl, 31);
    }
    *b_out = b;
    *before_out = b_before;
}

// A block's walk over its share: segments of one (sequence, KV head) each.
struct AdWalk {
    int r, r_end;            // next page of the list, end of the share
    int b, kvh, pg;          // where r lies: sequence, KV head, page among the sequence's visible pages
    int len, np;             // of sequence b: keys, visible pages
    bool first;              // the next segment is the block's first
};
struct AdSeg {
    int b, kvh, len, first_key, run_begin, page0, n_pages, slot;
    int pair_begin, pair_pages;      // where the (sequence, KV head)'s pages start in the step's list, and how many they are
    bool whole;
};

__device__ __forceinline__ AdWalk ad_walk_begin(const AdCut& c, const int32_t* seq_len, int n_seqs, int nkv, int window,
                                                int block, int lane) {
    AdWalk w;
    w.r = min(c.total, block * c.share);
    w.r_end = min(c.total, w.r + c.share);
    w.first = true;
    w.b = n_seqs;
    w.kvh = w.pg = w.len = w.np = 0;
    if (w.r < w.r_end) {
        int before;
        ad_locate(seq_len, n_seqs, nkv, window, w.r, lane, &w.b, &before);
        if (w.b >= n_seqs) {                                 // cannot happen while r < total
            w.r = w.r_end;
            return w;
        }
        w.len = seq_len[w.b];
        w.np = ad_pages_of(w.len, window);
        const int off = w.r - before;
        w.kvh = off / w.np;
        w.pg = off - w.kvh * w.np;
    }
    return w;
}

// The next segment of the walk; false when the share is used up.
__device__ __forceinline__ bool ad_walk_next(AdWalk& w, AdSeg& s, const int32_t* seq_len, int n_seqs, int nkv, int window) {
    if (w.r >= w.r_end || w.b >= n_seqs) return false;
    const int n = min(w.np - w.pg, w.r_end - w.r);
    s.b = w.b;
    s.kvh = w.kvh;
    s.len = w.len;
    s.first_key = ad_first_key(w.len, window);
    s.page0 = s.first_key / DL_PAGE + w.pg;
    s.run_begin = s.page0 * DL_PAGE;
    s.n_pages = n;
    s.whole = (w.pg == 0 && n == w.np);
    s.pair_begin = w.r - w.pg;
    s.pair_pages = w.np;
    s.slot = w.first ? 0 : 1;
    w.first = false;
    w.r += n;
    w.pg += n;
    if (w.pg == w.np) {
        w.pg = 0;
        if (++w.kvh == nkv) {
            w.kvh = 0;
            do {                                             // the next sequence that has pages
                ++w.b;
                w.len = w.b < n_seqs ? seq_len[w.b] : 0;
                w.np = ad_pages_of(w.len, window);
            } while (w.b < n_seqs && w.np == 0);
        }
    }
    return true;
}

// The step's own token, when the caller has not rotated it and written it to the cache yet: the
// kernel then rotates q as it loads it and puts the new key and value into the newest page itself
// (in the shared-memory stage and in the cache), so that no separate kernel has to run before it.
// k == nullptr: q is rotated and the cache is complete already.
struct AdFresh {
    const __nv_bfloat16* k;          // [B, nkv*hd] rows k_stride apart, unrotated
    int k_stride;
    const __nv_bfloat16* v;          // [B, nkv*hd] rows v_stride apart
    int v_stride;
    const float* cos_t;              // [table_rows, hd/2] (rotate != 0)
    const float* sin_t;
    int table_rows;
    int rotate;                      // 0: no rotation (the mixer encoded positions itself)
};

// The same roundings as the rope kernels (no contraction), so that the fused and the separate way
// give the same bits.
__device__ __forceinline__ float ad_rot_lo(float x0, float x1, float c, float s) { return __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s)); }
__device__ __forceinline__ float ad_rot_hi(float x0, float x1, float c, float s) { return __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c)); }

// Rotate the 8 dims of a low-half piece (x0) and its partner in the high half (x1) in place.
__device__ __forceinline__ void ad_rotate8(uint4& x0, uint4& x1, const float* cs, const float* sn) {
    const float4 c0 = *reinterpret_cast<const float4*>(cs), c1 = *reinterpret_cast<const float4*>(cs + 4);
    const float4 s0 = *reinterpret_cast<const float4*>(sn), s1 = *reinterpret_cast<const float4*>(sn + 4);
    const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float sv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    __nv_bfloat16* a = reinterpret_cast<__nv_bfloat16*>(&x0);
    __nv_bfloat16* b = reinterpret_cast<__nv_bfloat16*>(&x1);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const float f0 = __bfloat162float(a[e]), f1 = __bfloat162float(b[e]);
        a[e] = __float2bfloat16_rn(ad_rot_lo(f0, f1, c[e], sv[e]));
        b[e] = __float2bfloat16_rn(ad_rot_hi(f0, f1, c[e], sv[e]));
    }
}

// Merge the segments of one (sequence, KV head) that the cut spread over the blocks i0 .. i0 + n_seg - 1,
// in block order, and write the group's heads.  The pair's first segment sits in its block's first or
// last slot (`slot_first`), every other segment in its block's first.  Called by the consumer threads
// of the block that wrote the pair's last missing segment; thread -> (head of the group, four dims);
// the loads of up to BATCH segments are issued together and bypass the L1 (other multiprocessors wrote them).
template <int HD, int BATCH>
__device__ __forceinline__ void ad_merge_pair(__nv_bfloat16* __restrict__ out_pair, int group, int i0, int n_seg, int slot_first,
                                              const float* __restrict__ part_o, const float* __restrict__ part_ml, int tid,
                                              int n_threads) {
    constexpr int hd4 = HD / 4;
    for (int idx = tid; idx < group * hd4; idx += n_threads) {
        const int r = idx / hd4, d = (idx - r * hd4) * 4;
        float m = -INFINITY, l = 0.f;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int sp0 = 0; sp0 < n_seg; sp0 += BATCH) {
            float2 ml[BATCH];
            float4 o[BATCH];
#pragma unroll
            for (int j = 0; j < BATCH; ++j) {
                if (sp0 + j < n_seg) {
                    const int slot = (sp0 + j == 0) ? slot_first : 0;
                    const size_t row = ((size_t)(i0 + sp0 + j) * 2 + slot) * group + r;
                    ml[j] = __ldcg(reinterpret_cast<const float2*>(part_ml + row * 2));
                    o[j] = __ldcg(reinterpret_cast<const float4*>(part_o + row * HD + d));
                }
            }
#pragma unroll
            for (int j = 0; j < BATCH; ++j) {
                if (sp0 + j < n_seg) {
                    const float mn = fmaxf(m, ml[j].x);
                    const float f_old = (m == -INFINITY) ? 0.f : ad_ex2(m - mn);
                    const float f_new = (ml[j].x == -INFINITY) ? 0.f : ad_ex2(ml[j].x - mn);
                    acc.x = acc.x * f_old + o[j].x * f_new;
                    acc.y = acc.y * f_old + o[j].y * f_new;
                    acc.z = acc.z * f_old + o[j].z * f_new;
                    acc.w = acc.w * f_old + o[j].w * f_new;
                    l = l * f_old + ml[j].y * f_new;
                    m = mn;
                }
            }
        }
        const float inv = 1.f / l;
        __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
        __nv_bfloat162 hi = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
        uint2 packed;
        packed.x = *reinterpret_cast<uint32_t*>(&lo);
        packed.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(out_pair + (size_t)r * HD + d) = packed;
    }
}

// WIDE: the group has more than 8 query heads, so fragment rows 8..15 carry data too.
template <int HD, bool WIDE>
__global__ void __launch_bounds__(AD_THREADS, 1)
attention_decode_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, __nv_bfloat16* __restrict__ out,
                        int out_stride, __nv_bfloat16* __restrict__ k_pool,
                        __nv_bfloat16* __restrict__ v_pool, int n_pages,
                        const int32_t* __restrict__ seq_len, const int32_t* __restrict__ block_table,
                        int bt_stride, int n_seqs, int nh, int nkv, float scale, int window, int n_stages, int n_ring,
                        float* __restrict__ part_o,
                        float* __restrict__ part_ml, int* __restrict__ pair_counters, const AdFresh fresh,
                        int* __restrict__ status) {
    constexpr int DC = HD / 32;          // 32-dim slices of a head
    constexpr int DT = HD / 8;           // 8-dim output tiles
    constexpr int PAGE_ELEMS = DL_PAGE * HD;
    constexpr uint32_t PAGE_BYTES = PAGE_ELEMS * 2;
    extern __shared__ __align__(128) unsigned char ad_smem_raw[];
    __nv_bfloat16* stage_mem = reinterpret_cast<__nv_bfloat16*>(ad_smem_raw);      // [stage][K page | V page]
    const int group = nh / nkv;
    // after the stages: each consumer warp's partial output [group][HD + 4]
    // n_stages: consumer warps; n_ring: stages of the ring, a multiple of n_stages
    float* merge_o = reinterpret_cast<float*>(ad_smem_raw + (size_t)n_ring * 2 * PAGE_BYTES);
    __shared__ uint64_t full_bar[AD_MAX_RING], empty_bar[AD_MAX_RING];
    __shared__ float sm_m[AD_MAX_STAGES][16], sm_l[AD_MAX_STAGES][16];
    __shared__ volatile int gave_up;
    __shared__ int last_of_pair;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    // The kernel checks its own shared-memory layout: if the launch gave it less dynamic shared
    // memory than the stages and merge buffers need, it records status 11 and touches nothing.
    uint32_t smem_bytes;
    asm("mov.u32 %0, %dynamic_smem_size;" : "=r"(smem_bytes));
    const uint32_t smem_lo = ad_smem(ad_smem_raw), smem_hi = smem_lo + smem_bytes;
    if ((size_t)n_ring * 2 * PAGE_BYTES + (size_t)n_stages * group * (HD + 4) * 4 > smem_bytes || n_ring > AD_MAX_RING ||
        n_stages > AD_MAX_STAGES || n_ring % n_stages != 0) {
        if (threadIdx.x == 0) atomicExch(status, 11);
        return;
    }

    if (threadIdx.x == 0) {
        gave_up = 0;
        for (int s = 0; s < n_ring; ++s) {
            ad_mbar_init(&full_bar[s], 1);
            ad_mbar_init(&empty_bar[s], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    dl_launch_dependents();

    if (warp == AD_MAX_STAGES) {
        // ------------------------------------------------------------ producer
        // The warp reads 32 page ids at a time (one coalesced load); lane 0 issues the copies.
        // Of what this kernel reads, the kernel launched before it writes only q and each sequence's
        // newest cache page (lengths and block tables are staged before the step's first kernel).
        // So the producer starts on older pages at once and waits for that kernel only before it
        // copies a newest page: the ring fills while the kernel before is still finishing.  (When this
        // kernel writes the new token itself, the copy of a newest page just brings a stale slot that
        // the consumer overwrites in the stage, and the producer never waits.)
        int n = 0;                                           // pages issued so far, over all runs
        bool stop = false, waited = false;
        const uint64_t policy = ad_stream_policy();
        const AdCut cut = ad_cut(seq_len, n_seqs, nkv, window, gridDim.x, lane);
        AdWalk walk = ad_walk_begin(cut, seq_len, n_seqs, nkv, window, blockIdx.x, lane);
        AdSeg w;
        while (!stop && ad_walk_next(walk, w, seq_len, n_seqs, nkv, window)) {
            const int32_t* pages = block_table + (size_t)w.b * bt_stride + w.page0;
            for (int i0 = 0; i0 < w.n_pages && !stop; i0 += 32) {
                const int mine = (i0 + lane < w.n_pages) ? pages[i0 + lane] : 0;
                const int count = min(32, w.n_pages - i0);
                for (int j = 0; j < count; ++j, ++n) {
                    const int page = __shfl_sync(0xffffffffu, mine, j);
                    int bad = 0;
                    if (lane == 0) {
                        const int s = n % n_ring;
                        if (page < 0 || page >= n_pages) {   // host-validated
                            bad = 2;
                        } else if (n >= n_ring && !ad_mbar_wait(&empty_bar[s], ((n / n_ring) - 1) & 1, &gave_up)) {
                            bad = 1;
                        } else {
                            if (!waited && fresh.k == nullptr && w.page0 + i0 + j == (w.len - 1) / DL_PAGE) {
                                dl_grid_dependency_wait();
                                waited = true;
                            }
                            __nv_bfloat16* dst = stage_mem + (size_t)s * 2 * PAGE_ELEMS;
                            ad_mbar_expect(&full_bar[s], 2 * PAGE_BYTES);
                            ad_bulk_copy(dst, k_pool + dl_k_offset(page, nkv, w.kvh, 0, HD), PAGE_BYTES, &full_bar[s], policy);
                            ad_bulk_copy(dst + PAGE_ELEMS, v_pool + dl_v_offset(page, nkv, w.kvh, 0, HD), PAGE_BYTES, &full_bar[s], policy);
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
            for (int i = max(0, n - n_ring); i < n; ++i) {
                const long long t0 = clock64();
                while (!ad_mbar_try(&full_bar[i % n_ring], (i / n_ring) & 1) && clock64() - t0 < AD_WAIT_CYCLES) {}
            }
        }
    } else if (warp < n_stages) {
        // ------------------------------------------------------------ consumers (warp w owns stages w, w + n_stages, ...)
        // The cut needs the lengths only, which are older than the kernel before this one: it is made
        // while that kernel finishes, and q is waited for after it.
        float* my_o = merge_o + (size_t)warp * group * (HD + 4);
        const float scale2 = scale * 1.4426950408889634f;    // scores in units of log2
        int n0 = 0;                                          // pages of the runs before this one
        const AdCut cut = ad_cut(seq_len, n_seqs, nkv, window, gridDim.x, lane);
        AdWalk walk = ad_walk_begin(cut, seq_len, n_seqs, nkv, window, blockIdx.x, lane);
        AdSeg w;
        dl_grid_dependency_wait();       // q comes from the kernel before this one; out and the scratch may be in use by it
        while (ad_walk_next(walk, w, seq_len, n_seqs, nkv, window)) {      // the same segments in every warp
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
                if (fresh.k != nullptr && fresh.rotate) {
                    // slice c of the low half pairs with slice c + DC/2 of the high half, same lane
                    const int pos = min(w.len - 1, fresh.table_rows - 1);        // host-validated
                    const float* cs = fresh.cos_t + (size_t)pos * (HD / 2);
                    const float* sn = fresh.sin_t + (size_t)pos * (HD / 2);
#pragma unroll
                    for (int c = 0; c < DC / 2; ++c) {
                        ad_rotate8(qf_lo[c], qf_lo[c + DC / 2], cs + c * 32 + t * 8, sn + c * 32 + t * 8);
                        if (WIDE) ad_rotate8(qf_hi[c], qf_hi[c + DC / 2], cs + c * 32 + t * 8, sn + c * 32 + t * 8);
                    }
                }
            }
            float o[DT][4];
#pragma unroll
            for (int i = 0; i < DT; ++i)
#pragma unroll
                for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
            float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;   // maxima in units of log2

            const int i_first = ((warp - n0) % n_stages + n_stages) % n_stages;   // first i with (n0 + i) % n_stages == warp
            // The warp that will meet the page of the step's own token asks for that token's key, value
            // and table rows now, so that they are in registers when the page arrives.
            const int i_new = fresh.k != nullptr ? (w.len - 1) / DL_PAGE - w.page0 : -1;
            const bool mine_new = i_new >= 0 && i_new < w.n_pages && (n0 + i_new) % n_stages == warp;
            uint2 kn_lo = make_uint2(0u, 0u), kn_hi = make_uint2(0u, 0u);
            float4 kn_c = make_float4(1.f, 1.f, 1.f, 1.f), kn_s = make_float4(0.f, 0.f, 0.f, 0.f);
            __nv_bfloat16 vn_r[HD / 32];
            if (mine_new) {
                const __nv_bfloat16* kn = fresh.k + (size_t)w.b * fresh.k_stride + (size_t)w.kvh * HD;
                const __nv_bfloat16* vn = fresh.v + (size_t)w.b * fresh.v_stride + (size_t)w.kvh * HD;
                const int pos = min(w.len - 1, fresh.table_rows - 1);
                if (lane * 4 < HD / 2) {                         // four rotation pairs per lane (HD <= 256)
                    kn_lo = *reinterpret_cast<const uint2*>(kn + lane * 4);
                    kn_hi = *reinterpret_cast<const uint2*>(kn + HD / 2 + lane * 4);
                    if (fresh.rotate) {
                        kn_c = *reinterpret_cast<const float4*>(fresh.cos_t + (size_t)pos * (HD / 2) + lane * 4);
                        kn_s = *reinterpret_cast<const float4*>(fresh.sin_t + (size_t)pos * (HD / 2) + lane * 4);
                    }
                }
#pragma unroll
                for (int j = 0; j < HD / 32; ++j) vn_r[j] = vn[lane + 32 * j];
            }
            for (int i = i_first; i < w.n_pages; i += n_stages) {
                const int n = n0 + i;
                const int s = n % n_ring;
                if (!ad_mbar_wait(&full_bar[s], (n / n_ring) & 1, &gave_up)) {
                    if (!gave_up) atomicExch(status, 3);
                    gave_up = 1;
                    continue;                                 // keep walking so that every barrier below is reached
                }
                const int base = w.run_begin + i * DL_PAGE;  // first key of the page
                __nv_bfloat16* kp = stage_mem + (size_t)s * 2 * PAGE_ELEMS;
                __nv_bfloat16* vp = kp + PAGE_ELEMS;
                const bool ragged = (base + DL_PAGE > w.len) || (base < w.first_key);
                if (fresh.k != nullptr && base <= w.len - 1 && w.len - 1 < base + DL_PAGE) {
                    // The page of the step's own token: its slot is stale in the copy that arrived.  Put the
                    // (rotated) key and the value there, in the stage and in the cache.
                    const int in_page = (w.len - 1) - base;
                    const int page = block_table[(size_t)w.b * bt_stride + (w.len - 1) / DL_PAGE];
                    if (lane * 4 < HD / 2) {
                        const int i4 = lane * 4;
                        __nv_bfloat16 lo[4], hi[4];
                        *reinterpret_cast<uint2*>(lo) = kn_lo;
                        *reinterpret_cast<uint2*>(hi) = kn_hi;
                        if (fresh.rotate) {
                            const float cc[4] = {kn_c.x, kn_c.y, kn_c.z, kn_c.w}, ss[4] = {kn_s.x, kn_s.y, kn_s.z, kn_s.w};
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const float f0 = __bfloat162float(lo[e]), f1 = __bfloat162float(hi[e]);
                                lo[e] = __float2bfloat16_rn(ad_rot_lo(f0, f1, cc[e], ss[e]));
                                hi[e] = __float2bfloat16_rn(ad_rot_hi(f0, f1, cc[e], ss[e]));
                            }
                        }
                        *reinterpret_cast<uint2*>(kp + in_page * HD + i4) = *reinterpret_cast<uint2*>(lo);
                        *reinterpret_cast<uint2*>(kp + in_page * HD + HD / 2 + i4) = *reinterpret_cast<uint2*>(hi);
                        if (page >= 0 && page < n_pages) {
                            __nv_bfloat16* kg = k_pool + dl_k_offset(page, nkv, w.kvh, in_page, HD);
                            *reinterpret_cast<uint2*>(kg + i4) = *reinterpret_cast<uint2*>(lo);
                            *reinterpret_cast<uint2*>(kg + HD / 2 + i4) = *reinterpret_cast<uint2*>(hi);
                        }
                    }
#pragma unroll
                    for (int j = 0; j < HD / 32; ++j) {
                        const int d = lane + 32 * j;
                        vp[d * DL_PAGE + in_page] = vn_r[j];
                        if (page >= 0 && page < n_pages) v_pool[dl_v_offset(page, nkv, w.kvh, d, HD) + in_page] = vn_r[j];
                    }
                    __syncwarp();
                }
                if (ragged) {
                    // Keys outside [first, len) may hold anything (even NaN): make their values exact
                    // zeros in the stage once, so that the product below needs no special case.
                    // The invalid keys are a run at the page's start (older than the window) and a run at
                    // its end (beyond the sequence): each lane clears those runs in its rows of V, eight
                    // keys (16 bytes) at a time where a run covers whole groups of eight.
                    const int lo_end = min(DL_PAGE, max(0, w.first_key - base));       // keys [0, lo_end) are too old
                    const int hi_begin = max(0, min(DL_PAGE, w.len - base));             // keys [hi_begin, 64) do not exist yet
                    for (int d = lane; d < HD; d += 32) {
                        __nv_bfloat16* row = vp + d * DL_PAGE;
                        for (int k = 0; k < lo_end; ++k) row[k] = __float2bfloat16_rn(0.f);
                        int k = hi_begin;
                        for (; k < DL_PAGE && (k & 7); ++k) row[k] = __float2bfloat16_rn(0.f);
                        for (; k < DL_PAGE; k += 8) *reinterpret_cast<uint4*>(row + k) = make_uint4(0u, 0u, 0u, 0u);
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
                                if (key < w.first_key || key >= w.len) {
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
                // The stage may be released only after every MMA fed from it has been issued (an MMA
                // issues when its operands have arrived from shared memory).  The MMAs are not
                // volatile, so pin their results here: the compiler cannot sink them below this point.
#pragma unroll
                for (int i2 = 0; i2 < DT; ++i2) asm volatile("" : "+f"(o[i2][0]), "+f"(o[i2][1]), "+f"(o[i2][2]), "+f"(o[i2][3]));
                // ... and the reads themselves must be done before the copy engine may overwrite the stage:
                // without this fence a slot that was refilled at once showed rows of the new chunk to the old reads.
                __threadfence_block();
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
            const size_t part_row = ((size_t)blockIdx.x * 2 + w.slot) * group;
            // thread -> (row of the group, four dims): the warps' factors once per thread, float4 loads
            for (int idx = tid; idx < group * (HD / 4); idx += 32 * n_stages) {
                const int r = idx / (HD / 4), d = (idx - r * (HD / 4)) * 4;
                float m = -INFINITY;
#pragma unroll
                for (int cw = 0; cw < AD_MAX_STAGES; ++cw)
                    if (cw < n_stages) m = fmaxf(m, sm_m[cw][r]);
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                float l = 0.f;
#pragma unroll
                for (int cw = 0; cw < AD_MAX_STAGES; ++cw) {  // warp order: fixed
                    if (cw < n_stages) {
                        const float f = (sm_m[cw][r] == -INFINITY) ? 0.f : ad_ex2(sm_m[cw][r] - m);
                        const float4 o4 = *reinterpret_cast<const float4*>(merge_o + ((size_t)cw * group + r) * (HD + 4) + d);
                        acc.x += o4.x * f, acc.y += o4.y * f, acc.z += o4.z * f, acc.w += o4.w * f;
                        l += sm_l[cw][r] * f;
                    }
                }
                if (w.whole) {
                    const float inv = 1.f / l;
                    __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
                    __nv_bfloat162 hi = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
                    uint2 packed;
                    packed.x = *reinterpret_cast<uint32_t*>(&lo);
                    packed.y = *reinterpret_cast<uint32_t*>(&hi);
                    *reinterpret_cast<uint2*>(out + (size_t)w.b * out_stride + (size_t)(w.kvh * group + r) * HD + d) = packed;
                } else {
                    *reinterpret_cast<float4*>(part_o + (part_row + r) * HD + d) = acc;
                    if (d == 0) {
                        part_ml[(part_row + r) * 2] = m;
                        part_ml[(part_row + r) * 2 + 1] = l;
                    }
                }
            }
            ad_consumer_sync(n_stages);                              // the merge buffers are free for the next run
            if (!w.whole) {
                // The pair's pages are spread over the blocks i0 .. i1 of the cut.  Each of them counts itself
                // in once its segment is written (one acquire-release atomic: the consumer warps' stores
                // are ordered before it by the barrier above); whichever arrives last merges the
                // segments in block order - the same bits whatever the order of arrival.
                const int i0 = w.pair_begin / cut.share, i1 = (w.pair_begin + w.pair_pages - 1) / cut.share;
                if (tid == 0) {
                    int seen;
                    int* counter = pair_counters + w.b * nkv + w.kvh;
                    asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(seen) : "l"(counter) : "memory");
                    last_of_pair = (seen == i1 - i0) ? 1 : 0;
                    if (seen == i1 - i0) *counter = 0;               // ready for the next launch
                }
                ad_consumer_sync(n_stages);
                const bool last = last_of_pair != 0;
                ad_consumer_sync(n_stages);                          // everyone has read the flag before it is written again
                if (last)
                    ad_merge_pair<HD, WIDE ? 4 : 8>(out + (size_t)w.b * out_stride + (size_t)w.kvh * group * HD, group, i0, i1 - i0 + 1,
                                      (w.pair_begin == i0 * cut.share) ? 0 : 1, part_o, part_ml, tid, 32 * n_stages);
            }
        }
    }
    __syncthreads();                                         // nobody leaves while copies may still land
}

template <int HD, bool WIDE>
static int ad_launch(cudaStream_t s, const void* q, int q_stride, void* out, int out_stride, void* k_pool,
                     void* v_pool, int n_pages, const int32_t* seq_len, const int32_t* block_table,
                     int bt_stride, int n_seqs, int nh, int nkv, float scale, int window, int blocks, float* part_o,
                     float* part_ml, int part_slots, int* pair_counters, int n_counters, const AdFresh& fresh, int* status) {
    const int group = nh / nkv;
    int dev = 0, sms = 0, max_smem = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    const size_t stage = (size_t)2 * DL_PAGE * HD * 2;
    const size_t merge_per = (size_t)group * (HD + 4) * sizeof(float);     // one consumer warp's partial output
    int n_stages = AD_MAX_STAGES;                            // consumer warps
    while (n_stages > 2 && n_stages * (stage + merge_per) + 2048 > (size_t)max_smem) --n_stages;
    int depth = 1;                                           // ring stages per warp: what the shared memory holds
    while (depth < AD_MAX_DEPTH && n_stages * ((depth + 1) * stage + merge_per) + 2048 <= (size_t)max_smem) ++depth;
    const int n_ring = n_stages * depth;
    const size_t smem = n_stages * (depth * stage + merge_per);
    if (smem + 2048 > (size_t)max_smem)
        return dl_fail(DL_ERR_UNSUPPORTED, "attention_decode: head_dim %d with %d heads per group needs %zu bytes of shared memory", HD, group, smem);
    static int configured = 0;
    if (configured < (int)smem) {
        cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<HD, WIDE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "attention_decode: shared memory %zu: %s", smem, cudaGetErrorString(e));
        configured = (int)smem;
    }
    // One block per multiprocessor unless the caller asks for fewer, and never more than there can be pages.
    if (blocks <= 0 || blocks > sms) blocks = sms;
    const long long most_pages = (long long)n_seqs * nkv * bt_stride;
    if (blocks > most_pages) blocks = (int)most_pages;
    if (part_slots < 2 * blocks)
        return dl_fail(DL_ERR_ARGUMENT, "attention_decode: scratch for %d segments, %d blocks need %d", part_slots, blocks, 2 * blocks);
    if (pair_counters == nullptr || (long long)n_seqs * nkv > n_counters)
        return dl_fail(DL_ERR_ARGUMENT, "attention_decode: %d counters, %d sequences x %d KV heads need one each", n_counters, n_seqs, nkv);
    cudaError_t le = dl_launch_dependent(
        attention_decode_kernel<HD, WIDE>, dim3(blocks), dim3(AD_THREADS), smem, s, (const __nv_bfloat16*)q, q_stride,
        (__nv_bfloat16*)out, out_stride, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, n_pages, seq_len,
        block_table, bt_stride, n_seqs, nh, nkv, scale, window, n_stages, n_ring, part_o, part_ml, pair_counters, fresh, status);
    if (le != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "attention_decode: %s", cudaGetErrorString(le));
    return DL_OK;
}

// q: bf16 [B, nh*hd] rows q_stride apart (one token per sequence); out likewise.
// seq_len[b]: keys of sequence b including the new token; block_table: int32 [B, bt_stride] page ids.
// blocks: persistent blocks to use (<= 0: one per multiprocessor).
// part_o: float32 [part_slots, group, hd]; part_ml: float32 [part_slots, group, 2]: scratch for the
// segments of (sequence, head) pairs that the cut spreads over several blocks, two per block.
// pair_counters: int32 [n_counters >= n_seqs * nkv], zero before the first launch; every launch leaves
// them zero (launches that share them must be on one stream).
// status: int32, set non-zero if a wait expired.
// Launched with programmatic dependent launch: of this call's inputs, a kernel of this library
// launched directly before it may write only q and the newest page of each sequence (the rope and
// cache-write kernel does); lengths, block tables and older pages must be complete by then.
static int ad_dispatch(const void* q, int q_stride, void* out, int out_stride, void* k_pool, void* v_pool, int n_pages,
                       const int32_t* seq_len, const int32_t* block_table, int bt_stride, int n_seqs, int nh, int nkv, int hd,
                       float scale, int window, int blocks, float* part_o, float* part_ml, int part_slots, int* pair_counters,
                       int n_counters, const AdFresh& fresh, int* status, void* stream) {
    DL_REQUIRE(n_seqs >= 0 && nh > 0 && nkv > 0 && nh % nkv == 0, "attention_decode: bad head counts");
    DL_REQUIRE(nh / nkv <= 16, "attention_decode: groups of more than 16 query heads are not supported (%d)", nh / nkv);
    DL_REQUIRE(scale > 0.f, "attention_decode: the score scale must be positive");
    DL_REQUIRE(part_o && part_ml && part_slots >= 2, "attention_decode: needs scratch for the cut segments");
    DL_REQUIRE(status != nullptr, "attention_decode: needs a status word");
    DL_REQUIRE(bt_stride >= 1 && window >= 0, "attention_decode: bad block table stride or window");
    DL_REQUIRE(out_stride % 4 == 0 && ((uintptr_t)out % 8) == 0, "attention_decode: out must be 8-byte aligned");
    DL_REQUIRE(q_stride % 8 == 0 && ((uintptr_t)q % 16) == 0 && ((uintptr_t)k_pool % 16) == 0 && ((uintptr_t)v_pool % 16) == 0,
               "attention_decode: q and the pools must be 16-byte aligned");
    DL_REQUIRE((long long)n_seqs * nkv * bt_stride < (1ll << 30) && n_seqs <= 65535, "attention_decode: too many pages");
    if (fresh.k != nullptr) {
        DL_REQUIRE(fresh.v != nullptr && fresh.k_stride % 4 == 0 && fresh.v_stride % 4 == 0 && ((uintptr_t)fresh.k % 8) == 0 &&
                       ((uintptr_t)fresh.v % 8) == 0 && fresh.k_stride >= nkv * hd && fresh.v_stride >= nkv * hd,
                   "attention_decode: the new keys and values must be 8-byte aligned rows of nkv*hd");
        DL_REQUIRE(!fresh.rotate || ((hd == 64 || hd == 128) && fresh.cos_t && fresh.sin_t && fresh.table_rows > 0 &&
                                     ((uintptr_t)fresh.cos_t % 16) == 0 && ((uintptr_t)fresh.sin_t % 16) == 0),
                   "attention_decode: rotating inside the kernel takes head_dim 64 or 128 and 16-byte aligned tables");
    }
    if (n_seqs == 0) return DL_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const bool wide = nh / nkv > 8;
#define AD_CASE(HDV)                                                                                                   \
    if (hd == HDV) {                                                                                                   \
        if (wide)                                                                                                      \
            return ad_launch<HDV, true>(s, q, q_stride, out, out_stride, k_pool, v_pool, n_pages, seq_len, block_table, \
                                        bt_stride, n_seqs, nh, nkv, scale, window, blocks, part_o, part_ml, part_slots, \
                                        pair_counters, n_counters, fresh, status);                                     \
        return ad_launch<HDV, false>(s, q, q_stride, out, out_stride, k_pool, v_pool, n_pages, seq_len, block_table,   \
                                     bt_stride, n_seqs, nh, nkv, scale, window, blocks, part_o, part_ml, part_slots,   \
                                     pair_counters, n_counters, fresh, status);                                        \
    }
    AD_CASE(32) AD_CASE(64) AD_CASE(96) AD_CASE(128)
#undef AD_CASE
    return dl_fail(DL_ERR_UNSUPPORTED, "attention_decode: head_dim %d (takes 32, 64, 96, 128)", hd);
}

extern "C" int dl_attention_decode_bf16(const void* q, int q_stride, void* out, int out_stride, const void* k_pool,
                                        const void* v_pool, int n_pages, const int32_t* seq_len,
                                        const int32_t* block_table, int bt_stride, int n_seqs, int nh, int nkv,
                                        int hd, float scale, int window, int blocks, float* part_o, float* part_ml,
                                        int part_slots, int* pair_counters, int n_counters, int* status, void* stream) {
    AdFresh none = {};
    return ad_dispatch(q, q_stride, out, out_stride, const_cast<void*>(k_pool), const_cast<void*>(v_pool), n_pages, seq_len,
                       block_table, bt_stride, n_seqs, nh, nkv, hd, scale, window, blocks, part_o, part_ml, part_slots,
                       pair_counters, n_counters, none, status, stream);
}

// The same with the step's own token handled inside the kernel: q (unrotated), k_new and v_new
// ([B, nkv*hd] rows, unrotated) come straight from the projection; the kernel rotates q and k_new
// with the rotary tables (rotate != 0: cos, sin float32 [table_rows, hd/2], full-width rotation of
// head sizes 64 and 128; rotate == 0: no rotation), writes k_new and v_new into each sequence's
// newest page (position seq_len[b] - 1), and attends.  Replaces dl_rope_cache_write followed by
// dl_attention_decode_bf16 for a decode step, with the same bits.
extern "C" int dl_attention_decode_fresh_bf16(const void* q, int q_stride, const void* k_new, int k_stride, const void* v_new,
                                              int v_stride, const float* cos_t, const float* sin_t, int table_rows, int rotate,
                                              void* out, int out_stride, void* k_pool, void* v_pool, int n_pages,
                                              const int32_t* seq_len, const int32_t* block_table, int bt_stride, int n_seqs,
                                              int nh, int nkv, int hd, float scale, int window, int blocks, float* part_o,
                                              float* part_ml, int part_slots, int* pair_counters, int n_counters, int* status,
                                              void* stream) {
    DL_REQUIRE(k_new != nullptr && v_new != nullptr, "attention_decode_fresh: needs the new keys and values");
    AdFresh fresh;
    fresh.k = (const __nv_bfloat16*)k_new;
    fresh.k_stride = k_stride;
    fresh.v = (const __nv_bfloat16*)v_new;
    fresh.v_stride = v_stride;
    fresh.cos_t = cos_t;
    fresh.sin_t = sin_t;
    fresh.table_rows = table_rows;
    fresh.rotate = rotate;
    return ad_dispatch(q, q_stride, out, out_stride, k_pool, v_pool, n_pages, seq_len, block_table, bt_stride, n_seqs, nh, nkv,
                       hd, scale, window, blocks, part_o, part_ml, part_slots, pair_counters, n_counters, fresh, status, stream);
}
