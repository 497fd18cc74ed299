// Decode attention: one new token per sequence over its paged bfloat16 cache, split over keys.
//
// Role of the reference's attention_f16 with seq_q == 1 (native/kernels/attention.cu:19-197): scores
// scaled by 1/sqrt(hd), softmax with the running maximum subtracted, weighted sum of values, query
// head h reading KV head h / group.  A decode step is bound by the bytes of K and V, so each
// (sequence, KV head) is cut into runs of keys that separate blocks stream, and all query heads
// of the group share every key and value that is loaded: the group's heads are the rows of
// mma.sync.m16n8k16 tiles (rows beyond the group are zero).
//
// Registers only, no shared-memory staging.  A warp takes 32 keys at a time.  Lane (g, t) loads
// 16-byte pieces of K rows: dims 8t..8t+7 of a 32-dim slice are a consistent permutation of k for
// Q and K in two MMAs; the 8 key columns of score tile j are keys 8(g/2) + 2j + (g&1) of the run,
// so that after four tiles the lane holds scores of keys 8t..8t+7 - exactly the k-permutation
// that pairs with a 16-byte piece of a transposed V row (V pages are [dim][token]).  Softmax is
// float32 with exact expf.  Warps of a block, then the blocks of a (sequence, KV head), are merged
// in a fixed order; the last block to finish does the merge and writes bfloat16.
#include "common.cuh"

#define AD_WARPS 4

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

// Zero the bf16 elements of a 16-byte piece whose key index is >= limit (keys first, first+1, ...).
__device__ __forceinline__ uint4 ad_mask_keys(uint4 v, int first, int limit) {
    uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int k0 = first + 2 * i;
        if (k0 >= limit) w[i] = 0u;
        else if (k0 + 1 >= limit) w[i] &= 0x0000ffffu;
    }
    return v;
}

template <int HD>
__global__ void __launch_bounds__(32 * AD_WARPS)
attention_decode_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, __nv_bfloat16* __restrict__ out,
                        int out_stride, const __nv_bfloat16* __restrict__ k_pool,
                        const __nv_bfloat16* __restrict__ v_pool, int n_pages,
                        const int32_t* __restrict__ seq_len, const int32_t* __restrict__ block_table,
                        int bt_stride, int nh, int nkv, float scale, int window, int keys_per_split,
                        float* __restrict__ part_o, float* __restrict__ part_ml, int* __restrict__ counters) {
    constexpr int DC = HD / 32;          // 32-dim slices of a head
    constexpr int DT = HD / 8;           // 8-dim output tiles
    __shared__ float sm_o[AD_WARPS][16][HD + 4];
    __shared__ float sm_m[AD_WARPS][16], sm_l[AD_WARPS][16];
    __shared__ int is_last;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int group = nh / nkv;
    const int len = seq_len[b];                          // keys 0..len-1; the query sits at len-1
    const int first = (window > 0 && len - window > 0) ? len - window : 0;
    // runs are counted from the first visible key's page-aligned start
    const int origin = (first / DL_PAGE) * DL_PAGE;
    const int n_splits = (len - origin + keys_per_split - 1) / keys_per_split;
    if (split >= n_splits) return;
    const int run_begin = origin + split * keys_per_split;
    const int run_end = min(len, run_begin + keys_per_split);
    const int32_t* pages = block_table + (size_t)b * bt_stride;

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

    float o[DT][4];
#pragma unroll
    for (int i = 0; i < DT; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;

    for (int base = run_begin + warp * 32; base < run_end; base += AD_WARPS * 32) {
        const int page = pages[base / DL_PAGE];
        if (page < 0 || page >= n_pages) continue;       // host-validated; never read outside the pool
        const int in_page = base % DL_PAGE;              // 0 or 32
        const __nv_bfloat16* kp = k_pool + dl_k_offset(page, nkv, kvh, in_page, HD);
        const __nv_bfloat16* vp = v_pool + dl_v_offset(page, nkv, kvh, 0, HD) + in_page;

        // ---- S = Q K^T for 32 keys
        uint4 kf[4][DC];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int key = 8 * (g >> 1) + 2 * j + (g & 1);
#pragma unroll
            for (int c = 0; c < DC; ++c)
                kf[j][c] = __ldg(reinterpret_cast<const uint4*>(kp + (size_t)key * HD + c * 32 + t * 8));
        }
        float s[4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
#pragma unroll
            for (int c = 0; c < DC; ++c) {
                ad_mma(s[j], qf_lo[c].x, qf_hi[c].x, qf_lo[c].y, qf_hi[c].y, kf[j][c].x, kf[j][c].y);
                ad_mma(s[j], qf_lo[c].z, qf_hi[c].z, qf_lo[c].w, qf_hi[c].w, kf[j][c].z, kf[j][c].w);
            }
        }
        // V pieces: dims 8i+g, keys base+8t..+7 (issued before the softmax arithmetic)
        uint4 vf[DT];
#pragma unroll
        for (int i = 0; i < DT; ++i)
            vf[i] = __ldg(reinterpret_cast<const uint4*>(vp + (size_t)(8 * i + g) * DL_PAGE + 8 * t));

        // ---- mask, online softmax (lane holds keys base + 8t + 2j + {0,1} of rows g and g+8)
        float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int key = base + 8 * t + 2 * j + e;
                const bool ok = key >= first && key < len;
                s[j][e] = ok ? s[j][e] * scale : -INFINITY;
                s[j][2 + e] = ok ? s[j][2 + e] * scale : -INFINITY;
                mx_lo = fmaxf(mx_lo, s[j][e]);
                mx_hi = fmaxf(mx_hi, s[j][2 + e]);
            }
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
        const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
        // a run's first tile may be wholly masked by the window: keep the state untouched then
        const float c_lo = (mn_lo == -INFINITY) ? 1.f : expf(m_lo - mn_lo);
        const float c_hi = (mn_hi == -INFINITY) ? 1.f : expf(m_hi - mn_hi);
        float ps_lo = 0.f, ps_hi = 0.f;
        uint32_t pa[4][2];                               // [tile][row half] packed bf16 pairs
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float p0 = (s[j][0] == -INFINITY) ? 0.f : expf(s[j][0] - mn_lo);
            const float p1 = (s[j][1] == -INFINITY) ? 0.f : expf(s[j][1] - mn_lo);
            const float p2 = (s[j][2] == -INFINITY) ? 0.f : expf(s[j][2] - mn_hi);
            const float p3 = (s[j][3] == -INFINITY) ? 0.f : expf(s[j][3] - mn_hi);
            ps_lo += p0 + p1;
            ps_hi += p2 + p3;
            pa[j][0] = ad_pack(p0, p1);
            pa[j][1] = ad_pack(p2, p3);
        }
        l_lo = l_lo * c_lo + ps_lo;
        l_hi = l_hi * c_hi + ps_hi;
        m_lo = mn_lo;
        m_hi = mn_hi;

        // ---- O = O * corr + P V
        const bool ragged = (base + 32 > len) || (base < first);
#pragma unroll
        for (int i = 0; i < DT; ++i) {
            o[i][0] *= c_lo;
            o[i][1] *= c_lo;
            o[i][2] *= c_hi;
            o[i][3] *= c_hi;
            uint4 v = vf[i];
            if (ragged) {
                // keys outside [first, len) may hold anything (even NaN): make them exact zeros
                v = ad_mask_keys(v, base + 8 * t, len);
                if (base + 8 * t < first) {
                    uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int k0 = base + 8 * t + 2 * u;
                        if (k0 + 1 < first) w[u] = 0u;
                        else if (k0 < first) w[u] &= 0xffff0000u;
                    }
                }
            }
            ad_mma(o[i], pa[0][0], pa[0][1], pa[1][0], pa[1][1], v.x, v.y);
            ad_mma(o[i], pa[2][0], pa[2][1], pa[3][0], pa[3][1], v.z, v.w);
        }
    }

    // ---- merge the block's warps (fixed order)
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
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
    __syncthreads();

    // thread -> (row r of the group, dims d, d+128, ...): 128 threads cover group x HD
    const size_t part_row = ((size_t)(b * nkv + kvh) * gridDim.x + split) * group;
    for (int idx = threadIdx.x; idx < group * HD; idx += 32 * AD_WARPS) {
        const int r = idx / HD, d = idx - r * HD;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < AD_WARPS; ++w) m = fmaxf(m, sm_m[w][r]);
        float acc = 0.f, l = 0.f;
#pragma unroll
        for (int w = 0; w < AD_WARPS; ++w) {
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
    for (int idx = threadIdx.x; idx < group * HD; idx += 32 * AD_WARPS) {
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

// q: bf16 [B, nh*hd] rows q_stride apart (one token per sequence); out likewise.
// seq_len[b]: keys of sequence b including the new token.  max_splits = grid size over runs,
// at least ceil(longest visible span / keys_per_split).
// part_o: float32 [B, nkv, max_splits, group, hd]; part_ml: float32 [B, nkv, max_splits, group, 2];
// counters: int32 zeros [B * nkv] (left zero).
extern "C" int dl_attention_decode_bf16(const void* q, int q_stride, void* out, int out_stride, const void* k_pool,
                                        const void* v_pool, int n_pages, const int32_t* seq_len,
                                        const int32_t* block_table, int bt_stride, int n_seqs, int nh, int nkv,
                                        int hd, float scale, int window, int keys_per_split, int max_splits,
                                        float* part_o, float* part_ml, int* counters, void* stream) {
    DL_REQUIRE(n_seqs >= 0 && nh > 0 && nkv > 0 && nh % nkv == 0, "attention_decode: bad head counts");
    DL_REQUIRE(nh / nkv <= 16, "attention_decode: groups of more than 16 query heads are not supported (%d)", nh / nkv);
    DL_REQUIRE(keys_per_split >= DL_PAGE && keys_per_split % DL_PAGE == 0, "attention_decode: keys_per_split %d must be a multiple of %d", keys_per_split, DL_PAGE);
    DL_REQUIRE(max_splits >= 1 && (max_splits == 1 || (part_o && part_ml && counters)), "attention_decode: split runs need scratch");
    DL_REQUIRE(q_stride % 8 == 0 && ((uintptr_t)q % 16) == 0 && ((uintptr_t)k_pool % 16) == 0 && ((uintptr_t)v_pool % 16) == 0,
               "attention_decode: q and the pools must be 16-byte aligned");
    DL_REQUIRE(n_seqs <= 65535 && nkv <= 65535, "attention_decode: grid too large");
    if (n_seqs == 0) return DL_OK;
    dim3 grid(max_splits, nkv, n_seqs);
    cudaStream_t s = (cudaStream_t)stream;
#define AD_CASE(HDV)                                                                                             \
    if (hd == HDV) {                                                                                             \
        attention_decode_kernel<HDV><<<grid, 32 * AD_WARPS, 0, s>>>(                                             \
            (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)k_pool,     \
            (const __nv_bfloat16*)v_pool, n_pages, seq_len, block_table, bt_stride, nh, nkv, scale, window,      \
            keys_per_split, part_o, part_ml, counters);                                                          \
        DL_CHECK_LAUNCH("attention_decode");                                                                     \
        return DL_OK;                                                                                            \
    }
    AD_CASE(32) AD_CASE(64) AD_CASE(96) AD_CASE(128)
#undef AD_CASE
    return dl_fail(DL_ERR_UNSUPPORTED, "attention_decode: head_dim %d (takes 32, 64, 96, 128)", hd);
}
