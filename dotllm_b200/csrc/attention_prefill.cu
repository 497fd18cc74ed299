// Prefill attention: many new tokens per sequence (whole prompts or chunks) over the paged
// bfloat16 cache, causal, optionally windowed, packed sequences of unequal lengths.
//
// Role of the reference's attention_f16 with seq_q > 1 (native/kernels/attention.cu:19-197), which
// gives one block to every (query token, head) and walks the keys with scalar dot products.  Here a
// warp owns 16 consecutive query positions of one head as the rows of mma.sync.m16n8k16 tiles and
// walks the keys 32 at a time with an online softmax in float32 registers (exact expf); a block is
// four such warps on 64 consecutive positions, so that neighbouring warps find the keys and values
// they share in L1.  Operands are loaded as 16-byte pieces straight into registers with the same
// k-permutation as the decode kernel (csrc/attention_decode.cu): K rows by dims, transposed V rows
// by keys.  The new tokens' own keys and values are already in the cache when this runs, so one
// loop covers earlier context and the causal triangle.
#include "common.cuh"

#define AP_WARPS 4
#define AP_ROWS (16 * AP_WARPS)

__device__ __forceinline__ void ap_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t ap_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Zero the bf16 elements of a 16-byte piece (keys first..first+7) outside [lo, hi].
__device__ __forceinline__ uint4 ap_keep_keys(uint4 v, int first, int lo, int hi) {
    uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int k0 = first + 2 * i;
        const bool a = k0 >= lo && k0 <= hi, b = k0 + 1 >= lo && k0 + 1 <= hi;
        if (!a && !b) w[i] = 0u;
        else if (!a) w[i] &= 0xffff0000u;
        else if (!b) w[i] &= 0x0000ffffu;
    }
    return v;
}

template <int HD>
__global__ void __launch_bounds__(32 * AP_WARPS)
attention_prefill_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, __nv_bfloat16* __restrict__ out,
                         int out_stride, const __nv_bfloat16* __restrict__ k_pool,
                         const __nv_bfloat16* __restrict__ v_pool, int n_pages,
                         const int32_t* __restrict__ tile_seq, const int32_t* __restrict__ tile_row0,
                         const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_new,
                         const int32_t* __restrict__ cu_new, const int32_t* __restrict__ block_table,
                         int bt_stride, int nh, int nkv, float scale, int window) {
    constexpr int DC = HD / 32;
    constexpr int DT = HD / 8;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int tile = blockIdx.x, h = blockIdx.y;
    const int b = tile_seq[tile];
    const int row0 = tile_row0[tile] + 16 * warp;        // first of this warp's rows among the sequence's new tokens
    const int n_new = seq_new[b];
    if (row0 >= n_new) return;                           // warps are independent (no block barrier)
    const int start = seq_start[b];
    const int tok0 = cu_new[b] + row0;                   // packed token index of the warp's first row
    const int kvh = h / (nh / nkv);
    const int32_t* pages = block_table + (size_t)b * bt_stride;

    const bool ok_lo = row0 + g < n_new, ok_hi = row0 + g + 8 < n_new;
    const int pos_lo = ok_lo ? start + row0 + g : -1;    // invalid rows see no key
    const int pos_hi = ok_hi ? start + row0 + g + 8 : -1;
    const int last_row = min(row0 + 15, n_new - 1);
    const int pos_max = start + last_row;                // furthest key any row of the warp sees
    const int pos_min = start + row0;
    const int key_first = (window > 0 && pos_min - window + 1 > 0) ? pos_min - window + 1 : 0;
    const int first_lo = (window > 0) ? pos_lo - window + 1 : 0;
    const int first_hi = (window > 0) ? pos_hi - window + 1 : 0;

    uint4 qf_lo[DC], qf_hi[DC];
#pragma unroll
    for (int c = 0; c < DC; ++c) {
        qf_lo[c] = make_uint4(0u, 0u, 0u, 0u);
        qf_hi[c] = make_uint4(0u, 0u, 0u, 0u);
        if (ok_lo) qf_lo[c] = *reinterpret_cast<const uint4*>(q + (size_t)(tok0 + g) * q_stride + (size_t)h * HD + c * 32 + t * 8);
        if (ok_hi) qf_hi[c] = *reinterpret_cast<const uint4*>(q + (size_t)(tok0 + g + 8) * q_stride + (size_t)h * HD + c * 32 + t * 8);
    }

    float o[DT][4];
#pragma unroll
    for (int i = 0; i < DT; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;

    for (int base = (key_first / 32) * 32; base <= pos_max; base += 32) {
        const int page = pages[base / DL_PAGE];
        if (page < 0 || page >= n_pages) continue;       // host-validated; never read outside the pool
        const int in_page = base % DL_PAGE;
        const __nv_bfloat16* kp = k_pool + dl_k_offset(page, nkv, kvh, in_page, HD);
        const __nv_bfloat16* vp = v_pool + dl_v_offset(page, nkv, kvh, 0, HD) + in_page;

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
                ap_mma(s[j], qf_lo[c].x, qf_hi[c].x, qf_lo[c].y, qf_hi[c].y, kf[j][c].x, kf[j][c].y);
                ap_mma(s[j], qf_lo[c].z, qf_hi[c].z, qf_lo[c].w, qf_hi[c].w, kf[j][c].z, kf[j][c].w);
            }
        }
        uint4 vf[DT];
#pragma unroll
        for (int i = 0; i < DT; ++i)
            vf[i] = __ldg(reinterpret_cast<const uint4*>(vp + (size_t)(8 * i + g) * DL_PAGE + 8 * t));

        float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int key = base + 8 * t + 2 * j + e;
                s[j][e] = (key <= pos_lo && key >= first_lo) ? s[j][e] * scale : -INFINITY;
                s[j][2 + e] = (key <= pos_hi && key >= first_hi) ? s[j][2 + e] * scale : -INFINITY;
                mx_lo = fmaxf(mx_lo, s[j][e]);
                mx_hi = fmaxf(mx_hi, s[j][2 + e]);
            }
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
        const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
        const float c_lo = (mn_lo == -INFINITY) ? 1.f : expf(m_lo - mn_lo);
        const float c_hi = (mn_hi == -INFINITY) ? 1.f : expf(m_hi - mn_hi);
        float ps_lo = 0.f, ps_hi = 0.f;
        uint32_t pa[4][2];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float p0 = (s[j][0] == -INFINITY) ? 0.f : expf(s[j][0] - mn_lo);
            const float p1 = (s[j][1] == -INFINITY) ? 0.f : expf(s[j][1] - mn_lo);
            const float p2 = (s[j][2] == -INFINITY) ? 0.f : expf(s[j][2] - mn_hi);
            const float p3 = (s[j][3] == -INFINITY) ? 0.f : expf(s[j][3] - mn_hi);
            ps_lo += p0 + p1;
            ps_hi += p2 + p3;
            pa[j][0] = ap_pack(p0, p1);
            pa[j][1] = ap_pack(p2, p3);
        }
        l_lo = l_lo * c_lo + ps_lo;
        l_hi = l_hi * c_hi + ps_hi;
        m_lo = mn_lo;
        m_hi = mn_hi;

        // keys no row of the warp may see can hold anything (a reused page): exact zeros instead
        const bool ragged = (base + 31 > pos_max) || (base < key_first);
#pragma unroll
        for (int i = 0; i < DT; ++i) {
            o[i][0] *= c_lo;
            o[i][1] *= c_lo;
            o[i][2] *= c_hi;
            o[i][3] *= c_hi;
            uint4 v = vf[i];
            if (ragged) v = ap_keep_keys(v, base + 8 * t, key_first, pos_max);
            ap_mma(o[i], pa[0][0], pa[0][1], pa[1][0], pa[1][1], v.x, v.y);
            ap_mma(o[i], pa[2][0], pa[2][1], pa[3][0], pa[3][1], v.z, v.w);
        }
    }

    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    const float inv_lo = 1.0f / l_lo, inv_hi = 1.0f / l_hi;
    __nv_bfloat16* o_lo = out + (size_t)(tok0 + g) * out_stride + (size_t)h * HD;
    __nv_bfloat16* o_hi = out + (size_t)(tok0 + g + 8) * out_stride + (size_t)h * HD;
#pragma unroll
    for (int i = 0; i < DT; ++i) {
        if (ok_lo) *reinterpret_cast<__nv_bfloat162*>(o_lo + 8 * i + 2 * t) = __floats2bfloat162_rn(o[i][0] * inv_lo, o[i][1] * inv_lo);
        if (ok_hi) *reinterpret_cast<__nv_bfloat162*>(o_hi + 8 * i + 2 * t) = __floats2bfloat162_rn(o[i][2] * inv_hi, o[i][3] * inv_hi);
    }
}

// q, out: bf16 [T, nh*hd] packed new tokens of all sequences.  tile_seq / tile_row0: for every
// 64-row tile its sequence and its first row among that sequence's new tokens.  seq_start,
// seq_new: cached length before the step and new tokens, per sequence; cu_new: packed offsets.
extern "C" int dl_attention_prefill_bf16(const void* q, int q_stride, void* out, int out_stride,
                                         const void* k_pool, const void* v_pool, int n_pages,
                                         const int32_t* tile_seq, const int32_t* tile_row0, int n_tiles,
                                         const int32_t* seq_start, const int32_t* seq_new, const int32_t* cu_new,
                                         const int32_t* block_table, int bt_stride, int nh, int nkv, int hd,
                                         float scale, int window, void* stream) {
    DL_REQUIRE(n_tiles >= 0 && nh > 0 && nkv > 0 && nh % nkv == 0, "attention_prefill: bad sizes");
    DL_REQUIRE(q_stride % 8 == 0 && out_stride % 2 == 0 && ((uintptr_t)q % 16) == 0 && ((uintptr_t)out % 4) == 0 &&
                   ((uintptr_t)k_pool % 16) == 0 && ((uintptr_t)v_pool % 16) == 0,
               "attention_prefill: q and the pools must be 16-byte aligned");
    DL_REQUIRE(nh <= 65535, "attention_prefill: too many heads");
    if (n_tiles == 0) return DL_OK;
    dim3 grid(n_tiles, nh);
    cudaStream_t s = (cudaStream_t)stream;
#define AP_CASE(HDV)                                                                                            \
    if (hd == HDV) {                                                                                            \
        attention_prefill_kernel<HDV><<<grid, 32 * AP_WARPS, 0, s>>>(                                           \
            (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)k_pool,    \
            (const __nv_bfloat16*)v_pool, n_pages, tile_seq, tile_row0, seq_start, seq_new, cu_new, block_table, \
            bt_stride, nh, nkv, scale, window);                                                                 \
        DL_CHECK_LAUNCH("attention_prefill");                                                                   \
        return DL_OK;                                                                                           \
    }
    AP_CASE(32) AP_CASE(64) AP_CASE(96) AP_CASE(128)
#undef AP_CASE
    return dl_fail(DL_ERR_UNSUPPORTED, "attention_prefill: head_dim %d (takes 32, 64, 96, 128)", hd);
}
