// Rotary position encoding of Q and K fused with the write of K and V into the paged cache.
//
// Rotation is the half-split pairing (x[i], x[i + d/2]) -> (x0*cos - x1*sin, x0*sin + x1*cos)
// of the reference's rope_f32 with rope_type == 1 (native/kernels/rope_f32.cu:6-57) and of
// its CPU twin (src/DotLLM.Cpu/Kernels/RoPE.cs:250-256); the reference then copies the K and
// V rows into the cache (src/DotLLM.Cuda/CudaKvCache.cs:64-97).  Here the angles come from a
// float32 cos/sin table built once on the host in float64, the arithmetic is float32, Q is
// rotated in place and rotated K goes straight to its cache page.  V pages are transposed.
#include "common.cuh"

// The rotation, written with explicit roundings so that both kernels below (and any compiler
// version) produce the same bits: no contraction into fused multiply-adds.
__device__ __forceinline__ float rope_lo(float x0, float x1, float c, float s) { return __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s)); }
__device__ __forceinline__ float rope_hi(float x0, float x1, float c, float s) { return __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c)); }

// Grid: (token, head) with the query heads first, then the KV heads; a block's threads each take
// one rotation pair (query heads) or one dimension (KV heads), so a decode step's handful of
// tokens still spreads over hundreds of blocks and no thread loops over dependent loads.
template <typename T>
__global__ void __launch_bounds__(128)
rope_cache_write_kernel(T* __restrict__ q, int q_stride, const T* __restrict__ k, int k_stride,
                        const T* __restrict__ v, int v_stride, const float* __restrict__ cos_t,
                        const float* __restrict__ sin_t, int rotary_dim, int table_rows,
                        const int32_t* __restrict__ token_seq, const int32_t* __restrict__ token_pos,
                        const int32_t* __restrict__ block_table, int bt_stride, T* __restrict__ k_pool,
                        T* __restrict__ v_pool, int n_pages, int nh, int nkv, int hd, int write_cache) {
    dl_launch_dependents();
    dl_grid_dependency_wait();
    const int t = blockIdx.x;
    const int pos = token_pos[t];
    const int half = rotary_dim / 2;
    if (pos < 0 || (half > 0 && pos >= table_rows)) return;      // host-validated; never index outside
    const float* cs = cos_t + (size_t)pos * half;
    const float* sn = sin_t + (size_t)pos * half;

    if ((int)blockIdx.y < nh) {                                   // a query head: rotate in place
        T* p = q + (size_t)t * q_stride + (size_t)blockIdx.y * hd;
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const float x0 = dl_to_f32<T>(p[i]), x1 = dl_to_f32<T>(p[i + half]);
            const float c = cs[i], s = sn[i];
            p[i] = dl_from_f32<T>(rope_lo(x0, x1, c, s));
            p[i + half] = dl_from_f32<T>(rope_hi(x0, x1, c, s));
        }
        return;
    }
    if (!write_cache) return;
    const int h = blockIdx.y - nh;                                // a KV head: rotate K on its way to the page
    const int seq = token_seq[t];
    const int page = block_table[(size_t)seq * bt_stride + pos / DL_PAGE];
    if (page < 0 || page >= n_pages) return;
    const int in_page = pos % DL_PAGE;
    const T* krow = k + (size_t)t * k_stride + (size_t)h * hd;
    const T* vrow = v + (size_t)t * v_stride + (size_t)h * hd;
    T* kdst = k_pool + dl_k_offset(page, nkv, h, in_page, hd);
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float kv;
        if (d < half) {
            kv = rope_lo(dl_to_f32<T>(krow[d]), dl_to_f32<T>(krow[d + half]), cs[d], sn[d]);
        } else if (d < 2 * half) {
            const int i = d - half;
            kv = rope_hi(dl_to_f32<T>(krow[i]), dl_to_f32<T>(krow[d]), cs[i], sn[i]);
        } else {
            kv = dl_to_f32<T>(krow[d]);
        }
        kdst[d] = dl_from_f32<T>(kv);
        v_pool[dl_v_offset(page, nkv, h, d, hd) + in_page] = vrow[d];
    }
}

// The same work for steps of many tokens (prefill).  Grid: (tile of 64 packed tokens, head).  A
// block of a KV head stages the tile's V rows in shared memory and writes them transposed, token
// fastest, so that the tokens of one page (consecutive positions of one sequence) fill whole
// 128-byte lines of the transposed V page instead of one 2-byte element each.
#define RT_TOKENS 64
#ifndef RT_THREADS
#define RT_THREADS 256
#endif
template <typename T>
__global__ void __launch_bounds__(RT_THREADS)
rope_cache_write_tile_kernel(T* __restrict__ q, int q_stride, const T* __restrict__ k, int k_stride,
                             const T* __restrict__ v, int v_stride, const float* __restrict__ cos_t,
                             const float* __restrict__ sin_t, int rotary_dim, int table_rows,
                             const int32_t* __restrict__ token_seq, const int32_t* __restrict__ token_pos,
                             const int32_t* __restrict__ block_table, int bt_stride, T* __restrict__ k_pool,
                             T* __restrict__ v_pool, int n_pages, int n_tokens, int nh, int nkv, int hd, int write_cache) {
    extern __shared__ __align__(16) unsigned char rt_raw[];
    T* tile = reinterpret_cast<T*>(rt_raw);                  // [64 tokens][hd + pad]: V rows of one KV head
    __shared__ int s_pos[RT_TOKENS], s_page[RT_TOKENS];
    dl_launch_dependents();
    dl_grid_dependency_wait();
    const int t0 = blockIdx.x * RT_TOKENS;
    const int nt = min(RT_TOKENS, n_tokens - t0);
    const int half = rotary_dim / 2;
    // KV heads first: their blocks do more (K to its page, V through the transposing tile) and should not start last
    const int kv_first = write_cache ? nkv : 0;
    const bool is_q = (int)blockIdx.y >= kv_first;
    const int pitch = hd + (int)(4 / sizeof(T));             // an odd number of 32-bit words: no bank conflicts on the transpose
    if (threadIdx.x < RT_TOKENS) {
        int pos = -1, page = -1;
        if ((int)threadIdx.x < nt) {
            pos = token_pos[t0 + threadIdx.x];
            if (pos < 0 || (half > 0 && pos >= table_rows)) pos = -1;    // host-validated; never index outside
            if (pos >= 0 && !is_q && write_cache) {
                page = block_table[(size_t)token_seq[t0 + threadIdx.x] * bt_stride + pos / DL_PAGE];
                if (page < 0 || page >= n_pages) page = -1;
            }
        }
        s_pos[threadIdx.x] = pos;
        s_page[threadIdx.x] = page;
    }
    __syncthreads();
    if (is_q) {                                              // a query head: rotate in place
        for (int idx = threadIdx.x; idx < nt * half; idx += RT_THREADS) {
            const int i = idx / half, p = idx - i * half;
            const int pos = s_pos[i];
            if (pos < 0) continue;
            T* row = q + (size_t)(t0 + i) * q_stride + (size_t)((int)blockIdx.y - kv_first) * hd;
            const float x0 = dl_to_f32<T>(row[p]), x1 = dl_to_f32<T>(row[p + half]);
            const float c = cos_t[(size_t)pos * half + p], s = sin_t[(size_t)pos * half + p];
            row[p] = dl_from_f32<T>(rope_lo(x0, x1, c, s));
            row[p + half] = dl_from_f32<T>(rope_hi(x0, x1, c, s));
        }
        return;
    }
    if (!write_cache) return;
    const int h = blockIdx.y;                                // a KV head: rotate K on its way to the page, stage V
    for (int idx = threadIdx.x; idx < nt * hd; idx += RT_THREADS) {
        const int i = idx / hd, d = idx - i * hd;
        const int page = s_page[i], pos = s_pos[i];
        tile[i * pitch + d] = v[(size_t)(t0 + i) * v_stride + (size_t)h * hd + d];
        if (page < 0) continue;
        const T* krow = k + (size_t)(t0 + i) * k_stride + (size_t)h * hd;
        const float* cs = cos_t + (size_t)pos * half;
        const float* sn = sin_t + (size_t)pos * half;
        float kv;
        if (d < half) {
            kv = rope_lo(dl_to_f32<T>(krow[d]), dl_to_f32<T>(krow[d + half]), cs[d], sn[d]);
        } else if (d < 2 * half) {
            const int j = d - half;
            kv = rope_hi(dl_to_f32<T>(krow[j]), dl_to_f32<T>(krow[d]), cs[j], sn[j]);
        } else {
            kv = dl_to_f32<T>(krow[d]);
        }
        k_pool[dl_k_offset(page, nkv, h, pos % DL_PAGE, hd) + d] = dl_from_f32<T>(kv);
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < RT_TOKENS * hd; idx += RT_THREADS) {    // token fastest
        const int i = idx % RT_TOKENS, d = idx / RT_TOKENS;
        if (i >= nt) continue;
        const int page = s_page[i];
        if (page < 0) continue;
        v_pool[dl_v_offset(page, nkv, h, d, hd) + (s_pos[i] % DL_PAGE)] = tile[i * pitch + d];
    }
}

// The tile kernel for bfloat16 with a full-width rotation (rotary_dim == hd, hd a multiple of 16,
// 16-byte aligned rows): a thread moves 16 bytes at a time - eight rotation pairs for Q and K, eight
// values of V - instead of one element.
__device__ __forceinline__ void rope_rotate8(uint4& x0, uint4& x1, const float* cs, const float* sn) {
    const float4 c0 = *reinterpret_cast<const float4*>(cs), c1 = *reinterpret_cast<const float4*>(cs + 4);
    const float4 s0 = *reinterpret_cast<const float4*>(sn), s1 = *reinterpret_cast<const float4*>(sn + 4);
    const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float s[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    __nv_bfloat16* a = reinterpret_cast<__nv_bfloat16*>(&x0);
    __nv_bfloat16* b = reinterpret_cast<__nv_bfloat16*>(&x1);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const float f0 = __bfloat162float(a[e]), f1 = __bfloat162float(b[e]);
        a[e] = __float2bfloat16_rn(rope_lo(f0, f1, c[e], s[e]));
        b[e] = __float2bfloat16_rn(rope_hi(f0, f1, c[e], s[e]));
    }
}

__global__ void __launch_bounds__(RT_THREADS)
rope_cache_write_tile_vec_kernel(__nv_bfloat16* __restrict__ q, int q_stride, const __nv_bfloat16* __restrict__ k, int k_stride,
                                 const __nv_bfloat16* __restrict__ v, int v_stride, const float* __restrict__ cos_t,
                                 const float* __restrict__ sin_t, int table_rows, const int32_t* __restrict__ token_seq,
                                 const int32_t* __restrict__ token_pos, const int32_t* __restrict__ block_table, int bt_stride,
                                 __nv_bfloat16* __restrict__ k_pool, __nv_bfloat16* __restrict__ v_pool, int n_pages,
                                 int n_tokens, int nh, int nkv, int hd, int write_cache) {
    extern __shared__ __align__(16) unsigned char rt_raw[];
    __nv_bfloat16* tile = reinterpret_cast<__nv_bfloat16*>(rt_raw);      // [64 tokens][hd + 2]: V rows of one KV head
    __shared__ int s_pos[RT_TOKENS], s_page[RT_TOKENS];
    dl_launch_dependents();
    dl_grid_dependency_wait();
    const int t0 = blockIdx.x * RT_TOKENS;
    const int nt = min(RT_TOKENS, n_tokens - t0);
    const int half = hd / 2, groups = half / 8;              // groups of eight rotation pairs per head
    // KV heads first: their blocks do more (K to its page, V through the transposing tile) and should not start last
    const int kv_first = write_cache ? nkv : 0;
    const bool is_q = (int)blockIdx.y >= kv_first;
    const int pitch = hd + 2;
    if (threadIdx.x < RT_TOKENS) {
        int pos = -1, page = -1;
        if ((int)threadIdx.x < nt) {
            pos = token_pos[t0 + threadIdx.x];
            if (pos < 0 || pos >= table_rows) pos = -1;      // host-validated; never index outside
            if (pos >= 0 && !is_q && write_cache) {
                page = block_table[(size_t)token_seq[t0 + threadIdx.x] * bt_stride + pos / DL_PAGE];
                if (page < 0 || page >= n_pages) page = -1;
            }
        }
        s_pos[threadIdx.x] = pos;
        s_page[threadIdx.x] = page;
    }
    __syncthreads();
    if (is_q) {                                              // a query head: rotate in place
        for (int idx = threadIdx.x; idx < nt * groups; idx += RT_THREADS) {
            const int i = idx / groups, u = (idx - i * groups) * 8;
            const int pos = s_pos[i];
            if (pos < 0) continue;
            __nv_bfloat16* row = q + (size_t)(t0 + i) * q_stride + (size_t)((int)blockIdx.y - kv_first) * hd;
            uint4 x0 = *reinterpret_cast<const uint4*>(row + u), x1 = *reinterpret_cast<const uint4*>(row + half + u);
            rope_rotate8(x0, x1, cos_t + (size_t)pos * half + u, sin_t + (size_t)pos * half + u);
            *reinterpret_cast<uint4*>(row + u) = x0;
            *reinterpret_cast<uint4*>(row + half + u) = x1;
        }
        return;
    }
    if (!write_cache) return;
    const int h = blockIdx.y;                                // a KV head: rotate K on its way to the page, stage V
    for (int idx = threadIdx.x; idx < nt * groups; idx += RT_THREADS) {
        const int i = idx / groups, u = (idx - i * groups) * 8;
        const int page = s_page[i], pos = s_pos[i];
        const __nv_bfloat16* vrow = v + (size_t)(t0 + i) * v_stride + (size_t)h * hd;
        const uint4 v0 = *reinterpret_cast<const uint4*>(vrow + u), v1 = *reinterpret_cast<const uint4*>(vrow + half + u);
        uint32_t* t_lo = reinterpret_cast<uint32_t*>(tile + i * pitch + u);          // 4-byte aligned: pitch and u are even
        uint32_t* t_hi = reinterpret_cast<uint32_t*>(tile + i * pitch + half + u);
        t_lo[0] = v0.x; t_lo[1] = v0.y; t_lo[2] = v0.z; t_lo[3] = v0.w;
        t_hi[0] = v1.x; t_hi[1] = v1.y; t_hi[2] = v1.z; t_hi[3] = v1.w;
        if (page < 0) continue;
        const __nv_bfloat16* krow = k + (size_t)(t0 + i) * k_stride + (size_t)h * hd;
        uint4 x0 = *reinterpret_cast<const uint4*>(krow + u), x1 = *reinterpret_cast<const uint4*>(krow + half + u);
        rope_rotate8(x0, x1, cos_t + (size_t)pos * half + u, sin_t + (size_t)pos * half + u);
        __nv_bfloat16* kdst = k_pool + dl_k_offset(page, nkv, h, pos % DL_PAGE, hd);
        *reinterpret_cast<uint4*>(kdst + u) = x0;
        *reinterpret_cast<uint4*>(kdst + half + u) = x1;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < RT_TOKENS * hd; idx += RT_THREADS) {    // token fastest
        const int i = idx % RT_TOKENS, d = idx / RT_TOKENS;
        if (i >= nt) continue;
        const int page = s_page[i];
        if (page < 0) continue;
        v_pool[dl_v_offset(page, nkv, h, d, hd) + (s_pos[i] % DL_PAGE)] = tile[i * pitch + d];
    }
}

extern "C" int dl_rope_cache_write(void* q, int q_stride, const void* k, int k_stride, const void* v, int v_stride,
                                   int dtype, const float* cos_t, const float* sin_t, int rotary_dim,
                                   int table_rows, const int32_t* token_seq, const int32_t* token_pos,
                                   const int32_t* block_table, int bt_stride, void* k_pool, void* v_pool,
                                   int n_pages, int n_tokens, int nh, int nkv, int hd, int write_cache,
                                   void* stream) {
    DL_REQUIRE(n_tokens >= 0 && nh > 0 && nkv > 0 && hd > 0, "rope_cache_write: bad sizes");
    DL_REQUIRE(rotary_dim >= 0 && rotary_dim <= hd && rotary_dim % 2 == 0,
               "rope_cache_write: rotary_dim %d must be even and at most head_dim %d", rotary_dim, hd);
    DL_REQUIRE(rotary_dim == 0 || (cos_t && sin_t && table_rows > 0), "rope_cache_write: rotation needs tables");
    DL_REQUIRE(q_stride >= nh * hd && (!write_cache || (k_stride >= nkv * hd && v_stride >= nkv * hd)),
               "rope_cache_write: row strides shorter than the rows");
    DL_REQUIRE(!write_cache || (k && v && k_pool && v_pool && block_table && n_pages > 0),
               "rope_cache_write: cache write needs k, v, pools and a block table");
    if (n_tokens == 0) return DL_OK;
    cudaStream_t s = (cudaStream_t)stream;
    DL_REQUIRE(nh + nkv <= 65535, "rope_cache_write: too many heads");
    cudaError_t e;
    const size_t elem = dtype == DL_F32 ? 4 : 2;
    const size_t tile_smem = (size_t)RT_TOKENS * (hd + 4 / elem) * elem;
    if (n_tokens >= RT_TOKENS && tile_smem <= 48 * 1024 && (dtype == DL_F32 || dtype == DL_BF16)) {
        dim3 tgrid((n_tokens + RT_TOKENS - 1) / RT_TOKENS, write_cache ? nh + nkv : nh);
        const bool aligned = ((uintptr_t)q % 16) == 0 && q_stride % 8 == 0 && ((uintptr_t)cos_t % 16) == 0 &&
                             ((uintptr_t)sin_t % 16) == 0 &&
                             (!write_cache || (((uintptr_t)k % 16) == 0 && ((uintptr_t)v % 16) == 0 && k_stride % 8 == 0 &&
                                               v_stride % 8 == 0 && ((uintptr_t)k_pool % 16) == 0));
        if (dtype == DL_BF16 && rotary_dim == hd && hd % 16 == 0 && aligned) {
            e = dl_launch_dependent(rope_cache_write_tile_vec_kernel, tgrid, dim3(RT_THREADS), tile_smem, s, (__nv_bfloat16*)q,
                                    q_stride, (const __nv_bfloat16*)k, k_stride, (const __nv_bfloat16*)v, v_stride, cos_t, sin_t,
                                    table_rows, token_seq, token_pos, block_table, bt_stride, (__nv_bfloat16*)k_pool,
                                    (__nv_bfloat16*)v_pool, n_pages, n_tokens, nh, nkv, hd, write_cache);
            if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "rope_cache_write: %s", cudaGetErrorString(e));
            return DL_OK;
        }
        if (dtype == DL_F32)
            e = dl_launch_dependent(rope_cache_write_tile_kernel<float>, tgrid, dim3(RT_THREADS), tile_smem, s, (float*)q, q_stride,
                                    (const float*)k, k_stride, (const float*)v, v_stride, cos_t, sin_t, rotary_dim, table_rows,
                                    token_seq, token_pos, block_table, bt_stride, (float*)k_pool, (float*)v_pool, n_pages,
                                    n_tokens, nh, nkv, hd, write_cache);
        else
            e = dl_launch_dependent(rope_cache_write_tile_kernel<__nv_bfloat16>, tgrid, dim3(RT_THREADS), tile_smem, s,
                                    (__nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k, k_stride, (const __nv_bfloat16*)v,
                                    v_stride, cos_t, sin_t, rotary_dim, table_rows, token_seq, token_pos, block_table,
                                    bt_stride, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, n_pages, n_tokens, nh, nkv, hd,
                                    write_cache);
        if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "rope_cache_write: %s", cudaGetErrorString(e));
        return DL_OK;
    }
    dim3 grid(n_tokens, write_cache ? nh + nkv : nh);
    if (dtype == DL_F32)
        e = dl_launch_dependent(rope_cache_write_kernel<float>, grid, dim3(128), 0, s, (float*)q, q_stride, (const float*)k,
                                k_stride, (const float*)v, v_stride, cos_t, sin_t, rotary_dim, table_rows, token_seq,
                                token_pos, block_table, bt_stride, (float*)k_pool, (float*)v_pool, n_pages, nh, nkv, hd,
                                write_cache);
    else if (dtype == DL_BF16)
        e = dl_launch_dependent(rope_cache_write_kernel<__nv_bfloat16>, grid, dim3(128), 0, s, (__nv_bfloat16*)q, q_stride,
                                (const __nv_bfloat16*)k, k_stride, (const __nv_bfloat16*)v, v_stride, cos_t, sin_t,
                                rotary_dim, table_rows, token_seq, token_pos, block_table, bt_stride,
                                (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, n_pages, nh, nkv, hd, write_cache);
    else
        return dl_fail(DL_ERR_UNSUPPORTED, "rope_cache_write: dtype %d", dtype);
    if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "rope_cache_write: %s", cudaGetErrorString(e));
    return DL_OK;
}
