// Rotary position encoding of Q and K fused with the write of K and V into the paged cache.
//
// Rotation is the half-split pairing (x[i], x[i + d/2]) -> (x0*cos - x1*sin, x0*sin + x1*cos)
// of the reference's rope_f32 with rope_type == 1 (native/kernels/rope_f32.cu:6-57) and of
// its CPU twin (src/DotLLM.Cpu/Kernels/RoPE.cs:250-256); the reference then copies the K and
// V rows into the cache (src/DotLLM.Cuda/CudaKvCache.cs:64-97).  Here the angles come from a
// float32 cos/sin table built once on the host in float64, the arithmetic is float32, Q is
// rotated in place and rotated K goes straight to its cache page.  V pages are transposed.
#include "common.cuh"

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
            p[i] = dl_from_f32<T>(x0 * c - x1 * s);
            p[i + half] = dl_from_f32<T>(x0 * s + x1 * c);
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
            kv = dl_to_f32<T>(krow[d]) * cs[d] - dl_to_f32<T>(krow[d + half]) * sn[d];
        } else if (d < 2 * half) {
            const int i = d - half;
            kv = dl_to_f32<T>(krow[i]) * sn[i] + dl_to_f32<T>(krow[d]) * cs[i];
        } else {
            kv = dl_to_f32<T>(krow[d]);
        }
        kdst[d] = dl_from_f32<T>(kv);
        v_pool[dl_v_offset(page, nkv, h, d, hd) + in_page] = vrow[d];
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
    dim3 grid(n_tokens, write_cache ? nh + nkv : nh);
    cudaError_t e;
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
