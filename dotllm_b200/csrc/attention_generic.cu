// Causal (optionally windowed) attention of new tokens over the paged cache, any head size
// and head grouping, float32 or bfloat16 storage, all arithmetic in float32.
//
// Same math as the reference's attention_f32 (native/kernels/attention_f32.cu:8-136) and its
// scalar CPU twin (src/DotLLM.Cpu/Kernels/Attention.cs:446-519): s = (q.k) * scale, keys after
// the query's position masked (and keys older than `window`, when given), softmax with the
// running maximum subtracted, o = sum w v; query head h reads KV head h / (nh / nkv).
//
// One warp per (token, query head).  Keys are walked in tiles of 32 aligned to absolute
// positions, one key per lane for the scores and one output dimension per lane for the
// weighted sum, with exact expf.  The order of operations for a query therefore depends
// only on its position, never on how the tokens were cut into steps or batched: this is
// the kernel of the float32 path and the fallback of the bfloat16 path for sizes that the
// tensor-core kernels do not take.
//
// It is also the one kernel that honours a change of the scores before the softmax, the place where
// the reference's seam for position encodings that bias scores sits
// (src/DotLLM.Core/PositionEncoding/IPositionEncoding.cs:10-34): with `softcap` > 0 a score becomes
// softcap * tanh(score / softcap), and with `slopes` (one float per query head) slope * (key position -
// query position) is added after that (a penalty that grows with distance).
#include "common.cuh"

#define AG_WARPS 4
#define AG_MAX_HD 512

template <typename T>
__global__ void __launch_bounds__(32 * AG_WARPS)
attention_generic_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride,
                         const T* __restrict__ k_pool, const T* __restrict__ v_pool, int n_pages,
                         const int32_t* __restrict__ token_seq, const int32_t* __restrict__ token_pos,
                         const int32_t* __restrict__ block_table, int bt_stride, int nh, int nkv, int hd,
                         float scale, int window, float softcap, const float* __restrict__ slopes) {
    extern __shared__ float q_smem[];                 // [AG_WARPS][hd]
    const int lane = threadIdx.x;
    const int t = blockIdx.x;
    const int h = blockIdx.y * AG_WARPS + threadIdx.y;
    if (h >= nh) return;                              // warps are independent below (no block barrier)
    float* qs = q_smem + threadIdx.y * hd;
    const T* qrow = q + (size_t)t * q_stride + (size_t)h * hd;
    for (int d = lane; d < hd; d += 32) qs[d] = dl_to_f32<T>(qrow[d]);
    __syncwarp();

    const int pos = token_pos[t];
    const int seq = token_seq[t];
    const int kvh = h / (nh / nkv);
    const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const float slope = slopes != nullptr ? slopes[h] : 0.f;
    const int32_t* pages = block_table + (size_t)seq * bt_stride;

    float m = -INFINITY, l = 0.f;
    float acc[AG_MAX_HD / 32];
#pragma unroll
    for (int i = 0; i < AG_MAX_HD / 32; ++i) acc[i] = 0.f;

    for (int j0 = (first / 32) * 32; j0 <= pos; j0 += 32) {
        const int page = pages[j0 / DL_PAGE];
        if (page < 0 || page >= n_pages) continue;    // host-validated; never read outside the pool
        const int in_page0 = j0 % DL_PAGE;
        const int j = j0 + lane;
        const bool valid = (j >= first) && (j <= pos);
        float s = -INFINITY;
        if (valid) {
            const T* kr = k_pool + dl_k_offset(page, nkv, kvh, in_page0 + lane, hd);
            float dot = 0.f;
            for (int d = 0; d < hd; ++d) dot += qs[d] * dl_to_f32<T>(kr[d]);
            s = dot * scale;
            if (softcap > 0.f) s = softcap * tanhf(s / softcap);
            if (slopes != nullptr) s += slope * (float)(j - pos);
        }
        const float m_new = fmaxf(m, dl_warp_max(s));
        const float p = valid ? expf(s - m_new) : 0.f;
        const float corr = expf(m - m_new);           // exp(-inf) = 0 on the first tile
        l = l * corr + dl_warp_sum(p);
        m = m_new;
        const T* vt = v_pool + dl_v_offset(page, nkv, kvh, 0, hd) + in_page0;
#pragma unroll
        for (int i = 0; i < AG_MAX_HD / 32; ++i) {
            const int d = lane + 32 * i;
            if (i * 32 < hd) {
                float a = acc[i] * corr;
                const T* vd = vt + (size_t)(d < hd ? d : 0) * DL_PAGE;
                for (int kk = 0; kk < 32; ++kk) {
                    const float pk = __shfl_sync(0xffffffffu, p, kk);
                    // masked keys are never read: a reused page may hold anything there
                    if (j0 + kk >= first && j0 + kk <= pos && d < hd) a += pk * dl_to_f32<T>(vd[kk]);
                }
                acc[i] = a;
            }
        }
    }
    const float inv = 1.0f / l;
    T* orow = out + (size_t)t * out_stride + (size_t)h * hd;
#pragma unroll
    for (int i = 0; i < AG_MAX_HD / 32; ++i) {
        const int d = lane + 32 * i;
        if (i * 32 < hd && d < hd) orow[d] = dl_from_f32<T>(acc[i] * inv);
    }
}

template <typename T> __device__ __forceinline__ float4 ag_load4(const T* p);
template <> __device__ __forceinline__ float4 ag_load4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ __forceinline__ float4 ag_load4<__nv_bfloat16>(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}

// The same for groups of query heads that share a KV head four by four (the block's four warps are
// four query heads of one token and one KV head): the 32 keys and values of a tile are brought into
// shared memory once for the four warps, by all 128 threads, sixteen consecutive bytes of a row to
// consecutive threads, instead of every lane walking its own row of the cache.  Every lane then does
// exactly the arithmetic of the kernel above in the same order, so the results have the same bits.
template <typename T>
__global__ void __launch_bounds__(32 * AG_WARPS)
attention_generic_shared_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride,
                                const T* __restrict__ k_pool, const T* __restrict__ v_pool, int n_pages,
                                const int32_t* __restrict__ token_seq, const int32_t* __restrict__ token_pos,
                                const int32_t* __restrict__ block_table, int bt_stride, int nh, int nkv, int hd,
                                float scale, int window, float softcap, const float* __restrict__ slopes) {
    extern __shared__ float ag_smem[];                // [AG_WARPS][hd] queries, [32][hd + 1] keys, [hd][33] values
    const int lane = threadIdx.x, tid = threadIdx.y * 32 + threadIdx.x;
    const int t = blockIdx.x;
    const int h = blockIdx.y * AG_WARPS + threadIdx.y;        // < nh: the host launches this kernel only when nh % AG_WARPS == 0
    float* qs = ag_smem + threadIdx.y * hd;
    float* kt = ag_smem + AG_WARPS * hd;
    float* vt = kt + 32 * (hd + 1);
    const T* qrow = q + (size_t)t * q_stride + (size_t)h * hd;
    for (int d = lane; d < hd; d += 32) qs[d] = dl_to_f32<T>(qrow[d]);

    const int pos = token_pos[t];
    const int seq = token_seq[t];
    const int kvh = (blockIdx.y * AG_WARPS) / (nh / nkv);      // the same for the block's four heads
    const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const float slope = slopes != nullptr ? slopes[h] : 0.f;
    const int32_t* pages = block_table + (size_t)seq * bt_stride;

    float m = -INFINITY, l = 0.f;
    float acc[AG_MAX_HD / 32];
#pragma unroll
    for (int i = 0; i < AG_MAX_HD / 32; ++i) acc[i] = 0.f;

    for (int j0 = (first / 32) * 32; j0 <= pos; j0 += 32) {
        const int page = pages[j0 / DL_PAGE];
        if (page < 0 || page >= n_pages) continue;    // host-validated; the same for every thread of the block
        const int in_page0 = j0 % DL_PAGE;
        __syncthreads();                              // the tile before has been used (and the queries are in place)
        // four values at a time, eight pieces of each tile asked for before the first is stored
        const T* kbase = k_pool + dl_k_offset(page, nkv, kvh, in_page0, hd);
        const T* vbase = v_pool + dl_v_offset(page, nkv, kvh, 0, hd) + in_page0;
        const int hd4 = hd / 4, n_vec = 8 * hd;       // pieces of four in a row of K; pieces in a tile (K and V alike)
        for (int v0 = tid; v0 < n_vec; v0 += 32 * AG_WARPS * 4) {
            float4 kx[4], vx[4];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const int idx = v0 + b * 32 * AG_WARPS;
                kx[b] = vx[b] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (idx < n_vec) {
                    const int key = idx / hd4, c = idx - key * hd4;
                    if (j0 + key >= first && j0 + key <= pos) kx[b] = ag_load4<T>(kbase + (size_t)key * hd + 4 * c);   // masked keys are never read
                    const int d = idx >> 3, kq = idx & 7;
                    if (j0 + 4 * kq + 3 >= first && j0 + 4 * kq <= pos) vx[b] = ag_load4<T>(vbase + (size_t)d * DL_PAGE + 4 * kq);
                }
            }
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const int idx = v0 + b * 32 * AG_WARPS;
                if (idx < n_vec) {
                    const int key = idx / hd4, c = idx - key * hd4;
                    float* kd = kt + key * (hd + 1) + 4 * c;
                    kd[0] = kx[b].x, kd[1] = kx[b].y, kd[2] = kx[b].z, kd[3] = kx[b].w;
                    const int d = idx >> 3, kq = idx & 7;
                    float* vd = vt + d * 33 + 4 * kq;
                    vd[0] = vx[b].x, vd[1] = vx[b].y, vd[2] = vx[b].z, vd[3] = vx[b].w;
                }
            }
        }
        __syncthreads();
        const int j = j0 + lane;
        const bool valid = (j >= first) && (j <= pos);
        float s = -INFINITY;
        if (valid) {
            const float* kr = kt + lane * (hd + 1);
            float dot = 0.f;
            for (int d = 0; d < hd; ++d) dot += qs[d] * kr[d];
            s = dot * scale;
            if (softcap > 0.f) s = softcap * tanhf(s / softcap);
            if (slopes != nullptr) s += slope * (float)(j - pos);
        }
        const float m_new = fmaxf(m, dl_warp_max(s));
        const float p = valid ? expf(s - m_new) : 0.f;
        const float corr = expf(m - m_new);           // exp(-inf) = 0 on the first tile
        l = l * corr + dl_warp_sum(p);
        m = m_new;
#pragma unroll
        for (int i = 0; i < AG_MAX_HD / 32; ++i) {
            const int d = lane + 32 * i;
            if (i * 32 < hd) {
                float a = acc[i] * corr;
                const float* vd = vt + (size_t)(d < hd ? d : 0) * 33;
                for (int kk = 0; kk < 32; ++kk) {
                    const float pk = __shfl_sync(0xffffffffu, p, kk);
                    if (j0 + kk >= first && j0 + kk <= pos && d < hd) a += pk * vd[kk];
                }
                acc[i] = a;
            }
        }
    }
    const float inv = 1.0f / l;
    T* orow = out + (size_t)t * out_stride + (size_t)h * hd;
#pragma unroll
    for (int i = 0; i < AG_MAX_HD / 32; ++i) {
        const int d = lane + 32 * i;
        if (i * 32 < hd && d < hd) orow[d] = dl_from_f32<T>(acc[i] * inv);
    }
}

extern "C" int dl_attention_generic(const void* q, int q_stride, void* out, int out_stride, int dtype,
                                    const void* k_pool, const void* v_pool, int n_pages,
                                    const int32_t* token_seq, const int32_t* token_pos,
                                    const int32_t* block_table, int bt_stride, int n_tokens, int nh, int nkv,
                                    int hd, float scale, int window, float softcap, const float* slopes, void* stream) {
    DL_REQUIRE(n_tokens >= 0 && nh > 0 && nkv > 0 && hd > 0 && n_pages > 0, "attention: bad sizes");
    DL_REQUIRE(nh % nkv == 0, "attention: %d query heads are not a multiple of %d KV heads", nh, nkv);
    DL_REQUIRE(hd <= AG_MAX_HD, "attention: head_dim %d exceeds the supported maximum %d", hd, AG_MAX_HD);
    DL_REQUIRE(q_stride >= nh * hd && out_stride >= nh * hd, "attention: row strides shorter than the rows");
    DL_REQUIRE(window >= 0, "attention: window must be 0 (none) or positive");
    DL_REQUIRE(softcap >= 0.f, "attention: softcap must be 0 (none) or positive");
    if (n_tokens == 0) return DL_OK;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(n_tokens, (nh + AG_WARPS - 1) / AG_WARPS), block(32, AG_WARPS);
    // four heads a block with one KV head between them, and tiles that fit the default shared memory
    const size_t shared_smem = ((size_t)AG_WARPS * hd + 32 * (hd + 1) + (size_t)hd * 33) * sizeof(float);
    if (nh % AG_WARPS == 0 && (nh / nkv) % AG_WARPS == 0 && hd % 4 == 0 && shared_smem <= 48 * 1024 &&
        ((uintptr_t)k_pool % 16) == 0 && ((uintptr_t)v_pool % 16) == 0 && (dtype == DL_F32 || dtype == DL_BF16)) {
        if (dtype == DL_F32)
            attention_generic_shared_kernel<float><<<grid, block, shared_smem, s>>>(
                (const float*)q, q_stride, (float*)out, out_stride, (const float*)k_pool, (const float*)v_pool,
                n_pages, token_seq, token_pos, block_table, bt_stride, nh, nkv, hd, scale, window, softcap, slopes);
        else
            attention_generic_shared_kernel<__nv_bfloat16><<<grid, block, shared_smem, s>>>(
                (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)k_pool,
                (const __nv_bfloat16*)v_pool, n_pages, token_seq, token_pos, block_table, bt_stride, nh, nkv, hd,
                scale, window, softcap, slopes);
        DL_CHECK_LAUNCH("attention_generic");
        return DL_OK;
    }
    const size_t smem = (size_t)AG_WARPS * hd * sizeof(float);
    if (dtype == DL_F32)
        attention_generic_kernel<float><<<grid, block, smem, s>>>(
            (const float*)q, q_stride, (float*)out, out_stride, (const float*)k_pool, (const float*)v_pool,
            n_pages, token_seq, token_pos, block_table, bt_stride, nh, nkv, hd, scale, window, softcap, slopes);
    else if (dtype == DL_BF16)
        attention_generic_kernel<__nv_bfloat16><<<grid, block, smem, s>>>(
            (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)k_pool,
            (const __nv_bfloat16*)v_pool, n_pages, token_seq, token_pos, block_table, bt_stride, nh, nkv, hd,
            scale, window, softcap, slopes);
    else
        return dl_fail(DL_ERR_UNSUPPORTED, "attention: dtype %d", dtype);
    DL_CHECK_LAUNCH("attention_generic");
    return DL_OK;
}
