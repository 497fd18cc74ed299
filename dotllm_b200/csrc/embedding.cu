// Row gather: token embedding lookup into the float32 residual stream, and selection of
// the rows whose logits are wanted.
//
// Role of the reference's embedding_lookup_* kernels (native/kernels/embedding.cu:30-46,
// native/kernels/embedding_f32out.cu:10-70): one block per output row, the row copied
// with widening to float32 (or kept in bfloat16, for rows of activations that go on to a product).
#include "common.cuh"

template <typename T, typename TOut>
__global__ void __launch_bounds__(256)
gather_rows_kernel(const T* __restrict__ table, int table_stride, const int32_t* __restrict__ ids,
                   TOut* __restrict__ out, int width, int n_table_rows) {
    dl_launch_dependents();
    const int row = blockIdx.x;
    const int id = ids[row];
    TOut* dst = out + (size_t)row * width;
    if (id < 0 || id >= n_table_rows) {          // the host validates ids; never read outside the table
        for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = dl_from_f32<TOut>(0.f);
        return;
    }
    const T* src = table + (size_t)id * table_stride;
    for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = dl_from_f32<TOut>(dl_to_f32<T>(src[c]));
}

// out[r, :] = table[ids[r], :] as `out_dtype`.  table: [n_table_rows, width] of `dtype`, rows
// table_stride elements apart; out: contiguous [n_rows, width], float32 or (from a bfloat16 table) bfloat16.
extern "C" int dl_gather_rows(const void* table, int dtype, int table_stride, const int32_t* ids, void* out, int out_dtype,
                              int n_rows, int width, int n_table_rows, void* stream) {
    DL_REQUIRE(n_rows >= 0 && width > 0 && n_table_rows > 0 && table_stride >= width,
               "gather_rows: bad sizes rows=%d width=%d table=%d stride=%d", n_rows, width, n_table_rows, table_stride);
    if (n_rows == 0) return DL_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == DL_F32 && out_dtype == DL_F32)
        gather_rows_kernel<float, float><<<n_rows, 256, 0, s>>>((const float*)table, table_stride, ids, (float*)out, width, n_table_rows);
    else if (dtype == DL_BF16 && out_dtype == DL_F32)
        gather_rows_kernel<__nv_bfloat16, float><<<n_rows, 256, 0, s>>>((const __nv_bfloat16*)table, table_stride, ids, (float*)out,
                                                                         width, n_table_rows);
    else if (dtype == DL_BF16 && out_dtype == DL_BF16)
        gather_rows_kernel<__nv_bfloat16, __nv_bfloat16><<<n_rows, 256, 0, s>>>((const __nv_bfloat16*)table, table_stride, ids,
                                                                                 (__nv_bfloat16*)out, width, n_table_rows);
    else
        return dl_fail(DL_ERR_UNSUPPORTED, "gather_rows: from dtype %d to dtype %d", dtype, out_dtype);
    DL_CHECK_LAUNCH("gather_rows");
    return DL_OK;
}
