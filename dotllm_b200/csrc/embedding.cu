// Row gather: token embedding lookup into the float32 residual stream, and selection of
// the rows whose logits are wanted.
//
// Role of the reference's embedding_lookup_* kernels (native/kernels/embedding.cu:30-46,
// native/kernels/embedding_f32out.cu:10-70): one block per output row, the row copied
// with widening to float32.
#include "common.cuh"

template <typename T>
__global__ void __launch_bounds__(256)
gather_rows_kernel(const T* __restrict__ table, const int32_t* __restrict__ ids,
                   float* __restrict__ out, int width, int n_table_rows) {
    dl_launch_dependents();
    const int row = blockIdx.x;
    const int id = ids[row];
    float* dst = out + (size_t)row * width;
    if (id < 0 || id >= n_table_rows) {          // the host validates ids; never read outside the table
        for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = 0.f;
        return;
    }
    const T* src = table + (size_t)id * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = dl_to_f32<T>(src[c]);
}

// out[r, :] = float32(table[ids[r], :]).  table: [n_table_rows, width] of `dtype`.
extern "C" int dl_gather_rows(const void* table, int dtype, const int32_t* ids, float* out,
                              int n_rows, int width, int n_table_rows, void* stream) {
    DL_REQUIRE(n_rows >= 0 && width > 0 && n_table_rows > 0, "gather_rows: bad sizes rows=%d width=%d table=%d",
               n_rows, width, n_table_rows);
    if (n_rows == 0) return DL_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == DL_F32)
        gather_rows_kernel<float><<<n_rows, 256, 0, s>>>((const float*)table, ids, out, width, n_table_rows);
    else if (dtype == DL_BF16)
        gather_rows_kernel<__nv_bfloat16><<<n_rows, 256, 0, s>>>((const __nv_bfloat16*)table, ids, out, width,
                                                                  n_table_rows);
    else
        return dl_fail(DL_ERR_UNSUPPORTED, "gather_rows: dtype %d", dtype);
    DL_CHECK_LAUNCH("gather_rows");
    return DL_OK;
}
