// Tensor-map (TMA) helpers: host-side encoding of 2-D bfloat16 row-major matrices, and the
// device-side tiled bulk copy global -> shared that completes on an mbarrier.
//
// The driver's encoder is looked up at run time (cudaGetDriverEntryPoint), so the library links
// against the CUDA runtime only.  Copies issued here are plain CTA-local loads: no cluster
// multicast anywhere.
//
// Alignment rules a caller must keep (the hardware checks none of them at copy time): the matrix
// base is 16-byte aligned, the row pitch is a multiple of 16 bytes, and the innermost coordinate
// of every copy times the element size is a multiple of 16 bytes (a multiple of 8 bfloat16).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

enum DlTmapSwizzle { DL_TMAP_SWIZZLE_NONE = 0, DL_TMAP_SWIZZLE_128B = 1 };

// Encode a map over `rows` x `cols` bfloat16 with `pitch_bytes` between rows; each copy moves a
// box of box_rows x box_cols (box_cols * 2 bytes a multiple of 16, at most 256 elements per side;
// with the 128-byte swizzle box_cols * 2 == 128).  Out-of-range parts of a box read as zero.
// Returns 0 or a negative code (-1: no driver entry point, -2: the encoder refused).
int dl_tmap_encode_2d_bf16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_bytes,
                           uint32_t box_rows, uint32_t box_cols, int swizzle);

// The same through a per-process table keyed by (base, shape, pitch, box, swizzle): encoding costs a
// driver call, and a model's matrices and step buffers come back launch after launch.  Thread-safe.
int dl_tmap_cached_2d_bf16(CUtensorMap* out, const void* base, unsigned long long rows, unsigned long long cols,
                           unsigned long long pitch_bytes, uint32_t box_rows, uint32_t box_cols, int swizzle);

#ifdef __CUDACC__
// Copy the box whose first element is (row, col) into shared memory; `bar` receives the bytes.
__device__ __forceinline__ void dl_tma_load_2d(void* smem_dst, const CUtensorMap* map, int col, int row,
                                               uint64_t* bar) {
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem_dst);
    const uint32_t mbar = (uint32_t)__cvta_generic_to_shared(bar);
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(col), "r"(row), "r"(mbar)
        : "memory");
}
// A cache policy for data that is read once and is larger than the L2 (a decode step's weights): the
// lines are the first to be evicted, so that what is read again (activations, partial sums, code) stays.
__device__ __forceinline__ uint64_t dl_stream_policy() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
// dl_tma_load_2d with a cache policy for the lines it brings into the L2.
__device__ __forceinline__ void dl_tma_load_2d_hint(void* smem_dst, const CUtensorMap* map, int col, int row,
                                                    uint64_t* bar, uint64_t policy) {
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem_dst);
    const uint32_t mbar = (uint32_t)__cvta_generic_to_shared(bar);
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;"
        ::"r"(dst), "l"(map), "r"(col), "r"(row), "r"(mbar), "l"(policy)
        : "memory");
}
// Copy `bytes` (a multiple of 16, both addresses 16-byte aligned) of contiguous global memory into
// shared memory; `bar` receives the bytes.
__device__ __forceinline__ void dl_bulk_load(void* smem_dst, const void* src, uint32_t bytes, uint64_t* bar) {
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem_dst);
    const uint32_t mbar = (uint32_t)__cvta_generic_to_shared(bar);
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(mbar)
                 : "memory");
}
#endif
