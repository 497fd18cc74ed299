// An entry point that allocates nothing.  It has no counterpart in the reference (kkokosa/dotLLM
// allocates its device buffers through the driver API whenever it needs them).
//
// Who needs it: callers that cannot, or may not, obtain device memory at the moment they want a
// product computed - a plug-in running inside a host that reserved the whole GPU for its own arena
// at start-up, a control loop with a latency budget that rules out the allocator's locks and
// implicit synchronisation, or glue code that has raw device pointers but no allocator at all.
// They still own their inputs and outputs; what they cannot supply is the kernel's scratch.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Bytes of device memory that every GPU loading this library keeps for the scratch until the
// process exits, and the most 16-row tiles of W a call may span.
#define DL_GEMM_SKINNY_STATIC_SCRATCH_BYTES (8 * 1024 * 1024)
#define DL_GEMM_SKINNY_STATIC_MAX_TILES 16384

// y = x W^T (fuse_swiglu == 0, W [N, K]) or silu(x Wg^T) * (x Wu^T) (fuse_swiglu == 1, W [2N, K]):
// the same arithmetic, in the same order, as dl_gemm_skinny_bf16, with the split-k scratch taken
// from a fixed array inside the library instead of from the caller.
//
//   x    bfloat16 [M, K], rows x_stride elements apart, 1 <= M <= 16, K a multiple of 8
//   w    bfloat16, contiguous rows of K
//   out  [M, N] rows out_stride apart; out_dtype 0 = float32, 1 = bfloat16
//
// Returns 0, or a status whose text dl_last_error() gives.  Shapes whose partial sums do not fit
// the fixed scratch are refused with a message that says so; nothing is launched then.
//
// * No cudaMalloc, cudaFree or allocating library call is made, now or later.
// * The first call on a device looks up the scratch array's device address (one
//   cudaGetSymbolAddress, with that device current) and remembers it; make that first call
//   outside any stream capture.
// * All calls on a device share the one array.  The call clears what must start at zero, but two
//   calls that overlap on the GPU (different streams, no ordering between them) race on it.
int dl_gemm_skinny_bf16_static(const void* x, int x_stride, const void* w, void* out, int out_dtype,
                               int out_stride, int M, int N, int K, int fuse_swiglu, void* stream);

#ifdef __cplusplus
}
#endif
