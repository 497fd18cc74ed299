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
// * No cudaMalloc, cudaFree or allocating library call is made, now or later.  On the host the call
//   takes two short mutexes (the per-device address table and the table of tensor maps) and, the first
//   time it sees a matrix, encodes a tensor map for it (one driver call) and inserts it into a
//   host-side map: a caller that must not block on host locks either should make one warm-up call per
//   matrix first.
// * The first call on a device looks up the scratch array's device address (one
//   cudaGetSymbolAddress, with that device current) and remembers it; make that first call
//   outside any stream capture.
// * All calls on a device share the one array.  The call clears what must start at zero, but two
//   calls that overlap on the GPU (different streams, no ordering between them) race on it.
// * Every wait inside the kernel is bounded.  A wait that expires leaves `out` incomplete and sets a
//   word inside the scratch array; the call itself has long returned 0 by then.  Ask for that word
//   with dl_gemm_skinny_static_status at the next point where the results are needed.
int dl_gemm_skinny_bf16_static(const void* x, int x_stride, const void* w, void* out, int out_dtype,
                               int out_stride, int M, int N, int K, int fuse_swiglu, void* stream);

// Waits for `stream`, writes the give-up word of the static calls on the current device to *code
// (0: all waits were served; 1, 3, 5: a producer's, a consumer's, the row factors' wait expired)
// and clears it.  Allocates nothing.
int dl_gemm_skinny_static_status(int* code, void* stream);

#ifdef __cplusplus
}
#endif
