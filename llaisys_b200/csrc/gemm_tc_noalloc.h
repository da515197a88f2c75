// An entry point of the tensor-core matrix product that allocates nothing.
//
// This function has no counterpart in xsmccc/llaisys; it exists for callers of this library that
// must not allocate device memory at the time they call it: code that runs inside a region where
// the allocator is off limits (a real-time loop that may not block on the driver, a host
// callback, a plug-in that was handed a fixed memory budget by its host program).  The regular
// entry point, llb_gemm_tc, splits the reduction over several thread blocks when the weight has
// few row blocks and needs a scratch buffer for their partial sums, which its caller has to
// allocate.  Here that scratch is a fixed array inside the library's device image instead.
//
//   Y[T, N] = X[T, K] * W[N, K]^T (+ bias[N]),  bfloat16 operands, float32 accumulation.
//
// Limits.  The built-in scratch holds LLB_NOALLOC_SCRATCH_FLOATS float32 values (4 MiB) and
// LLB_NOALLOC_TILES tile counters, on every GPU that loads this library, from load until exit.
// A call whose partial tiles need more, i.e.
//     ceil(N / 128) * ceil(T / bn) * splits * bn * 128  >  LLB_NOALLOC_SCRATCH_FLOATS,
// or whose tile count exceeds LLB_NOALLOC_TILES, is refused with LLB_NOALLOC_TOO_LARGE and
// launches nothing; ask for fewer splits (splits = 1 needs no scratch at all).
//
// First call on a device.  The first call made while a given device is current looks up the
// device addresses of the built-in arrays (cudaGetSymbolAddress) and keeps them; later calls on
// that device reuse them.  Make that first call outside any CUDA stream capture.
//
// Sharing.  All calls on a device use the same scratch.  Calls on one stream follow one another
// and are safe.  Two calls that may run on the GPU at the same time (different streams) race on
// the scratch and give wrong results: do not overlap them.  The counters are back at zero when
// a call's kernel ends (a block that gives up a wait still arrives at its counter), and a partial
// tile is always written before it is read, so nothing has to be cleared between calls.
//
// Errors on the device.  Every wait inside the kernel is bounded.  If one runs out (it never
// should), the block records a code in an error word that lives beside the scratch, and the
// output of that call is not valid although the call returned 0: the launch is asynchronous.
// llb_gemm_tc_noalloc_status() waits for the stream, returns that word (0: every call since the
// last query was complete) and clears it.  Callers that cannot afford to trust blindly ask it
// before they use a result; it allocates nothing either.
//
// The function calls no cudaMalloc, cudaFree, or any other allocating routine, on the device or
// on the host heap; tensor maps are encoded on the stack on every call.
#pragma once
#include <cuda_runtime.h>

#define LLB_NOALLOC_SCRATCH_FLOATS (1 << 20)
#define LLB_NOALLOC_TILES 4096
#define LLB_NOALLOC_TOO_LARGE (-3001)     /* the call needs more scratch or more tile counters than are built in */
#define LLB_NOALLOC_SETUP_FAILED (-3002)  /* cudaGetSymbolAddress or cudaGetDevice failed on the first call */

#ifdef __cplusplus
extern "C" {
#endif

// X: [T, K] bfloat16, row stride ldx elements (K and ldx multiples of 8, 16-byte aligned).
// W: [N, K] bfloat16, dense, 16-byte aligned.  bias: [N] bfloat16 (bias_dtype 1) or float32 (0), or null.
// Y: [T, N] bfloat16 (y_dtype 1) or float32 (0), row stride ldy elements.
// bn: tokens per tile: 16, 32, 64, 128 or 256.  splits: blocks the reduction is divided over (>= 1).
// Returns 0, a cudaError_t (> 0) of the launch, or one of the negative codes above / of llb_gemm_tc.
__attribute__((visibility("default")))
int llb_gemm_tc_noalloc(const void* X, const void* W, const void* bias, int bias_dtype, void* Y, int y_dtype,
                        int T, int N, int K, int ldx, int ldy, int bn, int splits, cudaStream_t stream);

// Waits for `stream`, then returns 0 if no call on the current device gave up a wait since the last
// query, else the code of the wait (101-104) after clearing it, or LLB_NOALLOC_SETUP_FAILED.
__attribute__((visibility("default")))
int llb_gemm_tc_noalloc_status(cudaStream_t stream);

#ifdef __cplusplus
}
#endif
