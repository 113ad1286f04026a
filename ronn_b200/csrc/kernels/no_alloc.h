// Entry point that never allocates.  It has no counterpart in the reference runtime, whose operators all go through
// an allocating tensor library; it exists for hosts of this kernel library that cannot ask for device memory at
// call time.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Capacity of the built-in scratch area in floats (16 MiB): split-K slices x M x N of one call must fit.
#define RONN_NO_ALLOC_MAX_FLOATS (4 * 1024 * 1024)

// Error codes specific to this entry point (other negative values come from the GEMM launcher itself).
#define RONN_NO_ALLOC_E_TOO_LARGE (-40)   // slices * M * N exceeds RONN_NO_ALLOC_MAX_FLOATS
#define RONN_NO_ALLOC_E_SYMBOL (-41)      // the scratch symbol could not be resolved on the current device
#define RONN_NO_ALLOC_E_ARGS (-42)        // null pointer or non-positive size
#define RONN_NO_ALLOC_E_SHAPE (-43)       // N not a multiple of 8 or above RONN_NO_ALLOC_MAX_N; K, lda or ldw not a multiple of 8

// Widest output row the reduction pass takes (it keeps a row in registers across 1024 threads).
#define RONN_NO_ALLOC_MAX_N 32768

// out[M, N] = A[M, K] * W[N, K]^T + bias + residual, computed as `splitk` K-slices on the tensor cores whose fp32
// partial panels live in a fixed scratch array inside the library, followed by one reduction pass.
//   A, W, out, bias (or null), residual (or null): device pointers, 16-bit elements (dtype 0 = bf16, 1 = fp16);
//   lda / ldw in elements; out and residual are dense [M, N]; K, lda, ldw multiples of 8; N a multiple of 8 and at
//   most RONN_NO_ALLOC_MAX_N.  A call that breaks one of these rules returns RONN_NO_ALLOC_E_SHAPE before anything
//   is launched: neither the scratch nor `out` is written.
//   status: device word that receives a non-zero code if a bounded wait inside the kernel gave up (may be null).
// Returns 0, or a negative code; ronn_no_alloc_strerror() turns the codes above into text.
//
// What a caller has to know:
//  * The first call on each device resolves the address of the scratch array (cudaGetSymbolAddress) and sets the
//    kernels' launch attributes on that device (both are kept per device ordinal, so a process that drives several
//    GPUs makes one such call on each).  Make that first call during start-up, before any stream capture begins.
//  * There is ONE scratch array per device, shared by every call.  Two calls whose execution may overlap (different
//    streams without an ordering between them, or different host threads) race on it; order them on one stream or
//    with events.
//  * Nothing in the scratch has to be zero on entry and nothing is kept in it between calls: every K-slice writes its
//    whole [M, N] panel before the reduction pass reads it.
int ronn_gemm_splitk_no_alloc(const void* A, const void* W, void* out, const void* bias, const void* residual,
                              int M, int N, int K, int lda, int ldw, int dtype, int splitk, uint32_t* status,
                              cudaStream_t stream);

// Floats of scratch the call above would need for these sizes (slices after clamping to the number of K blocks).
long ronn_no_alloc_scratch_floats(int M, int N, int K, int splitk);

const char* ronn_no_alloc_strerror(int code);

#ifdef __cplusplus
}
#endif
