// Split-K GEMM + reduction with its scratch in a fixed device array: an entry point for callers that cannot allocate.
//
// Who cannot allocate: a host that has handed all device memory to its own planner (a serving process whose KV cache
// was sized to fill the GPU leaves no room for a growing workspace, and an allocation failure in the middle of a
// request is not an option there); a real-time loop in which a device allocation is unacceptable because it may
// synchronise the whole device; and plain C callers that link this library without PyTorch's caching allocator, which
// is what the regular split-K path (ops/kernels.py: splitk_workspace) relies on.  For them the partial-sum panels
// live in the array below, whose address is looked up once per device; no cudaMalloc, cudaFree or other allocating
// routine is reached from here.
#include "no_alloc.h"

#include <cuda_runtime.h>

// existing launchers of this library (gemm_umma.cu, elementwise.cu); both take the scratch as a plain pointer
extern "C" int ronn_gemm_splitk(const void* A, const void* W, float* workspace, int M, int N, int K, int lda, int ldw,
                                int dtype, int bn, int splitk, int* splitk_out, uint32_t* status, cudaStream_t stream);
extern "C" int ronn_splitk_finalize(const float* ws, int S, const void* bias, const void* residual, void* sum_out,
                                    const void* gamma, const void* beta, void* y, long rows, int N, float eps,
                                    int act, int norm, int dtype, cudaStream_t stream);

// 16 MiB of fp32 partial sums per device, e.g. 4 slices x 256 rows x 4096 columns.
static __device__ __align__(256) float g_no_alloc_scratch[RONN_NO_ALLOC_MAX_FLOATS];

namespace {

constexpr int kMaxDevices = 64;
float* g_scratch_ptr[kMaxDevices] = {};      // resolved address of g_no_alloc_scratch per device ordinal

// The symbol has one instance per device; its address is resolved on first use there and cached.
int scratch_for_current_device(float** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return RONN_NO_ALLOC_E_SYMBOL;
  if (g_scratch_ptr[dev] == nullptr) {
    float* ptr = nullptr;
    cudaError_t rc = cudaGetSymbolAddress((void**)&ptr, g_no_alloc_scratch);
    if (rc != cudaSuccess || ptr == nullptr) {
      cudaGetLastError();                    // leave no sticky error behind for the caller's next CUDA call
      return RONN_NO_ALLOC_E_SYMBOL;
    }
    g_scratch_ptr[dev] = ptr;
  }
  *out = g_scratch_ptr[dev];
  return 0;
}

int effective_slices(int K, int splitk) {
  const int num_kb = (K + 63) / 64;
  if (splitk < 1) splitk = 1;
  if (splitk > num_kb) splitk = num_kb;
  const int per = (num_kb + splitk - 1) / splitk;
  return (num_kb + per - 1) / per;
}

}  // namespace

extern "C" long ronn_no_alloc_scratch_floats(int M, int N, int K, int splitk) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  return long(effective_slices(K, splitk)) * long(M) * long(N);
}

extern "C" const char* ronn_no_alloc_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case RONN_NO_ALLOC_E_TOO_LARGE:
      return "split-K slices x M x N exceeds the built-in scratch (RONN_NO_ALLOC_MAX_FLOATS = 4194304 floats); "
             "use fewer slices or the allocating entry point";
    case RONN_NO_ALLOC_E_SYMBOL: return "the scratch array could not be resolved on the current device";
    case RONN_NO_ALLOC_E_ARGS: return "null operand or non-positive size";
    case RONN_NO_ALLOC_E_SHAPE:
      return "N must be a multiple of 8 and at most 32768, K / lda / ldw multiples of 8, dtype 0 (bf16) or 1 (fp16)";
    default: return "error reported by the GEMM launcher";
  }
}

extern "C" int ronn_gemm_splitk_no_alloc(const void* A, const void* W, void* out, const void* bias,
                                         const void* residual, int M, int N, int K, int lda, int ldw, int dtype,
                                         int splitk, uint32_t* status, cudaStream_t stream) {
  if (A == nullptr || W == nullptr || out == nullptr || M <= 0 || N <= 0 || K <= 0) return RONN_NO_ALLOC_E_ARGS;
  // everything either kernel would refuse is refused here, before the first launch: a call either runs both passes
  // or touches nothing (neither the scratch nor `out`)
  if ((N & 7) || N > RONN_NO_ALLOC_MAX_N || (K & 7) || (lda & 7) || (ldw & 7) || (dtype != 0 && dtype != 1))
    return RONN_NO_ALLOC_E_SHAPE;
  if (ronn_no_alloc_scratch_floats(M, N, K, splitk) > long(RONN_NO_ALLOC_MAX_FLOATS)) return RONN_NO_ALLOC_E_TOO_LARGE;
  float* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc != 0) return rc;
  int slices = 0;
  rc = ronn_gemm_splitk(A, W, scratch, M, N, K, lda, ldw, dtype, /*bn=*/0, splitk < 1 ? 1 : splitk, &slices, status,
                        stream);
  if (rc != 0) return rc;
  return ronn_splitk_finalize(scratch, slices, bias, residual, out, nullptr, nullptr, nullptr, long(M), N, 0.f,
                              /*act=*/0, /*norm=*/0, dtype, stream);
}
