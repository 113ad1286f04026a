// A chain of element-wise operators in ONE launch: y = op_n(... op_2(op_1(x, b_1), b_2) ..., b_n).
//
// The graph optimiser of the GPU provider collapses chains of unary / binary element-wise nodes into one
// com.ronn::FusedElementwise node (the reference's stated intent, "aggressive elementwise fusion to cut launches",
// crates/ronn-graph/src/passes/provider_specific.rs:48-87, which its pass never implements).  This kernel executes
// such a node: up to 8 operators, the running value kept in fp32 registers between them, 16-byte loads and stores,
// second operands of binary operators either full tensors, vectors broadcast along the last dimension (a bias) or
// scalars.  A chain of n operators therefore costs one read of x, one read per full-size operand and one write,
// instead of n reads and n writes.
#include "common.cuh"

namespace ronn {

constexpr int FEW_MAX_OPS = 8;

struct FusedEwArgs {
  const void* operand[FEW_MAX_OPS];   // second operand of a binary operator, or null
  long inner;                         // length of the last dimension (for vector operands); multiple of 8
  int n_ops;
  int code[FEW_MAX_OPS];              // 0 relu, 1 gelu(tanh), 2 sigmoid, 3 tanh, 4 neg, 5 abs, 6 exp, 7 sqrt, 8 swish,
                                      // 16 add, 17 mul, 18 sub, 19 div
  int mode[FEW_MAX_OPS];              // operand shape: 0 same as x, 1 vector over the last dimension, 2 scalar
};

__device__ __forceinline__ float few_unary(float v, int code) {
  switch (code) {
    case 0: return fmaxf(v, 0.f);
    case 1: return gelu_tanh_f(v);
    case 2: return 1.f / (1.f + __expf(-v));
    case 3: { const float e = __expf(2.f * v); return 1.f - 2.f / (e + 1.f); }
    case 4: return -v;
    case 5: return fabsf(v);
    case 6: return __expf(v);
    case 7: return sqrtf(v);
    default: return v / (1.f + __expf(-v));
  }
}
__device__ __forceinline__ float few_binary(float a, float b, int code) {
  switch (code) {
    case 16: return a + b;
    case 17: return a * b;
    case 18: return a - b;
    default: return a / b;
  }
}

template <class T>
__device__ __forceinline__ void few_chunk(const T* __restrict__ x, T* __restrict__ y, long i, const FusedEwArgs& a) {
  float f[8];
  unpack8<T>(*reinterpret_cast<const Vec8*>(x + i * 8), f);
  // every full-size operand of the chunk is requested before the arithmetic starts
  Vec8 ob[FEW_MAX_OPS];
#pragma unroll
  for (int k = 0; k < FEW_MAX_OPS; ++k)
    if (k < a.n_ops && a.code[k] >= 16 && a.mode[k] != 2) {
      const T* p = reinterpret_cast<const T*>(a.operand[k]);
      ob[k] = *reinterpret_cast<const Vec8*>(a.mode[k] == 0 ? p + i * 8 : p + (i * 8) % a.inner);
    }
#pragma unroll
  for (int k = 0; k < FEW_MAX_OPS; ++k)
    if (k < a.n_ops) {
      const int code = a.code[k];
      if (code < 16) {
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = few_unary(f[j], code);
      } else if (a.mode[k] == 2) {
        const float s = Cvt<T>::to_f(*reinterpret_cast<const T*>(a.operand[k]));
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = few_binary(f[j], s, code);
      } else {
        float g[8];
        unpack8<T>(ob[k], g);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = few_binary(f[j], g[j], code);
      }
    }
  *reinterpret_cast<Vec8*>(y + i * 8) = pack8<T>(f);
}

template <class T>
__global__ void __launch_bounds__(256)
fused_elementwise_kernel(const T* __restrict__ x, T* __restrict__ y, long n8, const __grid_constant__ FusedEwArgs a) {
  pdl_wait();
  pdl_trigger();
  const long stride = long(gridDim.x) * blockDim.x;
  for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < n8; i += stride) few_chunk<T>(x, y, i, a);
}

}  // namespace ronn

using namespace ronn;

// x, y: n elements (n % 8 == 0), 16-byte aligned.  codes / modes / operands: n_ops entries (operands[k] null for unary
// operators).  inner: length of the last dimension, needed (and a multiple of 8) when a mode is 1.  dtype 0 bf16, 1 fp16.
extern "C" int ronn_fused_elementwise(const void* x, void* y, long n, int n_ops, const int* codes, const int* modes,
                                      const void* const* operands, long inner, int dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n_ops < 1 || n_ops > FEW_MAX_OPS) return -1;
  if ((n & 7) || ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15)) return -2;
  FusedEwArgs a;
  a.n_ops = n_ops;
  a.inner = inner > 0 ? inner : 8;
  for (int k = 0; k < FEW_MAX_OPS; ++k) {
    a.code[k] = k < n_ops ? codes[k] : 0;
    a.mode[k] = k < n_ops ? modes[k] : 0;
    a.operand[k] = k < n_ops ? operands[k] : nullptr;
    if (k < n_ops) {
      const int c = a.code[k];
      if (!((c >= 0 && c <= 8) || (c >= 16 && c <= 19))) return -3;
      if (c >= 16) {
        if (a.operand[k] == nullptr || a.mode[k] < 0 || a.mode[k] > 2) return -4;
        if (a.mode[k] != 2 && (reinterpret_cast<uintptr_t>(a.operand[k]) & 15)) return -2;
        if (a.mode[k] == 1 && (inner <= 0 || (inner & 7) || n % inner)) return -5;
      }
    }
  }
  const long n8 = n >> 3;
  long blocks = (n8 + 255) / 256;
  const long cap = long(device_sm_count()) * 8;
  if (blocks > cap) blocks = cap;
  cudaError_t err;
  if (dtype == 0) err = launch(fused_elementwise_kernel<__nv_bfloat16>, dim3(unsigned(blocks)), dim3(256), 0, stream,
                               (const __nv_bfloat16*)x, (__nv_bfloat16*)y, n8, a);
  else if (dtype == 1) err = launch(fused_elementwise_kernel<__half>, dim3(unsigned(blocks)), dim3(256), 0, stream,
                                    (const __half*)x, (__half*)y, n8, a);
  else return -6;
  return (err == cudaSuccess && cudaGetLastError() == cudaSuccess) ? 0 : -100;
}
