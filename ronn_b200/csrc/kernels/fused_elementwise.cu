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

// One operator on the 8 values of a chunk.  The switch sits outside the loop over the values: one branch per
// operator and chunk, straight-line vector code inside.
__device__ __forceinline__ void few_unary8(float (&f)[8], int code) {
#define RONN_FEW_CASE(C, EXPR)              \
  case C: {                                 \
    _Pragma("unroll") for (int j = 0; j < 8; ++j) { const float v = f[j]; f[j] = (EXPR); } \
  } break;
  switch (code) {
    RONN_FEW_CASE(0, fmaxf(v, 0.f))
    RONN_FEW_CASE(1, gelu_tanh_f(v))
    RONN_FEW_CASE(2, __fdividef(1.f, 1.f + __expf(-v)))
    RONN_FEW_CASE(3, 1.f - __fdividef(2.f, __expf(2.f * v) + 1.f))
    RONN_FEW_CASE(4, -v)
    RONN_FEW_CASE(5, fabsf(v))
    RONN_FEW_CASE(6, __expf(v))
    RONN_FEW_CASE(7, sqrtf(v))
    default: {
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = __fdividef(f[j], 1.f + __expf(-f[j]));
    }
  }
#undef RONN_FEW_CASE
}
__device__ __forceinline__ void few_binary8(float (&f)[8], const float (&g)[8], int code) {
  switch (code) {
    case 16:
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] += g[j];
      break;
    case 17:
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] *= g[j];
      break;
    case 18:
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] -= g[j];
      break;
    default:
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = f[j] / g[j];
  }
}

// U chunks of 8 values per thread and step: every load of the step (x and the full-size operands of all U chunks) is
// issued before the arithmetic starts.  `inner8`: chunks per row of the last dimension, for vector operands (the
// column of a chunk is a 32-bit remainder: a 64-bit one costs ~100 instructions per chunk).
template <class T, int U>
__device__ __forceinline__ void few_step(const T* __restrict__ x, T* __restrict__ y, long i0, long stride, long n8,
                                         const FusedEwArgs& a, uint32_t inner8) {
  constexpr int PRE = 4;                 // operands of the first PRE operators are requested up front (registers)
  Vec8 xv[U];
  Vec8 ob[U][PRE];
  auto operand_chunk = [&](int k, long i) -> Vec8 {
    const T* p = reinterpret_cast<const T*>(a.operand[k]);
    const long off = a.mode[k] == 0 ? i * 8 : long(uint32_t(i) % inner8) * 8;      // n8 < 2^32 (launcher)
    return *reinterpret_cast<const Vec8*>(p + off);
  };
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const long i = i0 + u * stride;
    if (i < n8) {
      xv[u] = *reinterpret_cast<const Vec8*>(x + i * 8);
#pragma unroll
      for (int k = 0; k < PRE; ++k)
        if (k < a.n_ops && a.code[k] >= 16 && a.mode[k] != 2) ob[u][k] = operand_chunk(k, i);
    }
  }
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const long i = i0 + u * stride;
    if (i >= n8) continue;
    float f[8];
    unpack8<T>(xv[u], f);
#pragma unroll
    for (int k = 0; k < FEW_MAX_OPS; ++k)
      if (k < a.n_ops) {
        const int code = a.code[k];
        if (code < 16) {
          few_unary8(f, code);
        } else {
          float g[8];
          if (a.mode[k] == 2) {
            const float sc = Cvt<T>::to_f(*reinterpret_cast<const T*>(a.operand[k]));
#pragma unroll
            for (int j = 0; j < 8; ++j) g[j] = sc;
          } else if (k < PRE) {
            unpack8<T>(ob[u][k], g);
          } else {
            unpack8<T>(operand_chunk(k, i), g);
          }
          few_binary8(f, g, code);
        }
      }
    *reinterpret_cast<Vec8*>(y + i * 8) = pack8<T>(f);
  }
}

// One chunk per thread and step at the highest occupancy the register file allows: measured 192 us against 241 us for two
// chunks per step at three CTAs per SM and 420 us for four (131072 x 1024 bf16, four operators): resident warps hide
// the load latency better than loads in flight per thread do.
template <class T>
__global__ void __launch_bounds__(256, 6)
fused_elementwise_kernel(const T* __restrict__ x, T* __restrict__ y, long n8, const __grid_constant__ FusedEwArgs a) {
  pdl_wait();
  pdl_trigger();
  constexpr int U = 1;
  const long stride = long(gridDim.x) * blockDim.x;
  const uint32_t inner8 = uint32_t(a.inner >> 3) ? uint32_t(a.inner >> 3) : 1u;
  for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < n8; i += U * stride) few_step<T, U>(x, y, i, stride, n8, a, inner8);
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
  if ((n >> 3) >= (1l << 32)) return -7;                     // chunk indices are reduced modulo the row in 32 bits
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
  const long cap = long(device_sm_count()) * 12;
  if (blocks > cap) blocks = cap;
  cudaError_t err;
  if (dtype == 0) err = launch(fused_elementwise_kernel<__nv_bfloat16>, dim3(unsigned(blocks)), dim3(256), 0, stream,
                               (const __nv_bfloat16*)x, (__nv_bfloat16*)y, n8, a);
  else if (dtype == 1) err = launch(fused_elementwise_kernel<__half>, dim3(unsigned(blocks)), dim3(256), 0, stream,
                                    (const __half*)x, (__half*)y, n8, a);
  else return -6;
  return (err == cudaSuccess && cudaGetLastError() == cudaSuccess) ? 0 : -100;
}
