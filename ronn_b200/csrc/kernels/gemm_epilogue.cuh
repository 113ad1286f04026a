// Epilogue shared by the dense GEMM and the implicit-GEMM convolution: bias, activation, residual, store.
#pragma once
#include "common.cuh"

namespace ronn {

struct DenseEpilogue {
  void* C;
  const void* bias;        // [N] in the operand dtype, or null
  const void* residual;    // [M, ldc] in the operand dtype, or null
  int M, N, ldc;
  int m0, n0;
  int act;                 // 0 none, 1 relu, 2 gelu(tanh)
  int out_fp32;
  int res_first;           // 1: add the residual before the activation (convolution blocks), 0: after it

  template <class T>
  __device__ __forceinline__ void run(int row, int col, uint32_t (&r)[32]) const {
    const int gm = m0 + row;
    const int gn = n0 + col;
    if (gm >= M || gn >= N) return;
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
    const bool full = (gn + 32 <= N) && ((ldc & 7) == 0);
    if (bias) {
      const T* b = reinterpret_cast<const T*>(bias) + gn;
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (full || gn + i < N) v[i] += Cvt<T>::to_f(b[i]);
    }
    if (residual && res_first) {
      const T* res = reinterpret_cast<const T*>(residual) + size_t(gm) * ldc + gn;
      if (full) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          Vec8 pk = *reinterpret_cast<const Vec8*>(res + j * 8);
          float f[8];
          unpack8<T>(pk, f);
#pragma unroll
          for (int i = 0; i < 8; ++i) v[j * 8 + i] += f[i];
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (gn + i < N) v[i] += Cvt<T>::to_f(res[i]);
      }
    }
    if (act == 1) {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = fmaxf(v[i], 0.f);
    } else if (act == 2) {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = gelu_tanh_f(v[i]);
    }
    if (residual && !res_first) {
      const T* res = reinterpret_cast<const T*>(residual) + size_t(gm) * ldc + gn;
      if (full) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          Vec8 pk = *reinterpret_cast<const Vec8*>(res + j * 8);
          float f[8];
          unpack8<T>(pk, f);
#pragma unroll
          for (int i = 0; i < 8; ++i) v[j * 8 + i] += f[i];
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (gn + i < N) v[i] += Cvt<T>::to_f(res[i]);
      }
    }
    if (out_fp32) {
      float* out = reinterpret_cast<float*>(C) + size_t(gm) * ldc + gn;
      if (full && (ldc & 3) == 0) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          *reinterpret_cast<float4*>(out + j * 4) = make_float4(v[j * 4], v[j * 4 + 1], v[j * 4 + 2], v[j * 4 + 3]);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (gn + i < N) out[i] = v[i];
      }
    } else {
      T* out = reinterpret_cast<T*>(C) + size_t(gm) * ldc + gn;
      if (full) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float f[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) f[i] = v[j * 8 + i];
          *reinterpret_cast<Vec8*>(out + j * 8) = pack8<T>(f);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (gn + i < N) out[i] = Cvt<T>::from_f(v[i]);
      }
    }
  }
};

}  // namespace ronn
