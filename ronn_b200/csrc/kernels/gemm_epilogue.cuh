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

  // `stage` (optional): 32 x 80 bytes of shared memory owned by the calling warp.  With it, and when the whole warp
  // calls with the same `col`, 16-bit results leave as 64 contiguous bytes per row from 4 lanes (8 rows per store
  // instruction) instead of 32 rows of 16 bytes, which halves the number of write transactions and fills every sector.
  template <class T>
  __device__ __forceinline__ void run(int row, int col, uint32_t (&r)[32], uint8_t* stage = nullptr) const {
    const int gm = m0 + row;
    const int gn = n0 + col;
    if (gn >= N) return;                         // uniform across the warp
    // re-shaping the stores through shared memory pays for bandwidth-bound results; a decode-sized GEMM (a few row
    // tiles) is a latency chain and keeps the direct stores
    const bool staged = stage != nullptr && M >= 1024 && !out_fp32 && (gn + 32 <= N) && ((ldc & 7) == 0);
    if (gm >= M && !staged) return;
    if (gm >= M) {                               // staged path: rows past the end only take part in the exchange
      __syncwarp();
      store_staged<T>(stage, gm - (threadIdx.x & 31), gn);
      return;
    }
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
    } else if (staged) {
      uint8_t* mine = stage + (threadIdx.x & 31) * 80;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float f[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = v[j * 8 + i];
        *reinterpret_cast<Vec8*>(mine + j * 16) = pack8<T>(f);
      }
      __syncwarp();
      store_staged<T>(stage, gm - (threadIdx.x & 31), gn);
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

  // second half of the staged store: lane l writes 16-byte piece (l % 4) of rows (l / 4) + 8 i
  template <class T>
  __device__ __forceinline__ void store_staged(const uint8_t* stage, int base_row, int gn) const {
    const int lane = threadIdx.x & 31;
    const int piece = lane & 3;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int rr = (lane >> 2) + 8 * i;
      if (base_row + rr < M) {
        const Vec8 pk = *reinterpret_cast<const Vec8*>(stage + rr * 80 + piece * 16);
        *reinterpret_cast<Vec8*>(reinterpret_cast<T*>(C) + size_t(base_row + rr) * ldc + gn + piece * 8) = pk;
      }
    }
    __syncwarp();                                // the stage is free for the warp's next chunk
  }
};

}  // namespace ronn
