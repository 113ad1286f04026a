// Dense bf16/fp16 GEMM on tcgen05 tensor cores:  C[M,N] = act(A[M,K] * W[N,K]^T + bias) + residual.
//
// A is row-major activations, W is stored K-major ("[N,K]", the transposed form of an ONNX MatMul
// weight), so both operands are K-major UMMA tiles loaded by TMA with the 128-byte swizzle.  The
// accumulator lives in TMEM; the epilogue applies bias, activation (none / ReLU / tanh-GELU) and an
// optional residual add and writes bf16/fp16 or fp32.
//
// Replaces the reference's library matmul (crates/ronn-core/src/ops/matrix.rs:27-60) and its two
// never-compiled templates: the scalar fused matmul+bias and the one-wmma-tile-per-warp GEMM
// (crates/ronn-providers/src/gpu/cuda_kernels.rs:319-347, 479-534).
#include "common.cuh"
#include "tma_desc.cuh"
#include "umma_gemm.cuh"

namespace ronn {

struct DenseEpilogue {
  void* C;
  const void* bias;        // [N] in the operand dtype, or null
  const void* residual;    // [M, ldc] in the operand dtype, or null
  int M, N, ldc;
  int m0, n0;
  int act;                 // 0 none, 1 relu, 2 gelu(tanh)
  int out_fp32;

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
    if (act == 1) {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = fmaxf(v[i], 0.f);
    } else if (act == 2) {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = gelu_tanh_f(v[i]);
    }
    if (residual) {
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
        for (int i = 0; i < 32 && gn + i < N; ++i) v[i] += Cvt<T>::to_f(res[i]);
      }
    }
    if (out_fp32) {
      float* out = reinterpret_cast<float*>(C) + size_t(gm) * ldc + gn;
      if (full && (ldc & 3) == 0) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          *reinterpret_cast<float4*>(out + j * 4) = make_float4(v[j * 4], v[j * 4 + 1], v[j * 4 + 2], v[j * 4 + 3]);
      } else {
        for (int i = 0; i < 32 && gn + i < N; ++i) out[i] = v[i];
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
        for (int i = 0; i < 32 && gn + i < N; ++i) out[i] = Cvt<T>::from_f(v[i]);
      }
    }
  }
};

template <class T>
struct DenseEpiCall {
  DenseEpilogue e;
  __device__ __forceinline__ void operator()(int row, int col, uint32_t (&r)[32]) const { e.run<T>(row, col, r); }
};

template <int BN, int STAGES, class T>
__global__ void __launch_bounds__(GEMM_THREADS)
gemm_dense_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                  DenseEpilogue epi, int K, uint32_t idesc, uint32_t* status) {
  extern __shared__ uint8_t dyn_smem[];
  const int n0 = blockIdx.x * BN;
  const int m0 = blockIdx.y * GEMM_BM;
  epi.m0 = m0;
  epi.n0 = n0;
  TmaALoader al{&map_a, m0};
  DenseEpiCall<T> call{epi};
  int num_kb = (K + 63) / 64;
  int kb0 = 0;
  if (gridDim.z > 1) {
    // split-K: this CTA owns k-blocks [kb0, kb0 + num_kb) and writes raw fp32 partial sums to slice z of the workspace
    const int per = (num_kb + gridDim.z - 1) / gridDim.z;
    kb0 = blockIdx.z * per;
    num_kb = min(per, num_kb - kb0);
    call.e.C = reinterpret_cast<float*>(epi.C) + size_t(blockIdx.z) * size_t(epi.M) * size_t(epi.ldc);
  }
  gemm_tile<BN, STAGES, 0, TmaALoader, DenseEpiCall<T>>(dyn_smem, al, &map_b, n0, num_kb, 64, idesc, status, call, kb0);
}

template <int BN, int STAGES, class T>
static int launch_dense(const CUtensorMap& ma, const CUtensorMap& mb, DenseEpilogue epi, int M, int N, int K,
                        int is_bf16, uint32_t* status, cudaStream_t stream, int splitk = 1) {
  using L = GemmSmemLayout<BN, STAGES>;
  auto kern = gemm_dense_kernel<BN, STAGES, T>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYN_SMEM) != cudaSuccess) return -10;
    configured = true;
  }
  dim3 grid((N + BN - 1) / BN, (M + GEMM_BM - 1) / GEMM_BM, splitk);
  uint32_t idesc = umma_idesc(GEMM_BM, BN, is_bf16 ? 1u : 0u, 1u);
  cudaError_t err = launch(kern, grid, dim3(GEMM_THREADS), size_t(L::DYN_SMEM), stream, ma, mb, epi, K, idesc, status);
  return (err == cudaSuccess && cudaGetLastError() == cudaSuccess) ? 0 : -11;
}

int pick_bn(int M, int N) {
  const int mt = (M + GEMM_BM - 1) / GEMM_BM;
  const int cands[4] = {256, 128, 64, 32};
  for (int i = 0; i < 4; ++i) {
    int bn = cands[i];
    if (bn > 32 && N < bn) continue;
    int ctas = mt * ((N + bn - 1) / bn);
    if (ctas >= 120) return bn;
  }
  return 32;
}

}  // namespace ronn

using namespace ronn;

// dtype: 0 = bf16, 1 = fp16.  act: 0 none, 1 relu, 2 gelu.  bn: 0 = auto, else 32|64|128|256.
// lda/ldw/ldc in elements; K and the leading dimensions must be multiples of 8.
// Returns 0 on success, negative on configuration errors.
extern "C" int ronn_gemm(const void* A, const void* W, void* C, const void* bias, const void* residual, int M, int N,
                         int K, int lda, int ldw, int ldc, int dtype, int act, int out_fp32, int bn,
                         uint32_t* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return -1;
  if ((K & 7) || (lda & 7) || (ldw & 7)) return -2;
  if (bn == 0) bn = pick_bn(M, N);
  CUtensorMap ma, mb;
  int rc = make_tmap_2d(&ma, A, uint64_t(M), uint64_t(K), uint64_t(lda), GEMM_BM, 64, 2);
  if (rc) return rc - 20;
  rc = make_tmap_2d(&mb, W, uint64_t(N), uint64_t(K), uint64_t(ldw), uint32_t(bn), 64, 2);
  if (rc) return rc - 30;
  DenseEpilogue e{C, bias, residual, M, N, ldc, 0, 0, act, out_fp32};
  const int bf = dtype == 0;
#define RONN_DISPATCH(BN_, ST_)                                                                       \
  return bf ? launch_dense<BN_, ST_, __nv_bfloat16>(ma, mb, e, M, N, K, 1, status, stream)            \
            : launch_dense<BN_, ST_, __half>(ma, mb, e, M, N, K, 0, status, stream)
  switch (bn) {
    case 256: RONN_DISPATCH(256, 4);
    case 128: RONN_DISPATCH(128, 3);
    case 64: RONN_DISPATCH(64, 4);
    case 32: RONN_DISPATCH(32, 5);
    default: return -3;
  }
#undef RONN_DISPATCH
}

// Split-K variant for skinny problems (decode: M <= 256).  Each of `splitk` K-slices writes an fp32 partial
// [M, N] to workspace slice z; ronn_splitk_finalize sums the slices and applies bias / residual / norm.
// The effective split count (every slice non-empty) is returned through *splitk_out.
extern "C" int ronn_gemm_splitk(const void* A, const void* W, float* workspace, int M, int N, int K, int lda, int ldw,
                                int dtype, int bn, int splitk, int* splitk_out, uint32_t* status,
                                cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || splitk < 1) return -1;
  if ((K & 7) || (lda & 7) || (ldw & 7) || (N & 3)) return -2;
  const int num_kb = (K + 63) / 64;
  if (splitk > num_kb) splitk = num_kb;
  const int per = (num_kb + splitk - 1) / splitk;
  splitk = (num_kb + per - 1) / per;
  if (splitk_out) *splitk_out = splitk;
  if (bn == 0) bn = N >= 128 ? 128 : (N >= 64 ? 64 : 32);
  CUtensorMap ma, mb;
  int rc = make_tmap_2d(&ma, A, uint64_t(M), uint64_t(K), uint64_t(lda), GEMM_BM, 64, 2);
  if (rc) return rc - 20;
  rc = make_tmap_2d(&mb, W, uint64_t(N), uint64_t(K), uint64_t(ldw), uint32_t(bn), 64, 2);
  if (rc) return rc - 30;
  DenseEpilogue e{workspace, nullptr, nullptr, M, N, N, 0, 0, 0, 1};
  const int bf = dtype == 0;
#define RONN_DISPATCH(BN_, ST_)                                                                          \
  return bf ? launch_dense<BN_, ST_, __nv_bfloat16>(ma, mb, e, M, N, K, 1, status, stream, splitk)       \
            : launch_dense<BN_, ST_, __half>(ma, mb, e, M, N, K, 0, status, stream, splitk)
  switch (bn) {
    case 256: RONN_DISPATCH(256, 4);
    case 128: RONN_DISPATCH(128, 3);
    case 64: RONN_DISPATCH(64, 4);
    case 32: RONN_DISPATCH(32, 5);
    default: return -3;
  }
#undef RONN_DISPATCH
}
