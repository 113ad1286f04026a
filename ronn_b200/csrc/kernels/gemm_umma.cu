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
#include <stdlib.h>

#include "common.cuh"
#include "gemm_epilogue.cuh"
#include "tma_desc.cuh"
#include "umma_persistent.cuh"

namespace ronn {

// Tile list of a dense (optionally split-K) GEMM for the persistent mainloop.  Tiles are numbered with the
// M index fastest so that CTAs running side by side share the same weight tile in L2.
template <int BN, class T>
struct DenseProblem {
  static constexpr bool kForceStage = false;
  const CUtensorMap* map_a;
  const CUtensorMap* map_b;
  DenseEpilogue e;
  int m_tiles, n_tiles, num_kb, splitk, kb_per;

  __device__ __forceinline__ int num_tiles() const { return m_tiles * n_tiles * splitk; }
  __device__ __forceinline__ void tile(int t, int& m0, int& n0, int& kb0, int& nkb) const {
    const int per_z = m_tiles * n_tiles;
    const int z = t / per_z, r = t - z * per_z;
    m0 = (r % m_tiles) * PG_BM;
    n0 = (r / m_tiles) * BN;
    kb0 = z * kb_per;
    nkb = min(kb_per, num_kb - kb0);
  }
  __device__ __forceinline__ void load_a(uint8_t* smem, uint64_t* bar, int k_elem, int m0) const {
    tma_load_2d(smem, map_a, bar, k_elem, m0);
  }
  __device__ __forceinline__ void load_b(uint8_t* smem, uint64_t* bar, int k_elem, int n0) const {
    tma_load_2d(smem, map_b, bar, k_elem, n0);
  }
  __device__ __forceinline__ void epilogue(int t, int m0, int n0, int row, int col, uint32_t (&r)[32], uint8_t* stage) const {
    DenseEpilogue ep = e;
    ep.m0 = m0;
    ep.n0 = n0;
    if (splitk > 1)     // raw fp32 partial sums go to slice z of the workspace
      ep.C = reinterpret_cast<float*>(e.C) + size_t(t / (m_tiles * n_tiles)) * size_t(e.M) * size_t(e.ldc);
    ep.run<T>(row, col, r, stage);
  }
};

template <int BN, int STAGES, class T, int KA>
__global__ void __launch_bounds__(PG_THREADS)
gemm_dense_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                  DenseEpilogue epi, int K, int splitk, uint32_t idesc, uint32_t* status) {
  extern __shared__ uint8_t dyn_smem[];
  DenseProblem<BN, T> prob;
  prob.map_a = &map_a;
  prob.map_b = &map_b;
  prob.e = epi;
  prob.m_tiles = (epi.M + PG_BM - 1) / PG_BM;
  prob.n_tiles = (epi.N + BN - 1) / BN;
  prob.num_kb = (K + 63) / 64;
  prob.splitk = splitk;
  prob.kb_per = (prob.num_kb + splitk - 1) / splitk;
  gemm_persistent<BN, STAGES, 0, DenseProblem<BN, T>, KA>(dyn_smem, prob, 64, idesc, status);
}

static int sm_count() { return device_sm_count(); }

template <int BN, int STAGES, class T, int KA = 1>
static int launch_dense(const CUtensorMap& ma, const CUtensorMap& mb, DenseEpilogue epi, int M, int N, int K,
                        int is_bf16, uint32_t* status, cudaStream_t stream, int splitk = 1) {
  using L = PGemmSmem<BN, STAGES, false, KA>;
  auto kern = gemm_dense_kernel<BN, STAGES, T, KA>;
  static bool configured[MAX_DEVICES] = {false};
  if (first_use_on_device(configured)) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYN_SMEM) != cudaSuccess) return -10;
  }
  const int tiles = ((N + BN - 1) / BN) * ((M + PG_BM - 1) / PG_BM) * splitk;
  const int resident = sm_count() * (L::DYN_SMEM <= 112 * 1024 && L::TMEM_COLS <= 256 ? 2 : 1);
  dim3 grid(tiles < resident ? tiles : resident);
  uint32_t idesc = umma_idesc(PG_BM, BN, is_bf16 ? 1u : 0u, 1u);
  cudaError_t err = launch(kern, grid, dim3(PG_THREADS), size_t(L::DYN_SMEM), stream, ma, mb, epi, K, splitk, idesc, status);
  return (err == cudaSuccess && cudaGetLastError() == cudaSuccess) ? 0 : -11;
}

int pick_bn(int M, int N) {
  const int mt = (M + PG_BM - 1) / PG_BM;
  // 256-wide tiles pay off once the problem is compute bound; with one or two row tiles every CTA is a latency
  // chain and narrower tiles spread the weight stream over more SMs (measured: M 256, N 50264, K 1024 takes 36 us
  // with 128-wide tiles against 110 us with 256-wide ones)
  const int cands[4] = {256, 128, 64, 32};
  for (int i = (mt <= 2 ? 1 : 0); i < 4; ++i) {
    int bn = cands[i];
    if (bn > 32 && N < bn) continue;
    int ctas = mt * ((N + bn - 1) / bn);
    if (ctas >= 120) return bn;
  }
  return 32;
}

// Pipeline depth.  A CTA that is alone on its SM is fed by the bytes it keeps in flight, so when the whole problem
// is at most one CTA per SM the ring is twice as deep (6 / 8 / 10 stages for BN 128 / 64 / 32, one CTA per SM)
// instead of two co-resident CTAs with half the ring each.  bn | 0x1000 forces the deep ring, bn | 0x2000 the shallow.
static int deep_mode(int bn) { return (bn & 0x1000) ? 1 : ((bn & 0x2000) ? 0 : -1); }
static int wants_deep(int M, int N, int bn, int splitk) {
  static int forced = -2;                                  // RONN_GEMM_RING = deep | shallow overrides the choice
  if (forced == -2) {
    const char* e = getenv("RONN_GEMM_RING");
    forced = !e ? -1 : (e[0] == 'd' ? 1 : (e[0] == 's' ? 0 : -1));
  }
  if (forced >= 0) return forced;
  const int tiles = ((N + bn - 1) / bn) * ((M + PG_BM - 1) / PG_BM) * splitk;
  return tiles <= sm_count() ? 1 : 0;
}

}  // namespace ronn

using namespace ronn;

// dtype: 0 = bf16, 1 = fp16.  act: 0 none, 1 relu, 2 gelu.  bn: 0 = auto, else 32|64|128|256 (| 0x1000 deep ring,
// | 0x2000 shallow ring; default picks by tile count).
// lda/ldw/ldc in elements; K and the leading dimensions must be multiples of 8.
// Returns 0 on success, negative on configuration errors.
extern "C" int ronn_gemm(const void* A, const void* W, void* C, const void* bias, const void* residual, int M, int N,
                         int K, int lda, int ldw, int ldc, int dtype, int act, int out_fp32, int bn,
                         uint32_t* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return -1;
  if ((K & 7) || (lda & 7) || (ldw & 7)) return -2;
  int deep = deep_mode(bn);
  bn &= 0xfff;
  if (bn == 0) bn = pick_bn(M, N);
  if (deep < 0) deep = wants_deep(M, N, bn, 1);
  CUtensorMap ma, mb;
  int rc = make_tmap_2d(&ma, A, uint64_t(M), uint64_t(K), uint64_t(lda), PG_BM, 64, 2);
  if (rc) return rc - 20;
  rc = make_tmap_2d(&mb, W, uint64_t(N), uint64_t(K), uint64_t(ldw), uint32_t(bn), 64, 2);
  if (rc) return rc - 30;
  DenseEpilogue e{C, bias, residual, M, N, ldc, 0, 0, act, out_fp32};
  const int bf = dtype == 0;
#define RONN_DISPATCH(BN_, ST_, KA_)                                                                  \
  return bf ? launch_dense<BN_, ST_, __nv_bfloat16, KA_>(ma, mb, e, M, N, K, 1, status, stream)       \
            : launch_dense<BN_, ST_, __half, KA_>(ma, mb, e, M, N, K, 0, status, stream)
  switch (deep ? -bn : bn) {
    case 256: case -256: RONN_DISPATCH(256, 4, 1);
    case 128: RONN_DISPATCH(128, 3, 1);
    case 64: RONN_DISPATCH(64, 4, 1);
    case 32: RONN_DISPATCH(32, 5, 1);
    case -128: RONN_DISPATCH(128, 3, 2);       // deep ring, one CTA per SM: two K atoms per stage
    case -64: RONN_DISPATCH(64, 4, 2);
    case -32: RONN_DISPATCH(32, 5, 2);
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
  int deep = deep_mode(bn);
  bn &= 0xfff;
  if (bn == 0) bn = N >= 128 ? 128 : (N >= 64 ? 64 : 32);
  if (deep < 0) deep = wants_deep(M, N, bn, splitk);
  CUtensorMap ma, mb;
  int rc = make_tmap_2d(&ma, A, uint64_t(M), uint64_t(K), uint64_t(lda), PG_BM, 64, 2);
  if (rc) return rc - 20;
  rc = make_tmap_2d(&mb, W, uint64_t(N), uint64_t(K), uint64_t(ldw), uint32_t(bn), 64, 2);
  if (rc) return rc - 30;
  DenseEpilogue e{workspace, nullptr, nullptr, M, N, N, 0, 0, 0, 1};
  const int bf = dtype == 0;
#define RONN_DISPATCH(BN_, ST_, KA_)                                                                     \
  return bf ? launch_dense<BN_, ST_, __nv_bfloat16, KA_>(ma, mb, e, M, N, K, 1, status, stream, splitk)  \
            : launch_dense<BN_, ST_, __half, KA_>(ma, mb, e, M, N, K, 0, status, stream, splitk)
  switch (deep ? -bn : bn) {
    case 256: case -256: RONN_DISPATCH(256, 4, 1);
    case 128: RONN_DISPATCH(128, 3, 1);
    case 64: RONN_DISPATCH(64, 4, 1);
    case 32: RONN_DISPATCH(32, 5, 1);
    case -128: RONN_DISPATCH(128, 3, 2);       // deep ring, one CTA per SM: two K atoms per stage
    case -64: RONN_DISPATCH(64, 4, 2);
    case -32: RONN_DISPATCH(32, 5, 2);
    default: return -3;
  }
#undef RONN_DISPATCH
}
