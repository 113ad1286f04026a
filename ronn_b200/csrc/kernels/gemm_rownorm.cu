// GEMM whose epilogue also normalises whole rows:  x = A W^T + bias + residual ;  y = LayerNorm / RMSNorm(x).
//
// A row of x spans N / 128 output tiles, so the CTAs of one row block form a thread-block cluster along N: each CTA
// keeps its 128 x 128 accumulator in TMEM, writes its part of x, publishes per-row (sum, sum of squares) in its shared
// memory, and after a cluster barrier reads the other CTAs' statistics over distributed shared memory to normalise its
// own columns.  One launch replaces GEMM + norm kernel (attention output projection) or split-K GEMM + finalize pass
// (MLP down projection) of a decoder block; N <= 1024 (cluster of at most 8).
//
// The reference runs these as separate library calls with a host round trip in between
// (crates/ronn-providers/src/gpu/provider.rs:1135-1436; layer norm: crates/ronn-core/src/ops/neural_network.rs).
#include "common.cuh"
#include "ptx_sm100.cuh"
#include "tma_desc.cuh"

namespace ronn {

constexpr int RN_THREADS = 192;
constexpr int RN_BN = 128;
constexpr int RN_STAGES = 5;

struct RnSmem {
  static constexpr int A_BYTES = 128 * 128;
  static constexpr int B_BYTES = RN_BN * 128;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int TILE_BYTES = RN_STAGES * STAGE_BYTES;
  static constexpr int STATS_BYTES = 128 * 8;                       // float2 per row
  static constexpr int DYN_SMEM = TILE_BYTES + STATS_BYTES + (2 * RN_STAGES + 1) * 8 + 16 + 1024;
  static constexpr uint32_t TMEM_COLS = 128;
};

struct RowNormArgs {
  void* sum_out;           // [M, N] x = A W^T + bias + residual
  void* norm_out;          // [M, N] normalised x
  const void* bias;        // [N] or null
  const void* residual;    // [M, ld_res] or null
  const void* gamma;       // [N]
  const void* beta;        // [N] or null
  int M, N, K, ld_res;
  float eps;
  int mode;                // 1 LayerNorm, 2 RMSNorm
};

__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ float2 ld_cluster_f2(const void* local_smem, uint32_t cta_rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local_smem)), "r"(cta_rank));
  float2 v;
  asm volatile("ld.shared::cluster.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(remote) : "memory");
  return v;
}

// grid = (N / 128, row tiles), cluster = (N / 128, 1, 1): blockIdx.x is both the column tile and the rank in the cluster.
template <class T>
__global__ void __launch_bounds__(RN_THREADS)
gemm_rownorm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, RowNormArgs a,
                    uint32_t idesc, uint32_t* status) {
  using L = RnSmem;
  extern __shared__ uint8_t dyn_smem[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dyn_smem) + 1023) & ~uintptr_t(1023));
  float2* stats = reinterpret_cast<float2*>(tiles + L::TILE_BYTES);
  uint64_t* full = reinterpret_cast<uint64_t*>(tiles + L::TILE_BYTES + L::STATS_BYTES);
  uint64_t* empty = full + RN_STAGES;
  uint64_t* acc_full = empty + RN_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile uint32_t* abort = tmem_slot + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_ctas = gridDim.x;
  const int n0 = blockIdx.x * RN_BN, m0 = blockIdx.y * 128;
  const int num_kb = (a.K + 63) / 64;

  if (threadIdx.x == 0) {
    for (int s = 0; s < RN_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_full, 1);
    *abort = 0;
    mbar_fence_init();
    fence_proxy_async_smem();
  }
  __syncwarp();
  if (warp == 1) {
    tmem_alloc(tmem_slot, L::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      // weights never depend on the previous kernel: request the first stages before the dependency wait
      const int pre = num_kb < RN_STAGES ? num_kb : RN_STAGES;
      for (int kb = 0; kb < pre; ++kb) {
        mbar_expect_tx(&full[kb], L::STAGE_BYTES);
        tma_load_2d(tiles + kb * L::STAGE_BYTES + L::A_BYTES, &map_b, &full[kb], kb * 64, n0);
      }
      pdl_wait();
      pdl_trigger();
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % RN_STAGES;
        uint8_t* sa = tiles + s * L::STAGE_BYTES;
        if (kb < pre) {
          tma_load_2d(sa, &map_a, &full[s], kb * 64, m0);
          continue;
        }
        if (!mbar_wait(&empty[s], ((kb / RN_STAGES) & 1) ^ 1, abort, status, STATUS_WAIT_SLOT)) break;
        mbar_expect_tx(&full[s], L::STAGE_BYTES);
        tma_load_2d(sa, &map_a, &full[s], kb * 64, m0);
        tma_load_2d(sa + L::A_BYTES, &map_b, &full[s], kb * 64, n0);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = true;
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % RN_STAGES;
        if (!mbar_wait(&full[s], (kb / RN_STAGES) & 1, abort, status, STATUS_WAIT_TMA)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t sa = smem_u32(tiles + s * L::STAGE_BYTES);
        const uint64_t adesc = umma_desc_k128(sa), bdesc = umma_desc_k128(sa + L::A_BYTES);
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_f16(tmem_base, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0);
        umma_commit(&empty[s]);
      }
      if (ok) umma_commit(acc_full);
    }
    __syncwarp();
  }

  // ---------------------------------------------------------------- epilogue, phase A: x and the row statistics
  const int q = warp & 3;
  const int row = q * 32 + lane;
  const int gm = m0 + row;
  const bool epi = warp >= 2;
  const bool row_ok = epi && gm < a.M;
  T* xrow = reinterpret_cast<T*>(a.sum_out) + size_t(gm) * a.N + n0;
  bool ok = true;
  if (epi) {
    pdl_wait();
    ok = mbar_wait(acc_full, 0, abort, status, STATUS_WAIT_ACCUM);
    ok = __all_sync(0xffffffffu, ok);
    float s1 = 0.f, s2 = 0.f;
    if (ok) {
      tc_fence_after_sync();
      const T* bias = reinterpret_cast<const T*>(a.bias);
      const T* res = reinterpret_cast<const T*>(a.residual);
#pragma unroll 1
      for (int c = 0; c < RN_BN; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + (uint32_t(q * 32) << 16) + uint32_t(c), r);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[g * 8 + i]);
            const int col = n0 + c + g * 8;
            if (bias) {
              float f[8];
              unpack8<T>(*reinterpret_cast<const Vec8*>(bias + col), f);
#pragma unroll
              for (int i = 0; i < 8; ++i) v[i] += f[i];
            }
            if (res) {
              float f[8];
              unpack8<T>(*reinterpret_cast<const Vec8*>(res + size_t(gm) * a.ld_res + col), f);
#pragma unroll
              for (int i = 0; i < 8; ++i) v[i] += f[i];
            }
            const Vec8 pk = pack8<T>(v);
            *reinterpret_cast<Vec8*>(xrow + c + g * 8) = pk;
            unpack8<T>(pk, v);                       // the statistics are those of the stored (rounded) values
#pragma unroll
            for (int i = 0; i < 8; ++i) { s1 += v[i]; s2 += v[i] * v[i]; }
          }
        }
      }
    }
    stats[row] = make_float2(s1, s2);
  }
  // every thread of every CTA of the cluster takes part in the barrier; it also orders the stats writes (release)
  // before the remote reads below (acquire)
  __syncwarp();
  cluster_arrive();
  cluster_wait();
  // ---------------------------------------------------------------- phase B: normalise this CTA's columns
  if (epi && ok && row_ok && !*abort) {
    float S1 = 0.f, S2 = 0.f;
    for (int r = 0; r < n_ctas; ++r) {
      const float2 p = ld_cluster_f2(&stats[row], uint32_t(r));
      S1 += p.x;
      S2 += p.y;
    }
    const float inv_n = 1.f / float(a.N);
    float mean = 0.f, inv;
    if (a.mode == 2) {
      inv = rsqrtf(S2 * inv_n + a.eps);
    } else {
      mean = S1 * inv_n;
      inv = rsqrtf(fmaxf(S2 * inv_n - mean * mean, 0.f) + a.eps);
    }
    const T* gamma = reinterpret_cast<const T*>(a.gamma);
    const T* beta = reinterpret_cast<const T*>(a.beta);
    T* yrow = reinterpret_cast<T*>(a.norm_out) + size_t(gm) * a.N + n0;
#pragma unroll 1
    for (int c = 0; c < RN_BN; c += 8) {
      float v[8], g[8], o[8];
      unpack8<T>(*reinterpret_cast<const Vec8*>(xrow + c), v);      // written by this thread in phase A
      unpack8<T>(*reinterpret_cast<const Vec8*>(gamma + n0 + c), g);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = (v[i] - mean) * inv * g[i];
      if (beta) {
        float b[8];
        unpack8<T>(*reinterpret_cast<const Vec8*>(beta + n0 + c), b);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] += b[i];
      }
      *reinterpret_cast<Vec8*>(yrow + c) = pack8<T>(o);
    }
  }
  // no CTA may leave (and release its shared memory) while another one can still read its statistics
  __syncwarp();
  cluster_arrive();
  cluster_wait();
  if (*abort) {
    const long long t0 = clock64();
    while (clock64() - t0 < 400000ll) { __nanosleep(1000); }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, L::TMEM_COLS);
  }
}

template <class T>
static int launch_rownorm(const CUtensorMap& ma, const CUtensorMap& mb, const RowNormArgs& a, int is_bf16, uint32_t* status,
                          cudaStream_t stream) {
  auto kern = gemm_rownorm_kernel<T>;
  static bool configured[MAX_DEVICES] = {false};
  if (first_use_on_device(configured)) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, RnSmem::DYN_SMEM) != cudaSuccess) return -10;
  }
  const int n_tiles = a.N / RN_BN;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(n_tiles, (a.M + 127) / 128, 1);
  cfg.blockDim = dim3(RN_THREADS);
  cfg.dynamicSmemBytes = RnSmem::DYN_SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = n_tiles;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  prefer_max_shared(reinterpret_cast<const void*>(kern));
  const uint32_t idesc = umma_idesc(128, RN_BN, is_bf16 ? 1u : 0u, 1u);
  cudaError_t err = cudaLaunchKernelEx(&cfg, kern, ma, mb, a, idesc, status);
  return (err == cudaSuccess && cudaGetLastError() == cudaSuccess) ? 0 : -11;
}

}  // namespace ronn

using namespace ronn;

// x[M, N] = A[M, K] W[N, K]^T + bias + residual (written to sum_out) and y = norm(x) (written to norm_out).
// N a multiple of 128, N <= 1024; K, lda, ldw, ld_res multiples of 8.  mode 1 LayerNorm (gamma, beta), 2 RMSNorm
// (gamma).  dtype 0 bf16, 1 fp16.  sum_out must not alias residual.  Returns 0 on success.
extern "C" int ronn_gemm_rownorm(const void* A, const void* W, void* sum_out, void* norm_out, const void* bias,
                                 const void* residual, const void* gamma, const void* beta, int M, int N, int K, int lda,
                                 int ldw, int ld_res, float eps, int mode, int dtype, uint32_t* status,
                                 cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return -1;
  if ((N % RN_BN) || N > 8 * RN_BN || (K & 7) || (lda & 7) || (ldw & 7) || (residual && (ld_res & 7))) return -2;
  if (mode != 1 && mode != 2) return -3;
  if (gamma == nullptr || sum_out == nullptr || norm_out == nullptr) return -4;
  CUtensorMap ma, mb;
  int rc = make_tmap_2d(&ma, A, uint64_t(M), uint64_t(K), uint64_t(lda), 128, 64, 2);
  if (rc) return rc - 20;
  rc = make_tmap_2d(&mb, W, uint64_t(N), uint64_t(K), uint64_t(ldw), RN_BN, 64, 2);
  if (rc) return rc - 30;
  RowNormArgs a{sum_out, norm_out, bias, residual, gamma, beta, M, N, K, ld_res, eps, mode};
  return dtype == 0 ? launch_rownorm<__nv_bfloat16>(ma, mb, a, 1, status, stream)
                    : launch_rownorm<__half>(ma, mb, a, 0, status, stream);
}
