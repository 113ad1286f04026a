// Fused Conv + (folded BatchNorm) + residual + ReLU as an implicit GEMM on tcgen05 tensor cores.
//
//   out[n, oh, ow, co] = act( sum_{r,s,c} x[n, oh*st - pad + r*dil, ow*st - pad + s*dil, c] * w[co, r, s, c]
//                             + bias[co] ) (+ residual[n, oh, ow, co] before the activation)
//
// NHWC activations, weights [Cout, R, S, Cin] (so a weight row is one K-major GEMM row of length R*S*Cin
// and is fetched by TMA with the 128-byte swizzle).  The A operand (128 output pixels x 64 K-elements per
// stage) never exists in memory: four producer warps gather it with 16-byte cp.async (zero-fill for padding
// and the K tail) directly into the swizzled shared-memory layout the UMMA descriptor expects
// (chunk j of row m lands at chunk position j ^ (m & 7)).  Accumulation in TMEM, epilogue shared with the GEMM.
//
// Roles: warps 0-3 gather A; warp 4 lane 0 issues the weight TMA; warp 5 allocates TMEM and issues the MMAs;
// warps 6-9 run the epilogue.  The kernel is persistent with a double-buffered accumulator.
//
// Replaces the reference's depthwise one-thread-per-output template (crates/ronn-providers/src/gpu/cuda_kernels.rs:400-449)
// and its Candle conv2d call with fixed stride 1 / pad 1 (crates/ronn-providers/src/gpu/provider.rs:1292-1305); the BN
// folding itself is done by the fusion pass.  Cin % 8 == 0 (the provider pads a 3-channel stem to 8).
#include "gemm_epilogue.cuh"
#include "ptx_sm100.cuh"
#include "tma_desc.cuh"

namespace ronn {

constexpr int CONV_THREADS = 320;    // warps 0-3 gather A, 4 weight TMA, 5 MMA issuer, 6-9 epilogue
// Ring depth and cp.async look-ahead.  A gather warp signals K block i only once block i + LAG has been issued, so the
// MMA warp is STAGES - LAG blocks of slack behind the gather.  Measured on ResNet-18 shapes, two co-resident CTAs with
// four stages each beat one CTA with an eight-stage ring.
template <int BN> struct ConvPipe {
  static constexpr int STAGES = BN >= 128 ? 6 : 4;       // 128-wide tiles: one CTA per SM; narrower: two (96 KB each)
  static constexpr int LAG = 3;
};

struct ConvShape {
  int N, H, W, C;          // input
  int Ho, Wo, Cout;
  int R, S, stride, pad, dil;
  int M;                   // N * Ho * Wo
  int chunks;              // R * S * C / 8   (16-byte K chunks)
  int splitk;              // K slices per output tile (> 1: fp32 partial panels, reduced by the finalize kernel)
  int kb_per;              // K blocks per slice
};

// tile index -> (row tile, column tile, first K block, K blocks); K slices of one output tile are adjacent indices
struct ConvTile {
  int mt, nt, ks, kb0, nkb;
  __device__ __forceinline__ ConvTile(int t, int n_tiles, int num_kb, const ConvShape& cs) {
    ks = t % cs.splitk;
    const int rest = t / cs.splitk;
    nt = rest % n_tiles;
    mt = rest / n_tiles;
    kb0 = ks * cs.kb_per;
    nkb = min(cs.kb_per, num_kb - kb0);
  }
};

template <int BN>
struct ConvSmem {
  static constexpr int A_BYTES = 128 * 128;
  static constexpr int B_BYTES = BN * 128;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = ConvPipe<BN>::STAGES;
  static constexpr int LAG = ConvPipe<BN>::LAG;
  static constexpr int TILE_BYTES = STAGES * STAGE_BYTES;
  static constexpr int DYN_SMEM = TILE_BYTES + (2 * STAGES + 4) * 8 + 16 + 1024;
  static constexpr uint32_t TMEM_COLS = 2 * BN <= 64 ? 64u : (2 * BN <= 128 ? 128u : (2 * BN <= 256 ? 256u : 512u));
};

// Persistent: a CTA walks output tiles (tile = blockIdx.x, += gridDim.x); the smem ring and its barrier phases run
// across tiles and the accumulator is double-buffered in TMEM, so the gather of tile j+1 overlaps the epilogue of j.
template <int BN, class T, bool FAST>
__global__ void __launch_bounds__(CONV_THREADS)
conv_igemm_kernel(const T* __restrict__ x, const __grid_constant__ CUtensorMap map_w, ConvShape cs, DenseEpilogue epi,
                  uint32_t idesc, uint32_t* status) {
  using L = ConvSmem<BN>;
  extern __shared__ uint8_t dyn_smem[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dyn_smem) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(tiles + L::TILE_BYTES);
  uint64_t* empty = full + L::STAGES;
  uint64_t* acc_full = empty + L::STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile uint32_t* abort = tmem_slot + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = (cs.chunks + 7) / 8;
  const int n_tiles = (cs.Cout + BN - 1) / BN;
  const int ntiles = ((cs.M + 127) / 128) * n_tiles * cs.splitk;

  if (threadIdx.x == 0) {
    for (int s = 0; s < L::STAGES; ++s) {
      mbar_init(&full[s], 4 + 1);            // one arrival per gather warp + the weight TMA's expect_tx arrival
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);
    }
    *abort = 0;
    mbar_fence_init();
    fence_proxy_async_smem();
  }
  __syncwarp();
  if (warp == 5) {
    tmem_alloc(tmem_slot, L::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < 4) {
    // ---------------------------------------------------------------- A gather
    // Thread t owns 16-byte chunk (t & 7) of rows (t >> 3) + 16 i, i = 0..7: the 8 lanes of a row fetch one contiguous
    // 128-byte run of the input (a whole cache line when C % 64 == 0), so a warp instruction touches 4 lines, not 32.
    // Barrier traffic is per warp: lane 0 waits for the slot and arrives for the warp.
    pdl_wait();
    pdl_trigger();                               // successor may launch and set up under this kernel
    const int chunk = threadIdx.x & 7;
    const int rbase = threadIdx.x >> 3;
    uint32_t it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < ntiles; t += gridDim.x) {
      const ConvTile tl(t, n_tiles, num_kb, cs);
      int ih0[8], iw0[8], boff[8];               // per row: top-left input coordinate and image offset (elements)
      uint32_t okmask = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int m = tl.mt * 128 + rbase + 16 * i;
        int n_img = 0, oh = 0, ow = 0;
        if (m < cs.M) {
          okmask |= 1u << i;
          n_img = m / (cs.Ho * cs.Wo);
          const int rem = m - n_img * cs.Ho * cs.Wo;
          oh = rem / cs.Wo;
          ow = rem - oh * cs.Wo;
        }
        ih0[i] = oh * cs.stride - cs.pad;
        iw0[i] = ow * cs.stride - cs.pad;
        boff[i] = n_img * cs.H * cs.W * cs.C;
      }
      // filter tap (r, sx) and channel offset of this thread's chunk in the current K block, advanced incrementally
      int r, sx, cpos;
      {
        const int e = (tl.kb0 * 8 + chunk) * 8;          // first K element of this thread's chunk in this slice
        const int tap = e / cs.C;
        cpos = e - tap * cs.C;
        r = tap / cs.S;
        sx = tap - r * cs.S;
      }
      for (int kb = 0; kb < tl.nkb; ++kb, ++it) {
        const int s = it % L::STAGES;
        if (lane == 0 && ok && !mbar_wait(&empty[s], ((it / L::STAGES) & 1) ^ 1, abort, status, STATUS_WAIT_SLOT))
          ok = false;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (ok) {
          uint8_t* dst = tiles + s * L::STAGE_BYTES;
          const bool tap_ok = FAST || r < cs.R;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int row = rbase + 16 * i;
            const int ih = ih0[i] + r * cs.dil, iw = iw0[i] + sx * cs.dil;
            const bool valid = tap_ok && ((okmask >> i) & 1u) && unsigned(ih) < unsigned(cs.H) &&
                               unsigned(iw) < unsigned(cs.W);
            const T* src = valid ? x + (boff[i] + (ih * cs.W + iw) * cs.C + cpos) : x;
            cp_async_16(dst + row * 128 + ((uint32_t(chunk) ^ uint32_t(row & 7)) << 4), src, valid);
          }
          // next K block: 64 channels further along (tap-major, channel-minor) order
          cpos += 64;
          if (FAST) {
            if (cpos >= cs.C) {
              cpos -= cs.C;
              if (++sx == cs.S) { sx = 0; ++r; }
            }
          } else {
            while (cpos >= cs.C) {
              cpos -= cs.C;
              if (++sx == cs.S) { sx = 0; ++r; }
            }
          }
        }
        cp_async_commit();
        if (it >= L::LAG) {
          cp_async_wait<L::LAG>();
          __syncwarp();
          if (lane == 0) mbar_arrive(&full[(it - L::LAG) % L::STAGES]);
        }
      }
    }
    cp_async_wait<0>();
    __syncwarp();
    if (lane == 0)
      for (uint32_t k = (it > L::LAG ? it - L::LAG : 0); k < it; ++k) mbar_arrive(&full[k % L::STAGES]);
    pdl_trigger();
  } else if (warp == 4) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < ntiles && ok; t += gridDim.x) {
        const ConvTile tl(t, n_tiles, num_kb, cs);
        const int n0 = tl.nt * BN;
        for (int kb = 0; kb < tl.nkb; ++kb, ++it) {
          const int s = it % L::STAGES;
          if (!mbar_wait(&empty[s], ((it / L::STAGES) & 1) ^ 1, abort, status, STATUS_WAIT_SLOT)) { ok = false; break; }
          mbar_expect_tx(&full[s], L::B_BYTES);
          tma_load_2d(tiles + s * L::STAGE_BYTES + L::A_BYTES, &map_w, &full[s], (tl.kb0 + kb) * 64, n0);
        }
      }
    }
    __syncwarp();
    pdl_trigger();
  } else if (warp == 5) {
    if (lane == 0) {
      uint32_t it = 0, j = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < ntiles && ok; t += gridDim.x, ++j) {
        const uint32_t buf = j & 1;
        if (!mbar_wait(&acc_empty[buf], ((j >> 1) & 1) ^ 1, abort, status, STATUS_WAIT_EPI)) break;
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + buf * BN;
        const ConvTile tl(t, n_tiles, num_kb, cs);
        for (int kb = 0; kb < tl.nkb; ++kb, ++it) {
          const int s = it % L::STAGES;
          if (!mbar_wait(&full[s], (it / L::STAGES) & 1, abort, status, STATUS_WAIT_TMA)) { ok = false; break; }
          // the gather warps wrote this stage through the generic proxy and released it with their barrier arrival;
          // one proxy fence here, after the acquire, orders those writes before the tensor core's reads
          fence_proxy_async_smem();
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(tiles + s * L::STAGE_BYTES);
          const uint64_t adesc = umma_desc_k128(sa), bdesc = umma_desc_k128(sa + L::A_BYTES);
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_f16(tmem_d, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0);
          umma_commit(&empty[s]);
        }
        if (ok) umma_commit(&acc_full[buf]);
      }
    }
    __syncwarp();
    pdl_trigger();
  } else {
    // ---------------------------------------------------------------- epilogue (warps 6-9 own TMEM lane quarters 2,3,0,1)
    const int q = warp & 3;
    pdl_wait();
    void* const c_base = epi.C;
    uint32_t j = 0;
    for (int t = blockIdx.x; t < ntiles; t += gridDim.x, ++j) {
      const uint32_t buf = j & 1;
      if (!mbar_wait_warp_relaxed(&acc_full[buf], (j >> 1) & 1, abort, status, STATUS_WAIT_ACCUM)) break;
      tc_fence_after_sync();
      const ConvTile tl(t, n_tiles, num_kb, cs);
      epi.m0 = tl.mt * 128;
      epi.n0 = tl.nt * BN;
      if (cs.splitk > 1) epi.C = reinterpret_cast<float*>(c_base) + size_t(tl.ks) * cs.M * cs.Cout;
      const int row = q * 32 + lane;
      const uint32_t tacc = tmem_base + (uint32_t(q * 32) << 16) + buf * BN;
      // the TMEM load of the next 32 columns is in flight while this chunk is converted and stored
      if (BN == 32) {
        uint32_t r0[32];
        tmem_ld_32x32(tacc, r0);
        tmem_ld_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[buf]);
        epi.run<T>(row, 0, r0);
      } else {
        uint32_t r0[32], r1[32];
        tmem_ld_32x32(tacc, r0);
#pragma unroll 1
        for (int col = 0; col < BN; col += 64) {
          tmem_ld_wait();
          tmem_ld_32x32(tacc + uint32_t(col + 32), r1);
          epi.run<T>(row, col, r0);
          tmem_ld_wait();
          if (col + 64 < BN) {
            tmem_ld_32x32(tacc + uint32_t(col + 64), r0);
          } else {
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
          }
          epi.run<T>(row, col + 32, r1);
        }
      }
    }
    pdl_trigger();
  }
  if (*abort) {
    const long long t0 = clock64();
    while (clock64() - t0 < 400000ll) { __nanosleep(1000); }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, L::TMEM_COLS);
  }
}

template <int BN, class T, bool FAST>
static int launch_conv_impl(const void* x, const CUtensorMap& mw, const ConvShape& cs, const DenseEpilogue& e, int is_bf16,
                            uint32_t* status, cudaStream_t stream) {
  using L = ConvSmem<BN>;
  auto kern = conv_igemm_kernel<BN, T, FAST>;
  static bool configured[MAX_DEVICES] = {false};
  if (first_use_on_device(configured)) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYN_SMEM) != cudaSuccess) return -10;
  }
  const int sms = device_sm_count();
  // two CTAs per SM when shared memory (227 KB) and TMEM (512 columns) allow it
  const int per_sm = (L::DYN_SMEM <= 110 * 1024 && L::TMEM_COLS <= 256) ? 2 : 1;
  const int resident = sms * per_sm;
  const int tiles = ((cs.M + 127) / 128) * ((cs.Cout + BN - 1) / BN) * cs.splitk;
  dim3 grid(tiles < resident ? tiles : resident);
  const uint32_t idesc = umma_idesc(128, BN, is_bf16 ? 1u : 0u, 1u);
  cudaError_t err = launch(kern, grid, dim3(CONV_THREADS), size_t(L::DYN_SMEM), stream, (const T*)x, mw, cs, e, idesc, status);
  return (err == cudaSuccess && cudaGetLastError() == cudaSuccess) ? 0 : -11;
}

template <int BN, class T>
static int launch_conv(const void* x, const CUtensorMap& mw, const ConvShape& cs, const DenseEpilogue& e, int is_bf16,
                       uint32_t* status, cudaStream_t stream) {
  if ((cs.C & 63) == 0) return launch_conv_impl<BN, T, true>(x, mw, cs, e, is_bf16, status, stream);
  return launch_conv_impl<BN, T, false>(x, mw, cs, e, is_bf16, status, stream);
}

// ---------------------------------------------------------------------------------------------------- pooling (NHWC)
template <class T>
__global__ void maxpool_nhwc_kernel(const T* __restrict__ x, T* __restrict__ y, int N, int H, int W, int C, int Ho, int Wo,
                                    int k, int stride, int pad) {
  pdl_wait();
  pdl_trigger();
  const int c8n = C >> 3;
  const long total = long(N) * Ho * Wo * c8n;
  for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < total; i += long(gridDim.x) * blockDim.x) {
    const int c8 = int(i % c8n);
    long p = i / c8n;
    const int ow = int(p % Wo);
    p /= Wo;
    const int oh = int(p % Ho), n = int(p / Ho);
    float best[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) best[j] = -INFINITY;
    if (k == 3) {
      // the common window: all nine loads are issued before the first comparison (out-of-range taps re-read the
      // centre, which is always inside, and are ignored)
      Vec8 v[9];
      bool in[9];
      const T* centre = x + ((size_t(n) * H + min(oh * stride - pad + 1, H - 1)) * W + min(ow * stride - pad + 1, W - 1)) * C + c8 * 8;
#pragma unroll
      for (int t = 0; t < 9; ++t) {
        const int ih = oh * stride - pad + t / 3, iw = ow * stride - pad + t % 3;
        in[t] = ih >= 0 && ih < H && iw >= 0 && iw < W;
        const T* src = in[t] ? x + ((size_t(n) * H + ih) * W + iw) * C + c8 * 8 : centre;
        v[t] = *reinterpret_cast<const Vec8*>(src);
      }
#pragma unroll
      for (int t = 0; t < 9; ++t) {
        float f[8];
        unpack8<T>(v[t], f);
        if (in[t]) {
#pragma unroll
          for (int j = 0; j < 8; ++j) best[j] = fmaxf(best[j], f[j]);
        }
      }
    } else {
      for (int r = 0; r < k; ++r) {
        const int ih = oh * stride - pad + r;
        if (ih < 0 || ih >= H) continue;
        for (int s2 = 0; s2 < k; ++s2) {
          const int iw = ow * stride - pad + s2;
          if (iw < 0 || iw >= W) continue;
          float f[8];
          unpack8<T>(*reinterpret_cast<const Vec8*>(x + ((size_t(n) * H + ih) * W + iw) * C + c8 * 8), f);
#pragma unroll
          for (int j = 0; j < 8; ++j) best[j] = fmaxf(best[j], f[j]);
        }
      }
    }
    *reinterpret_cast<Vec8*>(y + ((size_t(n) * Ho + oh) * Wo + ow) * C + c8 * 8) = pack8<T>(best);
  }
}

// NCHW [N, C, H, W] with C <= 8 -> NHWC [N, H, W, 8], missing channels zero: the input conversion of an image network's
// first convolution (which needs its channel count padded to 8) in one pass.  One pixel per thread.
template <class T>
__global__ void nchw_to_nhwc8_kernel(const T* __restrict__ x, T* __restrict__ y, int C, long HW, long total) {
  pdl_wait();
  pdl_trigger();
  for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < total; i += long(gridDim.x) * blockDim.x) {
    const long n = i / HW, p = i - n * HW;
    alignas(16) T v[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) v[c] = c < C ? x[(n * C + c) * HW + p] : Cvt<T>::from_f(0.f);
    *reinterpret_cast<Vec8*>(y + i * 8) = *reinterpret_cast<const Vec8*>(v);
  }
}

// NCHW [N, C, H, W] (C <= 4, H and W even) -> 2x2 space-to-depth NHWC [N, H/2, W/2, 16]: channel (dy * 2 + dx) * C + c
// holds x[n, c, 2 y + dy, 2 x + dx], the rest is zero.  A 7x7 stride-2 convolution over x becomes a 4x4 stride-1
// convolution over this tensor whose K rows are whole 128-byte runs (4 taps x 16 channels).  One output pixel per thread.
template <class T>
__global__ void nchw_to_s2d16_kernel(const T* __restrict__ x, T* __restrict__ y, int C, int H, int W, long total) {
  pdl_wait();
  pdl_trigger();
  const int H2 = H >> 1, W2 = W >> 1;
  for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < total; i += long(gridDim.x) * blockDim.x) {
    const int xo = int(i % W2);
    const long t = i / W2;
    const int yo = int(t % H2);
    const long n = t / H2;
    alignas(16) T v[16];
#pragma unroll
    for (int k = 0; k < 16; ++k) v[k] = Cvt<T>::from_f(0.f);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int dy = q >> 1, dx = q & 1;
      for (int c = 0; c < C; ++c)
        v[q * C + c] = x[((n * C + c) * H + (2 * yo + dy)) * long(W) + 2 * xo + dx];
    }
    Vec8* dst = reinterpret_cast<Vec8*>(y + i * 16);
    dst[0] = *reinterpret_cast<const Vec8*>(v);
    dst[1] = *reinterpret_cast<const Vec8*>(v + 8);
  }
}

// y[n, c] = mean over HW of x[n, :, :, c]; one CTA per (n, 64-channel slab), threads split HW.
template <class T>
__global__ void global_avgpool_nhwc_kernel(const T* __restrict__ x, T* __restrict__ y, int HW, int C) {
  __shared__ float part[8][64];
  pdl_wait();
  pdl_trigger();
  const int n = blockIdx.x, c0 = blockIdx.y * 64;
  const int cg = threadIdx.x & 7, pg = threadIdx.x >> 3;            // 8 channel groups x 8 pixel groups (64 threads)
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  if (c0 + cg * 8 < C) {
#pragma unroll 4
    for (int p = pg; p < HW; p += 8) {
      float f[8];
      unpack8<T>(*reinterpret_cast<const Vec8*>(x + (size_t(n) * HW + p) * C + c0 + cg * 8), f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += f[j];
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) part[pg][cg * 8 + j] = acc[j];
  __syncthreads();
  if (threadIdx.x < 64 && c0 + threadIdx.x < C) {
    float s = 0.f;
#pragma unroll
    for (int g = 0; g < 8; ++g) s += part[g][threadIdx.x];
    y[size_t(n) * C + c0 + threadIdx.x] = Cvt<T>::from_f(s / float(HW));
  }
}

// The same for wide feature maps: one CTA of 256 threads per (n, 512-channel slab), 64 channel groups x 4 pixel groups,
// so a CTA streams HW x 1 KB instead of HW x 128 bytes (with one small CTA per 64 channels the kernel was bound by
// the CTA launch rate: 0.49 of the copy bandwidth at 8192 x 7 x 7 x 512).
template <class T>
__global__ void __launch_bounds__(256)
global_avgpool_wide_kernel(const T* __restrict__ x, T* __restrict__ y, int HW, int C) {
  __shared__ float part[4][512];
  pdl_wait();
  pdl_trigger();
  const int n = blockIdx.x, c0 = blockIdx.y * 512;
  const int cg = threadIdx.x & 63, pg = threadIdx.x >> 6;
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  const bool live = c0 + cg * 8 < C;
  if (live) {
    const T* base = x + size_t(n) * HW * C + c0 + cg * 8;
    int p = pg;
    for (; p + 12 < HW; p += 16) {                       // four loads in flight per thread
      Vec8 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = *reinterpret_cast<const Vec8*>(base + size_t(p + 4 * u) * C);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        float f[8];
        unpack8<T>(v[u], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += f[j];
      }
    }
    for (; p < HW; p += 4) {
      float f[8];
      unpack8<T>(*reinterpret_cast<const Vec8*>(base + size_t(p) * C), f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += f[j];
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) part[pg][cg * 8 + j] = acc[j];
  __syncthreads();
  for (int c = threadIdx.x; c < 512; c += 256)
    if (c0 + c < C)
      y[size_t(n) * C + c0 + c] = Cvt<T>::from_f((part[0][c] + part[1][c] + part[2][c] + part[3][c]) / float(HW));
}

}  // namespace ronn

using namespace ronn;

// x: NHWC [N,H,W,C]; w: [Cout, R, S, C] contiguous; bias [Cout] or null; residual NHWC like the output or null.
// act: 0 none, 1 relu.  dtype: 0 bf16, 1 fp16.  C % 8 == 0, Cout % 8 == 0.
extern "C" int ronn_splitk_finalize(const float* ws, int S, const void* bias, const void* residual, void* sum_out,
                                    const void* gamma, const void* beta, void* y, long rows, int N, float eps,
                                    int act, int norm, int dtype, cudaStream_t stream);

// x: NHWC [N, H, W, C]; w: [Cout, R, S, C] (K-major rows of R*S*C); out: NHWC [N, Ho, Wo, Cout];
// out = act(conv(x, w) + bias + residual).  act 0 none, 1 ReLU.  C and Cout multiples of 8.  dtype 0 bf16, 1 fp16.
// workspace (may be null): fp32 scratch of workspace_floats elements.  Layers whose output tiles cannot fill the GPU
// but whose K loop is long (the deep 3x3 layers) run as K slices into fp32 panels there and are reduced, with
// bias / residual / ReLU, by the split-K finalize kernel.
extern "C" int ronn_conv2d(const void* x, const void* w, const void* bias, const void* residual, void* out, int N, int H,
                           int W, int C, int Cout, int R, int S, int stride, int pad, int dil, int Ho, int Wo, int act,
                           int dtype, float* workspace, long workspace_floats, uint32_t* status, cudaStream_t stream) {
  if (N <= 0 || (C & 7) || (Cout & 7) || R <= 0 || S <= 0 || stride <= 0) return -2;
  if (long(H) * W * C * N >= (1l << 31) || long(N) * Ho * Wo * Cout >= (1l << 31)) return -4;   // 32-bit offsets inside
  ConvShape cs{N, H, W, C, Ho, Wo, Cout, R, S, stride, pad, dil, N * Ho * Wo, R * S * C / 8, 1, 0};
  const int Kg = R * S * C;
  const int num_kb = (cs.chunks + 7) / 8;
  const int m_tiles = (cs.M + 127) / 128;
  // Tile width: as wide as the layer allows (a 32-wide MMA costs as much issue time as a 128-wide one).  Parallelism
  // for layers with few output tiles comes from K slices instead, chosen by a small cost model in units of one K
  // block: waves x (K blocks per slice + fixed cost per tile) + the reduction pass.
  int bn = Cout >= 128 ? 128 : (Cout >= 64 ? 64 : 32);
  int tiles = m_tiles * ((Cout + bn - 1) / bn);
  int resident = 148 * (bn >= 128 ? 1 : 2);
  int splitk = 1;
  if (workspace != nullptr) {
    int best = 1 << 30;
    for (int sk = 1; sk <= 8; ++sk) {
      if (sk > 1 && (num_kb / sk < 6 || long(sk) * cs.M * Cout > workspace_floats)) break;
      const int waves = (tiles * sk + resident - 1) / resident;
      const int cost = waves * ((num_kb + sk - 1) / sk + 6) + (sk > 1 ? 8 : 0);
      if (cost < best) { best = cost; splitk = sk; }
    }
  } else {
    while (bn > 32 && m_tiles * ((Cout + bn - 1) / bn) < 148) bn >>= 1;
  }
  cs.kb_per = (num_kb + splitk - 1) / splitk;
  cs.splitk = (num_kb + cs.kb_per - 1) / cs.kb_per;
  CUtensorMap mw;
  int rc = make_tmap_2d(&mw, w, uint64_t(Cout), uint64_t(Kg), uint64_t(Kg), uint32_t(bn), 64, 2);
  if (rc) return rc - 30;
  DenseEpilogue e{out, bias, residual, cs.M, Cout, Cout, 0, 0, act, 0, 1};   // residual joins before the ReLU
  if (cs.splitk > 1) e = DenseEpilogue{workspace, nullptr, nullptr, cs.M, Cout, Cout, 0, 0, 0, 1, 0};
  const int bf = dtype == 0;
#define RONN_CONV(BN_) rc = bf ? launch_conv<BN_, __nv_bfloat16>(x, mw, cs, e, 1, status, stream) \
                               : launch_conv<BN_, __half>(x, mw, cs, e, 0, status, stream)
  switch (bn) {
    case 128: RONN_CONV(128); break;
    case 64: RONN_CONV(64); break;
    default: RONN_CONV(32); break;
  }
#undef RONN_CONV
  if (rc != 0 || cs.splitk == 1) return rc;
  // act 3: ReLU after the residual has been added (act 1 would apply it before)
  return ronn_splitk_finalize(workspace, cs.splitk, bias, residual, out, nullptr, nullptr, nullptr, long(cs.M), Cout, 0.f,
                              act ? 3 : 0, 0, dtype, stream);
}

extern "C" int ronn_maxpool_nhwc(const void* x, void* y, int N, int H, int W, int C, int Ho, int Wo, int k, int stride,
                                 int pad, int dtype, cudaStream_t stream) {
  if (C & 7) return -2;
  const long total = long(N) * Ho * Wo * (C >> 3);
  const int grid = int((total + 255) / 256 > 148 * 64 ? 148 * 64 : (total + 255) / 256);
  cudaError_t err;
  if (dtype == 0) err = launch(maxpool_nhwc_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, stream, (const __nv_bfloat16*)x, (__nv_bfloat16*)y, N, H, W, C, Ho, Wo, k, stride, pad);
  else err = launch(maxpool_nhwc_kernel<__half>, dim3(grid), dim3(256), 0, stream, (const __half*)x, (__half*)y, N, H, W, C, Ho, Wo, k, stride, pad);
  return err == cudaSuccess ? 0 : -100;
}

extern "C" int ronn_nchw_to_nhwc8(const void* x, void* y, int N, int C, int H, int W, int dtype, cudaStream_t stream) {
  if (C < 1 || C > 8 || N <= 0) return -2;
  const long HW = long(H) * W, total = long(N) * HW;
  const int grid = int((total + 255) / 256 > 148 * 64 ? 148 * 64 : (total + 255) / 256);
  cudaError_t err;
  if (dtype == 0) err = launch(nchw_to_nhwc8_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, stream, (const __nv_bfloat16*)x, (__nv_bfloat16*)y, C, HW, total);
  else err = launch(nchw_to_nhwc8_kernel<__half>, dim3(grid), dim3(256), 0, stream, (const __half*)x, (__half*)y, C, HW, total);
  return err == cudaSuccess ? 0 : -100;
}

extern "C" int ronn_nchw_to_s2d16(const void* x, void* y, int N, int C, int H, int W, int dtype, cudaStream_t stream) {
  if (C < 1 || C > 4 || N <= 0 || (H & 1) || (W & 1)) return -2;
  const long total = long(N) * (H / 2) * (W / 2);
  const int grid = int((total + 255) / 256 > 148 * 64 ? 148 * 64 : (total + 255) / 256);
  cudaError_t err;
  if (dtype == 0) err = launch(nchw_to_s2d16_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, stream, (const __nv_bfloat16*)x, (__nv_bfloat16*)y, C, H, W, total);
  else err = launch(nchw_to_s2d16_kernel<__half>, dim3(grid), dim3(256), 0, stream, (const __half*)x, (__half*)y, C, H, W, total);
  return err == cudaSuccess ? 0 : -100;
}

extern "C" int ronn_global_avgpool_nhwc(const void* x, void* y, int N, int HW, int C, int dtype, cudaStream_t stream) {
  if (C & 7) return -2;
  cudaError_t err;
  if (C >= 256) {
    dim3 wide(N, (C + 511) / 512);
    if (dtype == 0) err = launch(global_avgpool_wide_kernel<__nv_bfloat16>, wide, dim3(256), 0, stream, (const __nv_bfloat16*)x, (__nv_bfloat16*)y, HW, C);
    else err = launch(global_avgpool_wide_kernel<__half>, wide, dim3(256), 0, stream, (const __half*)x, (__half*)y, HW, C);
    return err == cudaSuccess ? 0 : -100;
  }
  dim3 grid(N, (C + 63) / 64);
  if (dtype == 0) err = launch(global_avgpool_nhwc_kernel<__nv_bfloat16>, grid, dim3(64), 0, stream, (const __nv_bfloat16*)x, (__nv_bfloat16*)y, HW, C);
  else err = launch(global_avgpool_nhwc_kernel<__half>, grid, dim3(64), 0, stream, (const __half*)x, (__half*)y, HW, C);
  return err == cudaSuccess ? 0 : -100;
}
