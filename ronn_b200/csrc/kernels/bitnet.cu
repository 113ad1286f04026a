// BitNet b1.58 device kernels: per-token int8 activation quantisation (optionally fused with RMSNorm) and the
// ternary x int8 BitLinear GEMM on the tcgen05 integer tensor-core path.
//
// Storage format of the weights is the reference's 2-bit code (crates/ronn-providers/src/bitnet/quantization.rs:131-153:
// 00 = -1, 01 = 0, 10 = +1, element i at bits 2*(i mod 4) of byte i/4), row-wise: W is [N, K/4] bytes.  The
// reference multiplies with a scalar triple loop on the CPU and re-quantises both operands on every call
// (crates/ronn-providers/src/bitnet/kernels.rs:134-178, 265-278); here weights stay packed in HBM (the decode GEMV/GEMM is
// weight-bandwidth bound, 2 bits per weight), are expanded to int8 on the fly by four producer warps straight into
// the 128-byte-swizzled shared-memory tile, and are multiplied with int8 activations by tcgen05.mma kind::i8 with
// exact int32 accumulation in TMEM.  Epilogue: acc * x_scale[token] * w_scale (+ bias).
#include <stdio.h>
#include <stdlib.h>

#include "gemm_epilogue.cuh"
#include "gemm_ll_phases.cuh"
#include "ptx_sm100.cuh"
#include "rowwise_stream.h"
#include "tma_desc.cuh"

namespace ronn {

// ---------------------------------------------------------------------------------------- activation quantisation
// q[row, :] = clamp(rint(v * 127 / max|v|)), scale[row] = max|v| / 127, with v = x (NORM = false) or
// v = x * rsqrt(mean(x^2) + eps) * gamma (NORM = true).  K % 16 == 0, K <= 16 * 4 * blockDim.
template <class T, bool NORM>
__global__ void act_quant_kernel(const T* __restrict__ x, const T* __restrict__ gamma, int8_t* __restrict__ q,
                                 float* __restrict__ scale, int K, float eps) {
  __shared__ float scratch[32];
  pdl_wait();
  pdl_trigger();
  const long row = blockIdx.x;
  const T* xr = x + row * K;
  const int nchunk = K >> 4;                 // 16 values per chunk (one 16-byte int8 store)
  float v[4][16];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
    if (ch < nchunk) {
      float a[8], b[8];
      unpack8<T>(*reinterpret_cast<const Vec8*>(xr + ch * 16), a);
      unpack8<T>(*reinterpret_cast<const Vec8*>(xr + ch * 16 + 8), b);
#pragma unroll
      for (int i = 0; i < 8; ++i) { v[c][i] = a[i]; v[c][8 + i] = b[i]; ss += a[i] * a[i] + b[i] * b[i]; }
    }
  }
  if (NORM) {
    const float inv = rsqrtf(block_sum(ss, scratch) / float(K) + eps);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int ch = threadIdx.x + c * blockDim.x;
      if (ch < nchunk) {
        float g0[8], g1[8];
        unpack8<T>(*reinterpret_cast<const Vec8*>(gamma + ch * 16), g0);
        unpack8<T>(*reinterpret_cast<const Vec8*>(gamma + ch * 16 + 8), g1);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          // round through the storage type so the fused path equals norm-then-quantise on 16-bit activations
          v[c][i] = Cvt<T>::to_f(Cvt<T>::from_f(v[c][i] * inv * g0[i]));
          v[c][8 + i] = Cvt<T>::to_f(Cvt<T>::from_f(v[c][8 + i] * inv * g1[i]));
        }
      }
    }
  }
  float m = 0.f;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
    if (ch < nchunk) {
#pragma unroll
      for (int i = 0; i < 16; ++i) m = fmaxf(m, fabsf(v[c][i]));
    }
  }
  m = fmaxf(block_max(m, scratch), 1e-5f);
  const float qs = __fdiv_rn(127.f, m);            // IEEE division: bit-identical to the host quantiser
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
    if (ch < nchunk) {
      alignas(16) int8_t o[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float r = fminf(fmaxf(rintf(__fmul_rn(v[c][i], qs)), -127.f), 127.f);
        o[i] = int8_t(int(r));
      }
      *reinterpret_cast<int4*>(q + row * K + ch * 16) = *reinterpret_cast<const int4*>(o);
    }
  }
  if (threadIdx.x == 0) scale[row] = __fdiv_rn(m, 127.f);
}

// SwiGLU on a fused [rows, 2 F] gate | up projection followed by the per-token int8 quantisation of the result, in one
// pass: v = silu(gate) * up (rounded through the storage type, as the two-kernel form stores it), q = rint(v * 127 /
// max|v|).  Saves the [rows, F] round trip through memory and a launch in front of the down projection.
// F % 16 == 0, F <= 16 * 4 * blockDim.
template <class T>
__global__ void swiglu_quant_kernel(const T* __restrict__ x, int8_t* __restrict__ q, float* __restrict__ scale, int F) {
  __shared__ float scratch[32];
  pdl_wait();
  pdl_trigger();
  const long row = blockIdx.x;
  const T* g = x + row * 2 * F;
  const T* u = g + F;
  const int nchunk = F >> 4;
  float v[4][16];
  float m = 0.f;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
    if (ch < nchunk) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float a[8], b[8];
        unpack8<T>(*reinterpret_cast<const Vec8*>(g + ch * 16 + h * 8), a);
        unpack8<T>(*reinterpret_cast<const Vec8*>(u + ch * 16 + h * 8), b);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float t = Cvt<T>::to_f(Cvt<T>::from_f(a[i] / (1.f + __expf(-a[i])) * b[i]));
          v[c][h * 8 + i] = t;
          m = fmaxf(m, fabsf(t));
        }
      }
    }
  }
  m = fmaxf(block_max(m, scratch), 1e-5f);
  const float qs = __fdiv_rn(127.f, m);
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
    if (ch < nchunk) {
      alignas(16) int8_t o[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float r = fminf(fmaxf(rintf(__fmul_rn(v[c][i], qs)), -127.f), 127.f);
        o[i] = int8_t(int(r));
      }
      *reinterpret_cast<int4*>(q + row * F + ch * 16) = *reinterpret_cast<const int4*>(o);
    }
  }
  if (threadIdx.x == 0) scale[row] = __fdiv_rn(m, 127.f);
}

// ---------------------------------------------------------------------------------------- BitLinear GEMM
constexpr int BL_THREADS = 320;
static_assert(BL_THREADS == PG_THREADS, "the low-latency all-reduce phases are written for the GEMM kernels' CTA size");
//          // warps 0-7 expand weights (0-3 also run the epilogue), 8 loads, 9 issues the MMAs

// A CTA's K chain is bound by latency, not by bandwidth (measured: the same time per K block for 8 and for 128
// activation rows): the time per K block is the round trip stage-freed -> loads issued -> data landed, divided by
// the number of stages in flight.  So the rings are as deep as shared memory allows, and the packed weights come
// in by TMA as well (WSTAGES stages of 4 K blocks each) instead of through registers, where the number of loads a
// warp can keep in flight is small.
template <int BN>
struct BitSmem {
  static constexpr int STAGES = BN <= 32 ? 8 : (BN <= 64 ? 7 : 5);
  static constexpr int WSTAGES = BN <= 64 ? 4 : 3;          // packed-weight stages: BN rows x 128 bytes = 4 K blocks
  static constexpr int A_BYTES = 128 * 128;
  static constexpr int B_BYTES = BN * 128;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int TILE_BYTES = STAGES * STAGE_BYTES;
  static constexpr int W_BYTES = BN * 128;
  static constexpr int WTILE_BYTES = WSTAGES * W_BYTES;
  static constexpr int DYN_SMEM = TILE_BYTES + WTILE_BYTES + (2 * STAGES + 2 * WSTAGES + 1) * 8 + 16 + 1024;
  static constexpr uint32_t TMEM_COLS = BN <= 32 ? 32u : (BN <= 64 ? 64u : 128u);
};

__device__ __forceinline__ void cluster_arrive_release() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait_acquire() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// 4 packed bytes (16 codes of 2 bits: 0 -> -1, 1 -> 0, 2 -> +1; code i at bits 2 * (i mod 4) of byte i / 4) -> 16 int8.
// Four masks pull codes i, i + 4, i + 8, i + 12 apart (one code per byte), a 4 x 4 byte transpose (eight byte
// permutes) puts them in order, and (b + 0x7f) ^ 0x80 per byte maps {0, 1, 2} to {-1, 0, +1} without a carry
// between bytes.
__device__ __forceinline__ int4 expand16(uint32_t w) {
  const uint32_t a0 = w & 0x03030303u, a1 = (w >> 2) & 0x03030303u, a2 = (w >> 4) & 0x03030303u, a3 = (w >> 6) & 0x03030303u;
  const uint32_t t01lo = __byte_perm(a0, a1, 0x5140), t23lo = __byte_perm(a2, a3, 0x5140);
  const uint32_t t01hi = __byte_perm(a0, a1, 0x7362), t23hi = __byte_perm(a2, a3, 0x7362);
  int4 o;
  o.x = int((__byte_perm(t01lo, t23lo, 0x5410) + 0x7f7f7f7fu) ^ 0x80808080u);
  o.y = int((__byte_perm(t01lo, t23lo, 0x7632) + 0x7f7f7f7fu) ^ 0x80808080u);
  o.z = int((__byte_perm(t01hi, t23hi, 0x5410) + 0x7f7f7f7fu) ^ 0x80808080u);
  o.w = int((__byte_perm(t01hi, t23hi, 0x7632) + 0x7f7f7f7fu) ^ 0x80808080u);
  return o;
}

// WTMA: the packed weights are fetched by TMA (needs K % 64 == 0 and a 16-byte aligned matrix); otherwise by plain loads.
// LLMODE: 0 = the tile is finished and stored by this CTA (or by its cluster); 1 / 2 = row-parallel projection under
// tensor parallelism: the scaled tile goes to the row owners as {data, sequence} words (phase A of the low-latency
// all-reduce, gemm_ll_phases.cuh) and the kernel goes on to reduce, broadcast (peer stores / multimem.st) and unpack.
template <int BN, class T, bool WTMA, int LLMODE>
__device__ __forceinline__ void bitlinear_cta(const CUtensorMap& map_x, const CUtensorMap& map_w,
                 const uint8_t* __restrict__ w_packed,
                 const float* __restrict__ x_scale, float w_scale, const T* __restrict__ bias, T* __restrict__ out,
                 int M, int N, int K, uint32_t idesc, uint32_t* status, const int* slot_state, long slot_stride,
                 int4* __restrict__ partials, const LLArgs& ll) {
  using L = BitSmem<BN>;
  constexpr int BL_STAGES = L::STAGES, WS = L::WSTAGES;
  extern __shared__ uint8_t dyn_smem[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dyn_smem) + 1023) & ~uintptr_t(1023));
  uint8_t* wtiles = tiles + L::TILE_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(wtiles + L::WTILE_BYTES);
  uint64_t* empty = full + BL_STAGES;
  uint64_t* wfull = empty + BL_STAGES;
  uint64_t* wempty = wfull + WS;
  uint64_t* accum = wempty + WS;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum + 1);
  volatile uint32_t* abort = tmem_slot + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BN, m0 = blockIdx.y * 128;
  // The K range is cut into gridDim.z slices, one per CTA of a cluster (1, 1, gridDim.z).  A CTA's chain of K blocks
  // is latency bound (an MMA of 128 rows takes ~70 cycles to issue however narrow it is, a barrier poll ~90: about
  // 600 cycles per block in each of the producer, expander and MMA loops), so a skinny GEMM that cannot fill the SMs
  // with output tiles gets faster by the number of slices.  The slices' int32 partial tiles meet in a workspace in
  // global memory (L2): measured, distributed shared memory moves ~13 bytes per cycle per SM and the same sum took
  // 3 us through it.
  const int S = int(gridDim.z);
  const int total_kb = (K + 127) / 128;
  const int kb_per = (total_kb + S - 1) / S;
  const int kb0 = int(blockIdx.z) * kb_per;
  const int num_kb = min(kb_per, total_kb - kb0);          // >= 1 (the launcher leaves no slice empty)
  const int kbytes = K >> 2;                 // packed bytes per weight row

  if (threadIdx.x == 0) {
    for (int s = 0; s < BL_STAGES; ++s) {
      mbar_init(&full[s], 4 + 1);            // one arrival per expander warp + the activation TMA's expect_tx arrival
      mbar_init(&empty[s], 1);
    }
    for (int s = 0; s < WS; ++s) {
      mbar_init(&wfull[s], 1);               // the weight TMA's expect_tx arrival
      mbar_init(&wempty[s], WTMA ? 8 : 4);   // one arrival per expander warp
    }
    mbar_init(accum, 1);
    *abort = 0;
    mbar_fence_init();
    fence_proxy_async_smem();
  }
  __syncwarp();
  if (warp == 9) {
    tmem_alloc(tmem_slot, L::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < 8) {
    // -------------------------------------------------- weight expansion: (row, chunk) pairs striped over 128 threads
    // weights are constants: no dependency wait needed before reading them
    constexpr int TASKS = BN * 8 / 128;      // 16-byte output chunks per thread per stage
    bool ok = true;
    if constexpr (WTMA) {
      // packed words come from the TMA-filled ring (128-byte swizzled: 16-byte chunk c of row r sits at c ^ (r & 7)).
      // Warps 0-3 take the even K blocks and warps 4-7 the odd ones: a group's wait - expand - arrive chain has two
      // block times to complete.
      const int grp = warp >> 2, gtid = threadIdx.x & 127;
      int seen_wb = -1;
      for (int kb = grp; kb < num_kb; kb += 2) {
        const int s = kb % BL_STAGES, wb = kb >> 2, ws = wb % WS, sub = kb & 3;
        if (lane == 0 && ok) {
          if (wb != seen_wb && !mbar_wait(&wfull[ws], (wb / WS) & 1, abort, status, STATUS_WAIT_TMA)) ok = false;
          if (ok && !mbar_wait(&empty[s], ((kb / BL_STAGES) & 1) ^ 1, abort, status, STATUS_WAIT_SLOT)) ok = false;
        }
        seen_wb = wb;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (ok) {
          uint8_t* sb = tiles + s * L::STAGE_BYTES + L::A_BYTES;
          const uint8_t* wp = wtiles + ws * L::W_BYTES;
#pragma unroll
          for (int t = 0; t < TASKS; ++t) {
            const int task = gtid + t * 128;
            const int r = task >> 3, j = task & 7;
            const uint32_t c = uint32_t(sub * 2 + (j >> 2));
            const uint32_t word = *reinterpret_cast<const uint32_t*>(wp + r * 128 + ((c ^ uint32_t(r & 7)) << 4) + (j & 3) * 4);
            *reinterpret_cast<int4*>(sb + r * 128 + ((uint32_t(j) ^ uint32_t(r & 7)) << 4)) = expand16(word);
          }
        }
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&full[s]);
          // the group's last block inside this packed stage: the next one it would take lies in another stage (or past the end)
          if (((kb + 2) >> 2) != wb || kb + 2 >= num_kb) mbar_arrive(&wempty[ws]);
        }
      }
    } else if (warp < 4) {
      auto fetch = [&](uint32_t (&dst)[TASKS], int kb) {
#pragma unroll
        for (int t = 0; t < TASKS; ++t) {
          const int task = threadIdx.x + t * 128;
          const int r = task >> 3, j = task & 7;
          const int n = n0 + r;
          const int byte0 = (kb0 + kb) * 32 + j * 4;
          dst[t] = 0x55555555u;              // all-zero weights outside the matrix
          if (kb < num_kb && n < N && byte0 < kbytes)
            dst[t] = __ldg(reinterpret_cast<const uint32_t*>(w_packed + size_t(n) * kbytes + byte0));
        }
      };
      // the packed words of the next DEPTH K blocks are in flight (in registers) while a block is expanded
      constexpr int DEPTH = TASKS <= 2 ? 8 : (TASKS <= 4 ? 6 : 4);
      uint32_t pq[DEPTH][TASKS];
#pragma unroll
      for (int d = 0; d < DEPTH; ++d) fetch(pq[d], d);
      for (int kb0 = 0; kb0 < num_kb; kb0 += DEPTH) {
#pragma unroll
        for (int d = 0; d < DEPTH; ++d) {
          const int kb = kb0 + d;
          if (kb < num_kb) {
            const int s = kb % BL_STAGES;
            if (lane == 0 && ok && !mbar_wait(&empty[s], ((kb / BL_STAGES) & 1) ^ 1, abort, status, STATUS_WAIT_SLOT)) ok = false;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (ok) {
              uint8_t* sb = tiles + s * L::STAGE_BYTES + L::A_BYTES;
#pragma unroll
              for (int t = 0; t < TASKS; ++t) {
                const int task = threadIdx.x + t * 128;
                const int r = task >> 3, j = task & 7;
                *reinterpret_cast<int4*>(sb + r * 128 + ((uint32_t(j) ^ uint32_t(r & 7)) << 4)) = expand16(pq[d][t]);
              }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&full[s]);
            fetch(pq[d], kb + DEPTH);
          }
        }
      }
    }
    if (warp < 4) {
      // -------------------------------------------------- epilogue
      pdl_wait();
      pdl_trigger();
      // double-buffered destination (the partial-sum slots of a tensor-parallel reduction): the slot is chosen by the
      // low bit of a device-side call counter, so a replayed CUDA graph follows the alternation without new arguments
      if (slot_state != nullptr)
        out = reinterpret_cast<T*>(reinterpret_cast<uint8_t*>(out) +
                                   size_t(*reinterpret_cast<const volatile int*>(slot_state) & 1) * size_t(slot_stride));
      bool acc_ok = mbar_wait(accum, 0, abort, status, STATUS_WAIT_ACCUM);
      acc_ok = __all_sync(0xffffffffu, acc_ok);
      tc_fence_after_sync();
      const int gm = m0 + threadIdx.x;
      if (LLMODE != 0) {
        if (acc_ok) {
          uint32_t seq;
          size_t poff;
          ll_resolve(ll, seq, poff);
          const float rs = gm < M ? x_scale[gm] * w_scale : 0.f;
          uint8_t* stage_w = tiles + warp * (32 * 80);         // the stage ring is idle: every MMA has completed
#pragma unroll 1
          for (int col = 0; col < BN; col += 32) {
            uint32_t r[32];
            tmem_ld_32x32(tmem_base + (uint32_t(warp * 32) << 16) + uint32_t(col), r);
            tmem_ld_wait();
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = float(int(r[i])) * rs;
            ll_scatter_chunk<T>(ll, seq, poff, ll.rank, gm, n0 + col, v, stage_w);
          }
        }
      } else if (acc_ok && S > 1) {
        // this slice's partial tile -> the workspace, 16 bytes per (4 columns, row): the rows of a warp are
        // consecutive, so a warp stores (and later loads) 512 contiguous bytes.  Written after the dependency wait:
        // the previous kernel on the stream may be another call that uses the same workspace.
        int4* mine = partials + (size_t(blockIdx.y * gridDim.x + blockIdx.x) * S + blockIdx.z) * (BN / 4) * 128;
        constexpr int STEP = BN >= 64 ? 64 : 32;               // two TMEM loads in flight where the tile has them
#pragma unroll 1
        for (int col = 0; col < BN; col += STEP) {
          uint32_t r[STEP / 32][32];
#pragma unroll
          for (int h = 0; h < STEP / 32; ++h) tmem_ld_32x32(tmem_base + (uint32_t(warp * 32) << 16) + uint32_t(col + 32 * h), r[h]);
          tmem_ld_wait();
#pragma unroll
          for (int h = 0; h < STEP / 32; ++h)
#pragma unroll
            for (int g = 0; g < 8; ++g)
              __stcg(&mine[(((col + 32 * h) >> 2) + g) * 128 + threadIdx.x],
                     make_int4(int(r[h][4 * g]), int(r[h][4 * g + 1]), int(r[h][4 * g + 2]), int(r[h][4 * g + 3])));
        }
      } else if (acc_ok) {
        const float rs = gm < M ? x_scale[gm] * w_scale : 0.f;
#pragma unroll 1
        for (int col = 0; col < BN; col += 32) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_base + (uint32_t(warp * 32) << 16) + uint32_t(col), r);
          tmem_ld_wait();
          const int gn = n0 + col;
          if (gm >= M || gn >= N) continue;
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = float(int(r[i])) * rs;
          if (bias) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (gn + i < N) v[i] += Cvt<T>::to_f(bias[gn + i]);
          }
          T* dst = out + size_t(gm) * N + gn;
          if (gn + 32 <= N && (N & 7) == 0) {
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
              float f[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) f[i] = v[jj * 8 + i];
              *reinterpret_cast<Vec8*>(dst + jj * 8) = pack8<T>(f);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (gn + i < N) dst[i] = Cvt<T>::from_f(v[i]);
          }
        }
      }
    }
  } else if (warp == 8) {
    if (lane == 0) {
      if constexpr (WTMA) {
        // weights are constants: their first stages are requested before the dependency wait
        const int nwb = (num_kb + 3) >> 2;
        for (int wb = 0; wb < WS && wb < nwb; ++wb) {
          mbar_expect_tx(&wfull[wb], L::W_BYTES);
          tma_load_2d(wtiles + wb * L::W_BYTES, &map_w, &wfull[wb], kb0 * 32 + wb * 128, n0);
        }
      }
      pdl_wait();                            // activations come from the previous kernel
      pdl_trigger();                         // successor may launch and set up under this kernel
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % BL_STAGES;
        if constexpr (WTMA) {
          // the packed-weight stage that the expanders have just released is refilled 4 * (WS - 1) K blocks ahead
          const int wb = (kb >> 2) + WS - 1;
          if ((kb & 3) == 0 && kb > 0 && wb < ((num_kb + 3) >> 2)) {
            const int ws = wb % WS;
            if (!mbar_wait(&wempty[ws], ((wb / WS) & 1) ^ 1, abort, status, STATUS_WAIT_SLOT)) break;
            mbar_expect_tx(&wfull[ws], L::W_BYTES);
            tma_load_2d(wtiles + ws * L::W_BYTES, &map_w, &wfull[ws], kb0 * 32 + wb * 128, n0);
          }
        }
        if (!mbar_wait(&empty[s], ((kb / BL_STAGES) & 1) ^ 1, abort, status, STATUS_WAIT_SLOT)) break;
        mbar_expect_tx(&full[s], L::A_BYTES);
        tma_load_2d(tiles + s * L::STAGE_BYTES, &map_x, &full[s], (kb0 + kb) * 128, m0);
      }
    }
    __syncwarp();
    pdl_trigger();
  } else {
    if (lane == 0) {
      // A barrier poll takes ~90 cycles to answer: the poll of the next stage is issued before this stage's MMAs and
      // read after them.
      bool ready = mbar_try_wait(&full[0], 0);
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % BL_STAGES;
        if (!ready && !mbar_wait(&full[s], (kb / BL_STAGES) & 1, abort, status, STATUS_WAIT_TMA)) break;
        // the expander warps wrote the weight tile through the generic proxy and released it with their arrivals: one
        // proxy fence after the acquire orders those writes before the tensor core's reads
        fence_proxy_async_smem();
        tc_fence_after_sync();
        const int kn = kb + 1;
        ready = kn < num_kb && mbar_try_wait(&full[kn % BL_STAGES], (kn / BL_STAGES) & 1);
        const uint32_t sa = smem_u32(tiles + s * L::STAGE_BYTES);
        const uint64_t adesc = umma_desc_k128(sa), bdesc = umma_desc_k128(sa + L::A_BYTES);
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_i8(tmem_base, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0);
        umma_commit(&empty[s]);
      }
      umma_commit(accum);
    }
    __syncwarp();
    pdl_trigger();
  }
  if (*abort) {
    const long long t0 = clock64();
    while (clock64() - t0 < 400000ll) { __nanosleep(1000); }
  }
  if (S > 1) {
    // every CTA of the cluster sums BN / S columns of the tile over all slices (exact: int32) and finishes them.  The
    // cluster barrier (release / acquire) orders the slices' workspace stores before the loads below.
    cluster_arrive_release();
    cluster_wait_acquire();
    if (warp < 4 && !*abort) {
      // A load from L2 of data another SM has just written takes over a thousand cycles, so all loads of a pass are
      // issued before the first is used.  The number of slices is a run-time value but registers want constant
      // indices: a pass loads PASS consecutive (column group, slice) pairs, slice fastest, sums neighbours in
      // log2(S) steps, and the pairs whose index is a multiple of S hold the finished groups of 4 columns.
      constexpr int PASS = BN / 4 < 16 ? BN / 4 : 16;
      const int lg = 31 - __clz(S);
      const int cwg = (BN / 4) >> lg;                        // column groups this CTA finishes
      const int z = int(cluster_ctarank());
      const int gm = m0 + threadIdx.x;
      const float rs = gm < M ? x_scale[gm] * w_scale : 0.f;
      const int4* tile_ws = partials + size_t(blockIdx.y * gridDim.x + blockIdx.x) * S * (BN / 4) * 128 + threadIdx.x;
#pragma unroll 1
      for (int p = 0; p < (BN / 4) / PASS; ++p) {
        int4 v[PASS];
#pragma unroll
        for (int j = 0; j < PASS; ++j) {
          const int flat = p * PASS + j, g = z * cwg + (flat >> lg), r = flat & (S - 1);
          v[j] = __ldcg(tile_ws + size_t(r * (BN / 4) + g) * 128);
        }
#pragma unroll
        for (int step = 1; step < 8; step <<= 1)
          if (S > step) {
#pragma unroll
            for (int j = 0; j < PASS; j += 2 * step)
              if (j + step < PASS) {
                v[j].x += v[j + step].x; v[j].y += v[j + step].y; v[j].z += v[j + step].z; v[j].w += v[j + step].w;
              }
          }
#pragma unroll
        for (int j = 0; j < PASS; ++j) {
          if ((j & (S - 1)) != 0) continue;
          const int gn = n0 + (z * cwg + ((p * PASS + j) >> lg)) * 4;
          if (gm >= M || gn >= N) continue;
          float f[4] = {float(v[j].x) * rs, float(v[j].y) * rs, float(v[j].z) * rs, float(v[j].w) * rs};
          if (bias) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
              if (gn + i < N) f[i] += Cvt<T>::to_f(bias[gn + i]);
          }
          T* dst = out + size_t(gm) * N + gn;
          if (gn + 4 <= N && (N & 3) == 0) {
            uint2 o;
            o.x = Pair16<T>::pack(f[0], f[1]);
            o.y = Pair16<T>::pack(f[2], f[3]);
            *reinterpret_cast<uint2*>(dst) = o;
          } else {
#pragma unroll
            for (int i = 0; i < 4; ++i)
              if (gn + i < N) dst[i] = Cvt<T>::from_f(f[i]);
          }
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, L::TMEM_COLS);
  }
}

template <int BN, class T, bool WTMA, int LLMODE>
__global__ void __launch_bounds__(BL_THREADS)
bitlinear_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                 const uint8_t* __restrict__ w_packed, const float* __restrict__ x_scale, float w_scale,
                 const T* __restrict__ bias, T* __restrict__ out, int M, int N, int K, uint32_t idesc, uint32_t* status,
                 const int* slot_state, long slot_stride, int4* __restrict__ partials, const __grid_constant__ LLArgs ll) {
  if (LLMODE == 0 || (ll.phases & 1))
    bitlinear_cta<BN, T, WTMA, LLMODE>(map_x, map_w, w_packed, x_scale, w_scale, bias, out, M, N, K, idesc, status,
                                       slot_state, slot_stride, partials, ll);
  if constexpr (LLMODE != 0) {
    __shared__ float s_red[8 * 16];
    __syncthreads();
    ll_phases<T, LLMODE == 2>(ll, status, s_red);
  }
}

// Offline packing on the device: int8 values in {-1,0,1} [rows, K] -> [rows, K/4] codes.
__global__ void ternary_pack_kernel(const int8_t* __restrict__ v, uint8_t* __restrict__ packed, long rows, int K) {
  const long total = rows * (K >> 2);
  for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < total; i += long(gridDim.x) * blockDim.x) {
    const int8_t* p = v + i * 4;
    uint32_t b = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int x = p[k];
      b |= uint32_t(x < 0 ? 0 : (x == 0 ? 1 : 2)) << (2 * k);
    }
    packed[i] = uint8_t(b);
  }
}

template <int BN, class T, bool WTMA>
static int launch_bitlinear(const CUtensorMap& mx, const CUtensorMap& mw, const void* w, const float* xs, float ws,
                            const void* bias, void* out, int M, int N, int K, int S, uint32_t* status, cudaStream_t stream,
                            const int* slot_state, long slot_stride, void* workspace) {
  using L = BitSmem<BN>;
  auto kern = bitlinear_kernel<BN, T, WTMA, 0>;
  LLArgs no_ll = {};
  static bool configured[MAX_DEVICES] = {false};
  if (first_use_on_device(configured)) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYN_SMEM) != cudaSuccess) return -10;
  }
  const uint32_t idesc = umma_idesc(128, BN, 1u, 2u);       // signed 8-bit operands, int32 accumulate
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((N + BN - 1) / BN, (M + 127) / 128, S);
  cfg.blockDim = dim3(BL_THREADS);
  cfg.dynamicSmemBytes = size_t(L::DYN_SMEM);
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;         // the K slices of one output tile form a cluster
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = unsigned(S);
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  prefer_max_shared(reinterpret_cast<const void*>(kern));
  cudaError_t err = cudaLaunchKernelEx(&cfg, kern, mx, mw, (const uint8_t*)w, xs, ws, (const T*)bias, (T*)out, M, N, K,
                                       idesc, status, slot_state, slot_stride, static_cast<int4*>(workspace), no_ll);
  return (err == cudaSuccess && cudaGetLastError() == cudaSuccess) ? 0 : -11;
}

}  // namespace ronn

using namespace ronn;

// dtype of x/gamma: 0 bf16, 1 fp16.  K % 16 == 0.
extern "C" int ronn_act_quant_int8(const void* x, void* q, float* scale, long rows, int K, int dtype,
                                   cudaStream_t stream) {
  if (rows <= 0) return 0;
  if ((K & 15) || K > 16 * 4 * 1024) return -2;
  {
    const int rc = rowwise_stream_try(3, x, nullptr, nullptr, nullptr, q, nullptr, scale, rows, K, K, 0, K, 0.f, dtype, stream);
    if (rc != 0) return rc < 0 ? rc : 0;
  }
  int threads = (((K >> 4) + 3) / 4 + 31) / 32 * 32;
  if (threads < 32) threads = 32;
  cudaError_t err;
  if (dtype == 0) err = launch(act_quant_kernel<__nv_bfloat16, false>, dim3(unsigned(rows)), dim3(threads), 0, stream, (const __nv_bfloat16*)x, (const __nv_bfloat16*)nullptr, (int8_t*)q, scale, K, 0.f);
  else err = launch(act_quant_kernel<__half, false>, dim3(unsigned(rows)), dim3(threads), 0, stream, (const __half*)x, (const __half*)nullptr, (int8_t*)q, scale, K, 0.f);
  return err == cudaSuccess ? 0 : -100;
}

// RMSNorm(x) * gamma, then per-token int8 quantisation, in one pass over the row.
extern "C" int ronn_norm_quant_int8(const void* x, const void* gamma, void* q, float* scale, void* unused, long rows,
                                    int K, float eps, int dtype, cudaStream_t stream) {
  (void)unused;
  if (rows <= 0) return 0;
  if ((K & 15) || K > 16 * 4 * 1024) return -2;
  {
    const int rc = rowwise_stream_try(4, x, nullptr, gamma, nullptr, q, nullptr, scale, rows, K, K, 0, K, eps, dtype, stream);
    if (rc != 0) return rc < 0 ? rc : 0;
  }
  int threads = (((K >> 4) + 3) / 4 + 31) / 32 * 32;
  if (threads < 32) threads = 32;
  cudaError_t err;
  if (dtype == 0) err = launch(act_quant_kernel<__nv_bfloat16, true>, dim3(unsigned(rows)), dim3(threads), 0, stream, (const __nv_bfloat16*)x, (const __nv_bfloat16*)gamma, (int8_t*)q, scale, K, eps);
  else err = launch(act_quant_kernel<__half, true>, dim3(unsigned(rows)), dim3(threads), 0, stream, (const __half*)x, (const __half*)gamma, (int8_t*)q, scale, K, eps);
  return err == cudaSuccess ? 0 : -100;
}

// Tile width and number of K slices: the pair with the lowest estimated time, from a model fitted to measurements
// (128 x 2560..13824 x 864..6912 in a CUDA graph).  A CTA costs a fixed part (launch, barrier and TMEM set-up, first
// loads from DRAM: 2.3 us) and 0.32 / 0.36 / 0.48 us per 128-deep K block of its slice for 32 / 64 / 128 columns (the
// MMA issuer's loop: every MMA streams its 128 x 32-byte A operand from shared memory, ~70 cycles, four per block,
// plus ~220 cycles of barrier traffic; wide tiles add expansion time).  Slicing K costs 1.5 us (cluster barrier and
// an L2 round trip on data other SMs have just written) plus 0.4 us per MB of partial tiles.  The grid runs in waves
// of one CTA per SM.
static void bitlinear_plan(int M, int N, int K, bool may_slice, int& bn, int& S) {
  const int mt = (M + 127) / 128, total_kb = (K + 127) / 128, sms = device_sm_count();
  bn = 128;
  S = 1;
  float best = 1e30f;
  const int bns[3] = {128, 64, 32};
  const float per_kb[3] = {0.476f, 0.364f, 0.324f};
  for (int i = 0; i < 3; ++i)
    for (int s = 1; s <= (may_slice ? 8 : 1); s <<= 1) {
      if (bns[i] / s < 8 || s > total_kb) continue;
      const int per = (total_kb + s - 1) / s;
      if ((total_kb + per - 1) / per != s) continue;       // a slice would be empty
      const int ctas = mt * ((N + bns[i] - 1) / bns[i]) * s;
      if (s > 1 && ctas > sms) continue;                     // slices only where they fill otherwise idle SMs
      const int waves = (ctas + sms - 1) / sms;
      const float part_mb = float(ctas) * float(bns[i]) * 512.f / 1048576.f;
      const float t = float(waves) * (2.3f + per_kb[i] * float(per)) + (s > 1 ? 1.5f + 0.4f * part_mb : 0.f);
      if (t < best) { best = t; bn = bns[i]; S = s; }
    }
  if (const char* e = getenv("RONN_BITLINEAR_TILE")) {       // "bn,slices" override for experiments
    int b = 0, s = 0;
    if (sscanf(e, "%d,%d", &b, &s) == 2 && (b == 32 || b == 64 || b == 128) && s >= 1 && s <= 8 && b / s >= 8 &&
        (s & (s - 1)) == 0 && (may_slice || s == 1)) {
      const int per = (total_kb + s - 1) / s;
      if (s <= total_kb && (total_kb + per - 1) / per == s && (s == 1 || mt * ((N + b - 1) / b) * s <= sms)) { bn = b; S = s; }
    }
  }
}

// Bytes of scratch memory a call of this shape wants for its K slices (0: the shape is not sliced).  At most one CTA
// per SM is sliced, so the answer never exceeds 148 x 64 KB.
extern "C" long ronn_bitlinear_workspace_bytes(int M, int N, int K) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  int bn, S;
  bitlinear_plan(M, N, K, true, bn, S);
  if (S == 1) return 0;
  return long((M + 127) / 128) * ((N + bn - 1) / bn) * S * bn * 512;
}

// x: [rows, 2 F] (gate | up), dtype 0 bf16 / 1 fp16 -> q int8 [rows, F], scale fp32 [rows].
extern "C" int ronn_swiglu_quant_int8(const void* x, void* q, float* scale, long rows, int F, int dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if ((F & 15) || F > 16 * 4 * 1024) return -2;
  int threads = (((F >> 4) + 3) / 4 + 31) / 32 * 32;
  if (threads < 32) threads = 32;
  cudaError_t err;
  if (dtype == 0) err = launch(swiglu_quant_kernel<__nv_bfloat16>, dim3(unsigned(rows)), dim3(threads), 0, stream, (const __nv_bfloat16*)x, (int8_t*)q, scale, F);
  else if (dtype == 1) err = launch(swiglu_quant_kernel<__half>, dim3(unsigned(rows)), dim3(threads), 0, stream, (const __half*)x, (int8_t*)q, scale, F);
  else return -6;
  return err == cudaSuccess ? 0 : -100;
}

// xq: int8 [M, K] (row stride ldx bytes); w_packed: [N, K/4]; x_scale: fp32 [M]; out: [M, N] in `dtype` (0 bf16, 1 fp16).
// K % 16 == 0 and ldx % 16 == 0.  workspace: null, or ronn_bitlinear_workspace_bytes(M, N, K) bytes (16-byte aligned)
// that no other call in flight uses; without it the K range is not sliced.
static int bitlinear_impl(const void* xq, const void* w_packed, const float* x_scale, float w_scale, const void* bias,
                          void* out, int M, int N, int K, int ldx, int dtype, const int* slot_state, long slot_stride,
                          void* workspace, uint32_t* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return -1;
  if ((K & 15) || (ldx & 15)) return -2;
  if (reinterpret_cast<uintptr_t>(workspace) & 15) return -2;
  int bn, S;
  bitlinear_plan(M, N, K, workspace != nullptr, bn, S);
  CUtensorMap mx;
  int rc = make_tmap_2d(&mx, xq, uint64_t(M), uint64_t(K), uint64_t(ldx), 128, 128, 1);
  if (rc) return rc - 20;
  // packed weights by TMA: rows of K / 4 bytes must be a multiple of 16 bytes and the matrix 16-byte aligned
  const bool wtma = (K & 63) == 0 && (reinterpret_cast<uintptr_t>(w_packed) & 15) == 0;
  CUtensorMap mw = mx;
  if (wtma) {
    rc = make_tmap_2d(&mw, w_packed, uint64_t(N), uint64_t(K >> 2), uint64_t(K >> 2), uint32_t(bn), 128, 1);
    if (rc) return rc - 30;
  }
#define RONN_BL2(BN_, T_, W_) launch_bitlinear<BN_, T_, W_>(mx, mw, w_packed, x_scale, w_scale, bias, out, M, N, K, S, status, stream, slot_state, slot_stride, workspace)
#define RONN_BL(BN_) return dtype == 0 ? (wtma ? RONN_BL2(BN_, __nv_bfloat16, true) : RONN_BL2(BN_, __nv_bfloat16, false)) \
                                       : (wtma ? RONN_BL2(BN_, __half, true) : RONN_BL2(BN_, __half, false))
  switch (bn) {
    case 128: RONN_BL(128);
    case 64: RONN_BL(64);
    default: RONN_BL(32);
  }
#undef RONN_BL
#undef RONN_BL2
}

extern "C" int ronn_bitlinear(const void* xq, const void* w_packed, const float* x_scale, float w_scale,
                              const void* bias, void* out, void* workspace, int M, int N, int K, int ldx, int dtype,
                              uint32_t* status, cudaStream_t stream) {
  return bitlinear_impl(xq, w_packed, x_scale, w_scale, bias, out, M, N, K, ldx, dtype, nullptr, 0, workspace, status, stream);
}

// Same GEMM, but the [M, N] result goes to out_base + (*slot_state & 1) * slot_stride bytes: the current partial-sum
// slot of a tensor-parallel reduction (ronn_peer_reduce), resolved on the device.
extern "C" int ronn_bitlinear_to_slot(const void* xq, const void* w_packed, const float* x_scale, float w_scale,
                                      void* out_base, const int* slot_state, long slot_stride, void* workspace, int M,
                                      int N, int K, int ldx, int dtype, uint32_t* status, cudaStream_t stream) {
  if (slot_state == nullptr || out_base == nullptr) return -1;
  return bitlinear_impl(xq, w_packed, x_scale, w_scale, nullptr, out_base, M, N, K, ldx, dtype, slot_state, slot_stride,
                        workspace, status, stream);
}

template <int BN, class T, int LLMODE>
static int launch_bitlinear_ll(const CUtensorMap& mx, const CUtensorMap& mw, const RonnBitLinearLLParams* p, LLArgs& a,
                               uint32_t* status, cudaStream_t stream) {
  using L = BitSmem<BN>;
  auto kern = bitlinear_kernel<BN, T, true, LLMODE>;
  static bool configured[MAX_DEVICES] = {false};
  if (first_use_on_device(configured)) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYN_SMEM) != cudaSuccess) return -10;
  }
  const int M = a.M, N = a.N, K = p->ll.K;
  const int grid_x = (N + BN - 1) / BN, grid_y = (M + 127) / 128;
  // phases B and C wait on work of the whole grid and of the peers: every CTA must be resident at once
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, BL_THREADS, L::DYN_SMEM) != cudaSuccess || per_sm < 1)
    return -12;
  if (grid_x * grid_y > device_sm_count() * per_sm) return -12;
  a.wpr = ll_pick_wpr(M, N, grid_x * grid_y);
  if (a.wpr == 0) return -5;
  const uint32_t idesc = umma_idesc(128, BN, 1u, 2u);
  cudaError_t err = launch(kern, dim3(grid_x, grid_y, 1), dim3(BL_THREADS), size_t(L::DYN_SMEM), stream, mx, mw,
                           static_cast<const uint8_t*>(p->w_packed), p->x_scale, p->w_scale, static_cast<const T*>(nullptr),
                           static_cast<T*>(nullptr), M, N, K, idesc, status, static_cast<const int*>(nullptr), 0l,
                           static_cast<int4*>(nullptr), a);
  return (err == cudaSuccess && cudaGetLastError() == cudaSuccess) ? 0 : -11;
}

// Row-parallel BitLinear of a tensor-parallel rank fused with the cross-rank sum, residual add (and norm) in ONE launch:
// int8 activations [M, K] of this rank's K shard x packed ternary weights [N, K / 4], the scaled partial rows travel
// as {data, sequence} words (see gemm_ll.h for the areas and the protocol).  K % 64 == 0, N % 32 == 0, the grid
// (N / 32 or N / 64 tiles) must fit the SMs.  Returns -12 when it does not: the caller then uses the two-launch path.
extern "C" int ronn_bitlinear_ll(const RonnBitLinearLLParams* p, uint32_t* status, cudaStream_t stream) {
  if (!p || !p->xq || !p->w_packed || !p->x_scale) return -1;
  const int M = p->ll.M, N = p->ll.N, K = p->ll.K;
  if (K <= 0 || (K & 63) || (p->ldx & 15) || (reinterpret_cast<uintptr_t>(p->w_packed) & 15)) return -2;
  LLArgs a;
  if (const int rc = ll_fill_args(&p->ll, a)) return rc;
  if (p->ll.scatter_parity_stride < long(p->ll.world) * a.owner_rows * N * 4 || p->ll.result_parity_stride < long(M) * N * 4)
    return -8;
  const int mt = (M + 127) / 128, sms = device_sm_count();
  const int bn = mt * ((N + 31) / 32) <= sms ? 32 : 64;
  CUtensorMap mx, mw;
  int rc = make_tmap_2d(&mx, p->xq, uint64_t(M), uint64_t(K), uint64_t(p->ldx), 128, 128, 1);
  if (rc) return rc - 20;
  rc = make_tmap_2d(&mw, p->w_packed, uint64_t(N), uint64_t(K >> 2), uint64_t(K >> 2), uint32_t(bn), 128, 1);
  if (rc) return rc - 30;
  const bool bf = p->ll.dtype == 0;
#define RONN_BLL(BN_, T_) (a.nvls ? launch_bitlinear_ll<BN_, T_, 2>(mx, mw, p, a, status, stream) \
                                  : launch_bitlinear_ll<BN_, T_, 1>(mx, mw, p, a, status, stream))
  if (bn == 32) return bf ? RONN_BLL(32, __nv_bfloat16) : RONN_BLL(32, __half);
  return bf ? RONN_BLL(64, __nv_bfloat16) : RONN_BLL(64, __half);
#undef RONN_BLL
}

extern "C" int ronn_ternary_pack(const void* values, void* packed, long rows, int K, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (K & 3) return -2;
  const long total = rows * (K >> 2);
  const int grid = int((total + 255) / 256 > 148 * 16 ? 148 * 16 : (total + 255) / 256);
  ternary_pack_kernel<<<grid, 256, 0, stream>>>((const int8_t*)values, (uint8_t*)packed, rows, K);
  return cudaGetLastError() == cudaSuccess ? 0 : -100;
}
