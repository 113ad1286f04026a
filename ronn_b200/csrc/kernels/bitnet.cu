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
#include "gemm_epilogue.cuh"
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

// ---------------------------------------------------------------------------------------- BitLinear GEMM
constexpr int BL_THREADS = 192;
constexpr int BL_STAGES = 4;

template <int BN>
struct BitSmem {
  static constexpr int A_BYTES = 128 * 128;
  static constexpr int B_BYTES = BN * 128;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int TILE_BYTES = BL_STAGES * STAGE_BYTES;
  static constexpr int DYN_SMEM = TILE_BYTES + (2 * BL_STAGES + 1) * 8 + 16 + 1024;
  static constexpr uint32_t TMEM_COLS = BN <= 32 ? 32u : (BN <= 64 ? 64u : 128u);
};

// 4 packed bytes (16 ternary codes) -> 16 int8 in {-1, 0, +1}
__device__ __forceinline__ int4 expand16(uint32_t p) {
  alignas(16) int8_t o[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const uint32_t code = (p >> (2 * i)) & 3u;
    o[i] = code == 0u ? int8_t(-1) : (code == 2u ? int8_t(1) : int8_t(0));
  }
  return *reinterpret_cast<const int4*>(o);
}

template <int BN, class T>
__global__ void __launch_bounds__(BL_THREADS)
bitlinear_kernel(const __grid_constant__ CUtensorMap map_x, const uint8_t* __restrict__ w_packed,
                 const float* __restrict__ x_scale, float w_scale, const T* __restrict__ bias, T* __restrict__ out,
                 int M, int N, int K, uint32_t idesc, uint32_t* status, const int* slot_state, long slot_stride) {
  using L = BitSmem<BN>;
  extern __shared__ uint8_t dyn_smem[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dyn_smem) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(tiles + L::TILE_BYTES);
  uint64_t* empty = full + BL_STAGES;
  uint64_t* accum = empty + BL_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum + 1);
  volatile uint32_t* abort = tmem_slot + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BN, m0 = blockIdx.y * 128;
  const int num_kb = (K + 127) / 128;
  const int kbytes = K >> 2;                 // packed bytes per weight row

  if (threadIdx.x == 0) {
    for (int s = 0; s < BL_STAGES; ++s) {
      mbar_init(&full[s], 4 + 1);            // one arrival per expander warp + the activation TMA's expect_tx arrival
      mbar_init(&empty[s], 1);
    }
    mbar_init(accum, 1);
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
    // -------------------------------------------------- weight expansion: (row, chunk) pairs striped over 128 threads
    // weights are constants: no dependency wait needed before reading them
    constexpr int TASKS = BN * 8 / 128;      // 16-byte output chunks per thread per stage
    // The packed words of K block kb + 2 are requested before block kb is expanded, so the global-load latency of
    // a stage is covered by two stages of expansion; barrier traffic is one wait and one arrival per warp.
    auto fetch = [&](uint32_t (&dst)[TASKS], int kb) {
#pragma unroll
      for (int t = 0; t < TASKS; ++t) {
        const int task = threadIdx.x + t * 128;
        const int r = task >> 3, j = task & 7;
        const int n = n0 + r;
        const int byte0 = kb * 32 + j * 4;
        dst[t] = 0x55555555u;                // all-zero weights outside the matrix
        if (kb < num_kb && n < N && byte0 < kbytes)
          dst[t] = __ldg(reinterpret_cast<const uint32_t*>(w_packed + size_t(n) * kbytes + byte0));
      }
    };
    uint32_t p0[TASKS], p1[TASKS], p2[TASKS];
    fetch(p0, 0);
    fetch(p1, 1);
    bool ok = true;
    for (int kb = 0; kb < num_kb; ++kb) {
      const int s = kb % BL_STAGES;
      fetch(p2, kb + 2);
      if (lane == 0 && ok && !mbar_wait(&empty[s], ((kb / BL_STAGES) & 1) ^ 1, abort, status, STATUS_WAIT_SLOT)) ok = false;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (ok) {
        uint8_t* sb = tiles + s * L::STAGE_BYTES + L::A_BYTES;
#pragma unroll
        for (int t = 0; t < TASKS; ++t) {
          const int task = threadIdx.x + t * 128;
          const int r = task >> 3, j = task & 7;
          *reinterpret_cast<int4*>(sb + r * 128 + ((uint32_t(j) ^ uint32_t(r & 7)) << 4)) = expand16(p0[t]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&full[s]);
#pragma unroll
      for (int t = 0; t < TASKS; ++t) {
        p0[t] = p1[t];
        p1[t] = p2[t];
      }
    }
    // -------------------------------------------------- epilogue
    pdl_wait();
    pdl_trigger();
    // double-buffered destination (the partial-sum slots of a tensor-parallel reduction): the slot is chosen by the low
    // bit of a device-side call counter, so a replayed CUDA graph follows the alternation without new arguments
    if (slot_state != nullptr)
      out = reinterpret_cast<T*>(reinterpret_cast<uint8_t*>(out) +
                                 size_t(*reinterpret_cast<const volatile int*>(slot_state) & 1) * size_t(slot_stride));
    bool acc_ok = mbar_wait(accum, 0, abort, status, STATUS_WAIT_ACCUM);
    acc_ok = __all_sync(0xffffffffu, acc_ok);
    tc_fence_after_sync();
    const int gm = m0 + threadIdx.x;
    if (acc_ok) {
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
  } else if (warp == 4) {
    if (lane == 0) {
      pdl_wait();                            // activations come from the previous kernel
      pdl_trigger();                         // successor may launch and set up under this kernel
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % BL_STAGES;
        if (!mbar_wait(&empty[s], ((kb / BL_STAGES) & 1) ^ 1, abort, status, STATUS_WAIT_SLOT)) break;
        mbar_expect_tx(&full[s], L::A_BYTES);
        tma_load_2d(tiles + s * L::STAGE_BYTES, &map_x, &full[s], kb * 128, m0);
      }
    }
    __syncwarp();
    pdl_trigger();
  } else {
    if (lane == 0) {
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % BL_STAGES;
        if (!mbar_wait(&full[s], (kb / BL_STAGES) & 1, abort, status, STATUS_WAIT_TMA)) break;
        // the expander warps wrote the weight tile through the generic proxy and released it with their arrivals: one
        // proxy fence after the acquire orders those writes before the tensor core's reads
        fence_proxy_async_smem();
        tc_fence_after_sync();
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
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, L::TMEM_COLS);
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

template <int BN, class T>
static int launch_bitlinear(const CUtensorMap& mx, const void* w, const float* xs, float ws, const void* bias, void* out,
                            int M, int N, int K, uint32_t* status, cudaStream_t stream, const int* slot_state = nullptr,
                            long slot_stride = 0) {
  using L = BitSmem<BN>;
  auto kern = bitlinear_kernel<BN, T>;
  static bool configured[MAX_DEVICES] = {false};
  if (first_use_on_device(configured)) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYN_SMEM) != cudaSuccess) return -10;
  }
  dim3 grid((N + BN - 1) / BN, (M + 127) / 128);
  const uint32_t idesc = umma_idesc(128, BN, 1u, 2u);       // signed 8-bit operands, int32 accumulate
  cudaError_t err = launch(kern, grid, dim3(BL_THREADS), size_t(L::DYN_SMEM), stream, mx, (const uint8_t*)w, xs, ws,
                           (const T*)bias, (T*)out, M, N, K, idesc, status, slot_state, slot_stride);
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

// xq: int8 [M, K] (row stride ldx bytes); w_packed: [N, K/4]; x_scale: fp32 [M]; out: [M, N] in `dtype` (0 bf16, 1 fp16).
// K % 16 == 0 and ldx % 16 == 0.
static int bitlinear_impl(const void* xq, const void* w_packed, const float* x_scale, float w_scale, const void* bias,
                          void* out, int M, int N, int K, int ldx, int dtype, const int* slot_state, long slot_stride,
                          uint32_t* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return -1;
  if ((K & 15) || (ldx & 15)) return -2;
  int bn = 128;
  const int mt = (M + 127) / 128;
  while (bn > 32 && mt * ((N + bn - 1) / bn) < 120) bn >>= 1;
  CUtensorMap mx;
  int rc = make_tmap_2d(&mx, xq, uint64_t(M), uint64_t(K), uint64_t(ldx), 128, 128, 1);
  if (rc) return rc - 20;
#define RONN_BL(BN_) return dtype == 0 ? launch_bitlinear<BN_, __nv_bfloat16>(mx, w_packed, x_scale, w_scale, bias, out, M, N, K, status, stream, slot_state, slot_stride) \
                                       : launch_bitlinear<BN_, __half>(mx, w_packed, x_scale, w_scale, bias, out, M, N, K, status, stream, slot_state, slot_stride)
  switch (bn) {
    case 128: RONN_BL(128);
    case 64: RONN_BL(64);
    default: RONN_BL(32);
  }
#undef RONN_BL
}

extern "C" int ronn_bitlinear(const void* xq, const void* w_packed, const float* x_scale, float w_scale,
                              const void* bias, void* out, void* unused, int M, int N, int K, int ldx, int dtype,
                              uint32_t* status, cudaStream_t stream) {
  (void)unused;
  return bitlinear_impl(xq, w_packed, x_scale, w_scale, bias, out, M, N, K, ldx, dtype, nullptr, 0, status, stream);
}

// Same GEMM, but the [M, N] result goes to out_base + (*slot_state & 1) * slot_stride bytes: the current partial-sum
// slot of a tensor-parallel reduction (ronn_peer_reduce), resolved on the device.
extern "C" int ronn_bitlinear_to_slot(const void* xq, const void* w_packed, const float* x_scale, float w_scale,
                                      void* out_base, const int* slot_state, long slot_stride, int M, int N, int K,
                                      int ldx, int dtype, uint32_t* status, cudaStream_t stream) {
  if (slot_state == nullptr || out_base == nullptr) return -1;
  return bitlinear_impl(xq, w_packed, x_scale, w_scale, nullptr, out_base, M, N, K, ldx, dtype, slot_state, slot_stride,
                        status, stream);
}

extern "C" int ronn_ternary_pack(const void* values, void* packed, long rows, int K, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (K & 3) return -2;
  const long total = rows * (K >> 2);
  const int grid = int((total + 255) / 256 > 148 * 16 ? 148 * 16 : (total + 255) / 256);
  ternary_pack_kernel<<<grid, 256, 0, stream>>>((const int8_t*)values, (uint8_t*)packed, rows, K);
  return cudaGetLastError() == cudaSuccess ? 0 : -100;
}
