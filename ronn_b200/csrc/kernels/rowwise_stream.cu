// Row-wise kernels for many rows (prefill- and encoder-sized activations): LayerNorm / RMSNorm (+ residual), softmax,
// per-token int8 quantisation and RMSNorm + quantisation.
//
// With thousands of rows these ops are pure HBM streams, and the one-row-per-CTA kernels used for decode keep only
// as many bytes in flight as fit in registers (about 35 KB per SM), which is less than bandwidth x latency on this
// part.  Here every warp owns a ring of row buffers in shared memory that the bulk-copy engine fills
// (cp.async.bulk global -> shared, completion on an mbarrier), so up to 190 KB per SM are in flight whatever the
// register budget, and the row is re-read from shared memory for each pass (statistics, normalise) instead of being held
// in registers.  One warp per row; a row of H 16-bit values must be 16-byte aligned with H % 8 == 0.
//
// Replaces, for large row counts, the per-node library calls of the reference GPU provider
// (crates/ronn-providers/src/gpu/provider.rs:1376-1408 LayerNorm chain, crates/ronn-core/src/ops/reduction.rs:432-450
// softmax) and the BitNet activation quantiser (crates/ronn-providers/src/bitnet/kernels.rs:277-278).
#include "common.cuh"
#include "ptx_sm100.cuh"
#include "rowwise_stream.h"

namespace ronn {

constexpr int RS_WARPS = 8;
constexpr int RS_MAX_STAGES = 8;
constexpr uint32_t RS_WAIT_CODE = 0x5201u;      // status value: a row load never completed

// Status word of the process for each device (set once by the host library with ronn_set_rowwise_status): the
// launchers of these kernels have no status parameter of their own.
static uint32_t* g_status_ptr[64] = {};

struct RowArgs {
  const void* x;
  const void* res;
  const void* gamma;
  const void* beta;
  void* y;
  void* sum_out;
  float* scale_out;
  uint32_t* status;
  long rows, ld_x, ld_res, ld_y;
  int H, stages;
  float eps;
};

__device__ __forceinline__ void bulk_load_row(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// MODE: 0 LayerNorm, 1 RMSNorm, 2 softmax, 3 per-row absmax int8 quantisation, 4 RMSNorm * gamma then quantisation.
template <class T, int MODE, bool HAS_RES>
__global__ void __launch_bounds__(RS_WARPS * 32, 4) rowwise_stream_kernel(const RowArgs a) {
  extern __shared__ __align__(128) uint8_t rs_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int S = a.stages;
  const uint32_t row_bytes = uint32_t(a.H) * sizeof(T);
  const uint32_t slot_bytes = row_bytes * (HAS_RES ? 2u : 1u);
  uint8_t* ring = rs_smem + size_t(warp) * S * slot_bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(rs_smem + size_t(RS_WARPS) * S * slot_bytes) + warp * RS_MAX_STAGES;
  volatile uint32_t* abort_flag =
      reinterpret_cast<volatile uint32_t*>(rs_smem + size_t(RS_WARPS) * S * slot_bytes + RS_WARPS * RS_MAX_STAGES * 8);
  if (threadIdx.x == 0) *abort_flag = 0;
  if (lane == 0) {
    for (int s = 0; s < S; ++s) mbar_init(&bars[s], 1);
    mbar_fence_init();
  }
  __syncthreads();
  pdl_wait();
  pdl_trigger();

  const long total = long(gridDim.x) * RS_WARPS;
  const long first = long(blockIdx.x) * RS_WARPS + warp;
  const T* x = static_cast<const T*>(a.x);
  const T* res = static_cast<const T*>(a.res);
  auto issue = [&](long row, int stage) {
    uint8_t* dst = ring + size_t(stage) * slot_bytes;
    mbar_expect_tx(&bars[stage], slot_bytes);
    bulk_load_row(dst, x + row * a.ld_x, row_bytes, &bars[stage]);
    if (HAS_RES) bulk_load_row(dst + row_bytes, res + row * a.ld_res, row_bytes, &bars[stage]);
  };
  if (lane == 0) {
    for (int s = 0; s < S; ++s) {
      const long row = first + s * total;
      if (row < a.rows) issue(row, s);
    }
  }
  __syncwarp();

  const int nchunk = a.H >> 3;
  const float inv_h = 1.f / float(a.H);
  const T* gamma = static_cast<const T*>(a.gamma);
  const T* beta = static_cast<const T*>(a.beta);
  long it = 0;
  bool ok = true;
  for (long row = first; row < a.rows; row += total, ++it) {
    const int stage = int(it % S);
    if (!mbar_wait(&bars[stage], uint32_t(it / S) & 1u, abort_flag, a.status, RS_WAIT_CODE)) {
      ok = false;
      break;
    }
    Vec8* xs = reinterpret_cast<Vec8*>(ring + size_t(stage) * slot_bytes);
    const Vec8* rs = reinterpret_cast<const Vec8*>(ring + size_t(stage) * slot_bytes + row_bytes);

    if (MODE == 0 || MODE == 1) {
      T* y = static_cast<T*>(a.y) + row * a.ld_y;
      T* so = a.sum_out ? static_cast<T*>(a.sum_out) + row * a.ld_y : nullptr;
      // One pass over the row for the statistics.  LayerNorm accumulates sum and sum of squares of (v - shift) with
      // the row's first value as the shift, so that var = E[(v - shift)^2] - (E[v - shift])^2 does not cancel when the
      // mean is large against the spread (the kernel is bound by instruction issue: a separate pass for the squared
      // deviations costs a shared-memory read and a conversion per value).
      float shift = 0.f;
      if (MODE == 0) {
        float first[8];
        unpack8<T>(xs[0], first);
        shift = first[0];
        if (HAS_RES) {
          unpack8<T>(rs[0], first);
          shift += first[0];
        }
      }
      float s = 0.f, s2 = 0.f;
#pragma unroll 4
      for (int c = lane; c < nchunk; c += 32) {
        float v[8];
        unpack8<T>(xs[c], v);
        if (HAS_RES) {
          float r[8];
          unpack8<T>(rs[c], r);
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] += r[i];
          const Vec8 pk = pack8<T>(v);            // the residual stream stores this rounding; normalise the same values
          if (so) *reinterpret_cast<Vec8*>(so + c * 8) = pk;
          xs[c] = pk;
          unpack8<T>(pk, v);
        } else if (so) {
          *reinterpret_cast<Vec8*>(so + c * 8) = xs[c];
        }
        if (MODE == 1) {
#pragma unroll
          for (int i = 0; i < 8; ++i) s2 = fmaf(v[i], v[i], s2);
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float d = v[i] - shift;
            s += d;
            s2 = fmaf(d, d, s2);
          }
        }
      }
      float mean = 0.f, inv;
      if (MODE == 1) {
        inv = rsqrtf(warp_sum(s2) * inv_h + a.eps);
      } else {
        const float d = warp_sum(s) * inv_h;
        const float var = fmaxf(warp_sum(s2) * inv_h - d * d, 0.f);
        mean = shift + d;
        inv = rsqrtf(var + a.eps);
      }
#pragma unroll 4
      for (int c = lane; c < nchunk; c += 32) {
        float v[8], g[8], b[8], o[8];
        unpack8<T>(xs[c], v);
        if (gamma) unpack8<T>(*reinterpret_cast<const Vec8*>(gamma + c * 8), g);
        if (beta) unpack8<T>(*reinterpret_cast<const Vec8*>(beta + c * 8), b);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float t = (v[i] - mean) * inv;
          if (gamma) t *= g[i];
          if (beta) t += b[i];
          o[i] = t;
        }
        *reinterpret_cast<Vec8*>(y + c * 8) = pack8<T>(o);
      }
    } else if (MODE == 2) {
      T* y = static_cast<T*>(a.y) + row * a.ld_y;
      float m = -INFINITY;
#pragma unroll 4
      for (int c = lane; c < nchunk; c += 32) {
        float v[8];
        unpack8<T>(xs[c], v);
#pragma unroll
        for (int i = 0; i < 8; ++i) m = fmaxf(m, v[i]);
      }
      m = warp_max(m);
      float s = 0.f;
#pragma unroll 4
      for (int c = lane; c < nchunk; c += 32) {
        float v[8];
        unpack8<T>(xs[c], v);
#pragma unroll
        for (int i = 0; i < 8; ++i) s += __expf(v[i] - m);
      }
      const float inv = 1.f / warp_sum(s);
#pragma unroll 4
      for (int c = lane; c < nchunk; c += 32) {
        float v[8], o[8];
        unpack8<T>(xs[c], v);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = __expf(v[i] - m) * inv;
        *reinterpret_cast<Vec8*>(y + c * 8) = pack8<T>(o);
      }
    } else {
      int8_t* q = static_cast<int8_t*>(a.y) + row * a.ld_y;
      float m = 0.f;
      if (MODE == 4) {
        float ss = 0.f;
#pragma unroll 4
        for (int c = lane; c < nchunk; c += 32) {
          float v[8];
          unpack8<T>(xs[c], v);
#pragma unroll
          for (int i = 0; i < 8; ++i) ss += v[i] * v[i];
        }
        const float inv = rsqrtf(warp_sum(ss) * inv_h + a.eps);
#pragma unroll 4
        for (int c = lane; c < nchunk; c += 32) {
          float v[8], g[8];
          unpack8<T>(xs[c], v);
          unpack8<T>(*reinterpret_cast<const Vec8*>(gamma + c * 8), g);
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = v[i] * inv * g[i];
          const Vec8 pk = pack8<T>(v);            // rounded through the storage type, like norm-then-quantise
          xs[c] = pk;
          unpack8<T>(pk, v);
#pragma unroll
          for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(v[i]));
        }
      } else {
#pragma unroll 4
        for (int c = lane; c < nchunk; c += 32) {
          float v[8];
          unpack8<T>(xs[c], v);
#pragma unroll
          for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(v[i]));
        }
      }
      m = fmaxf(warp_max(m), 1e-5f);
      const float qs = __fdiv_rn(127.f, m);       // IEEE division: bit-identical to the host quantiser
#pragma unroll 4
      for (int c = lane; c < nchunk; c += 32) {
        float v[8];
        unpack8<T>(xs[c], v);
        // round(v * qs) clamped to [-127, 127], without the conversion instructions (they run on the special-function
        // unit at a quarter of the FMA rate and bounded this pass): adding 1.5 * 2^23 rounds to the nearest integer,
        // ties to even like rintf, and leaves that integer in the low mantissa bits, whose low byte is the int8 value.
        uint32_t bits[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float p = fminf(fmaxf(__fmul_rn(v[i], qs), -127.f), 127.f);
          bits[i] = __float_as_uint(__fadd_rn(p, 12582912.f));
        }
        int2 packed;
        packed.x = int(__byte_perm(__byte_perm(bits[0], bits[1], 0x0040), __byte_perm(bits[2], bits[3], 0x0040), 0x5410));
        packed.y = int(__byte_perm(__byte_perm(bits[4], bits[5], 0x0040), __byte_perm(bits[6], bits[7], 0x0040), 0x5410));
        *reinterpret_cast<int2*>(q + c * 8) = packed;
      }
      if (lane == 0) a.scale_out[row] = __fdiv_rn(m, 127.f);
    }

    // Every lane is done with the slot: hand it back to the copy engine for the row S turns ahead.
    if (HAS_RES || MODE == 4) fence_proxy_async_smem();   // generic-proxy writes to the slot before the async-proxy write
    __syncwarp();
    if (lane == 0) {
      const long next = row + long(S) * total;
      if (next < a.rows) issue(next, stage);
    }
  }

  if (!ok) {
    // A load timed out.  Give the other loads this warp armed a bounded time to land before the CTA (and its shared
    // memory) goes away.
    for (int j = 1; j < S; ++j) {
      const long idx = it + j;
      if (first + idx * total >= a.rows) break;
      uint64_t* bar = &bars[int(idx % S)];
      const uint32_t parity = uint32_t(idx / S) & 1u;
      for (int p = 0; p < (1 << 20); ++p)
        if (mbar_try_wait(bar, parity)) break;
    }
  }
}

template <class T, int MODE, bool HAS_RES>
static int launch_stream(const RowArgs& a, size_t smem, int grid, cudaStream_t stream) {
  auto kern = rowwise_stream_kernel<T, MODE, HAS_RES>;
  static bool configured[MAX_DEVICES] = {false};                 // per instantiation
  if (first_use_on_device(configured)) {
    // The ring of every resident CTA has to fit: ask for the largest shared-memory carve-out, or the driver may
    // size it for a single CTA and leave the SM with eight warps.
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared) !=
            cudaSuccess) {
      cudaGetLastError();
      return -101;
    }
  }
  return launch(kern, dim3(grid), dim3(RS_WARPS * 32), smem, stream, a) == cudaSuccess ? 1 : -100;
}

int rowwise_stream_try(int mode, const void* x, const void* res, const void* gamma, const void* beta, void* y,
                       void* sum_out, float* scale_out, long rows, int H, long ld_x, long ld_res, long ld_y, float eps,
                       int dtype, cudaStream_t stream) {
  static int enabled = -1;
  if (enabled < 0) {
    const char* e = getenv("RONN_ROWWISE_STREAM");
    enabled = (e && e[0] == '0') ? 0 : 1;
  }
  if (!enabled || rows < 2048 || (dtype != 0 && dtype != 1) || (H & 7) || H < 64) return 0;
  if ((ld_x & 7) || (res && (ld_res & 7))) return 0;
  const bool quant = mode >= 3;
  if (!quant && (ld_y & 7)) return 0;
  if (quant && (ld_y & 7)) return 0;
  auto misaligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) != 0; };
  if (misaligned(x) || (res && misaligned(res)) || misaligned(y) || (sum_out && misaligned(sum_out)) ||
      (gamma && misaligned(gamma)) || (beta && misaligned(beta)))
    return 0;
  if (mode == 4 && !gamma) return 0;
  const size_t slot = size_t(H) * 2 * (res ? 2 : 1);
  // Many warps with short rings rather than few warps with long ones: the bytes in flight are the same (ring bytes
  // per SM), and the warps hide each other's reduction latency.
  int stages = int((48 * 1024) / (RS_WARPS * slot));
  if (stages > RS_MAX_STAGES) stages = RS_MAX_STAGES;
  if (stages < 2) stages = 2;
  const size_t smem = RS_WARPS * stages * slot + RS_WARPS * RS_MAX_STAGES * 8 + 16;
  if (smem > 200 * 1024) return 0;
  int per_sm = int((224 * 1024) / (smem + 1024));
  if (per_sm > 4) per_sm = 4;                   // register file: 256 threads x 64 registers x 4
  if (per_sm < 1) per_sm = 1;
  long grid = (rows + RS_WARPS - 1) / RS_WARPS;
  if (grid > 148l * per_sm) grid = 148l * per_sm;
  int dev = 0;
  cudaGetDevice(&dev);
  uint32_t* status = (dev >= 0 && dev < 64) ? g_status_ptr[dev] : nullptr;
  RowArgs a{x, res, gamma, beta, y, sum_out, scale_out, status, rows, ld_x, ld_res, ld_y, H, stages, eps};
#define RS_GO(T_)                                                                                       \
  switch (mode) {                                                                                       \
    case 0: return res ? launch_stream<T_, 0, true>(a, smem, int(grid), stream)                         \
                       : launch_stream<T_, 0, false>(a, smem, int(grid), stream);                       \
    case 1: return res ? launch_stream<T_, 1, true>(a, smem, int(grid), stream)                         \
                       : launch_stream<T_, 1, false>(a, smem, int(grid), stream);                       \
    case 2: return res ? 0 : launch_stream<T_, 2, false>(a, smem, int(grid), stream);                   \
    case 3: return res ? 0 : launch_stream<T_, 3, false>(a, smem, int(grid), stream);                   \
    case 4: return res ? 0 : launch_stream<T_, 4, false>(a, smem, int(grid), stream);                   \
    default: return 0;                                                                                  \
  }
  if (dtype == 0) { RS_GO(__nv_bfloat16) }
  RS_GO(__half)
#undef RS_GO
}

}  // namespace ronn

// Registers the device word that receives 0x5201 when a row load of a streaming row-wise kernel does not complete
// within the wait limit (the first code wins; the host reads and clears the word).  Applies to the current device.
extern "C" int ronn_set_rowwise_status(uint32_t* word) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
  ronn::g_status_ptr[dev] = word;
  return 0;
}
