// Small device helpers shared by the memory-bound kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ronn {

// ---- programmatic dependent launch ------------------------------------------------------------------
// A kernel launched through ronn::launch may start while its predecessor in the stream is still draining.
// pdl_wait() blocks until the predecessor has completed and its writes are visible (a no-op for a normal
// launch); everything a kernel does before it must not touch data the predecessor produces or reads.
// pdl_trigger() lets the successor begin launching once every CTA has called it or exited.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

bool pdl_enabled();          // defined in elementwise.cu; RONN_PDL=0 disables

// With RONN_MAX_SHARED_CARVEOUT=1 every kernel asks for the largest shared-memory carve-out.  The tensor-core kernels
// need 80-200 KB per CTA; a small kernel that left its SM configured for a large L1 keeps their CTAs off that SM until
// it has drained, which serialises kernels that run on concurrent streams (measured: 9 % on an attention chain run
// beside a GEMM chain).  Off by default: on a single stream the attention kernel is 1-2 % faster with the larger L1.
// Done once per kernel function.
void prefer_max_shared(const void* kern);      // defined in elementwise.cu

// Launch attributes set with cudaFuncSetAttribute and the SM count belong to a DEVICE, not to the process: launchers
// keep one flag per device ordinal, so a process that drives several GPUs configures its kernels on each of them.
constexpr int MAX_DEVICES = 64;
inline bool first_use_on_device(bool (&seen)[MAX_DEVICES]) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return true;
  if (seen[dev]) return false;
  seen[dev] = true;
  return true;
}
inline int device_sm_count() {
  static int n[MAX_DEVICES] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) dev = 0;
  if (n[dev] == 0 &&
      (cudaDeviceGetAttribute(&n[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n[dev] <= 0))
    n[dev] = 148;
  return n[dev];
}

template <class... KArgs, class... Args>
inline cudaError_t launch(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                          Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  prefer_max_shared(reinterpret_cast<const void*>(kern));
  return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

template <class T> struct Cvt;
template <> struct Cvt<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};
template <> struct Cvt<__half> {
  static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
};
template <> struct Cvt<float> {
  static __device__ __forceinline__ float to_f(float v) { return v; }
  static __device__ __forceinline__ float from_f(float v) { return v; }
};

// 16-byte vector of eight 16-bit values
struct alignas(16) Vec8 {
  uint32_t w[4];
};

// Two 16-bit values in one 32-bit word <-> two floats, on register values (no 16-bit memory accesses).
template <class T> struct Pair16;
template <> struct Pair16<__nv_bfloat16> {
  static __device__ __forceinline__ void unpack(uint32_t w, float& lo, float& hi) {
    lo = __uint_as_float(w << 16);
    hi = __uint_as_float(w & 0xffff0000u);
  }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
};
template <> struct Pair16<__half> {
  static __device__ __forceinline__ void unpack(uint32_t w, float& lo, float& hi) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
    lo = f.x;
    hi = f.y;
  }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
};

// `v` may live in registers, global or shared memory: it is read with ONE 16-byte access (reading its 16-bit fields
// one by one from shared memory costs eight 2-byte loads with four-way bank conflicts each).
template <class T>
__device__ __forceinline__ void unpack8(const Vec8& v, float (&f)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(&v);
  Pair16<T>::unpack(raw.x, f[0], f[1]);
  Pair16<T>::unpack(raw.y, f[2], f[3]);
  Pair16<T>::unpack(raw.z, f[4], f[5]);
  Pair16<T>::unpack(raw.w, f[6], f[7]);
}
template <class T>
__device__ __forceinline__ Vec8 pack8(const float (&f)[8]) {
  Vec8 v;
  v.w[0] = Pair16<T>::pack(f[0], f[1]);
  v.w[1] = Pair16<T>::pack(f[2], f[3]);
  v.w[2] = Pair16<T>::pack(f[4], f[5]);
  v.w[3] = Pair16<T>::pack(f[6], f[7]);
  return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide reductions for blocks of up to 1024 threads; `scratch` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = (lane < nw) ? scratch[lane] : 0.f;
  return warp_sum(r);
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = (lane < nw) ? scratch[lane] : -INFINITY;
  return warp_max(r);
}

__device__ __forceinline__ float gelu_tanh_f(float x) {
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  const float e = __expf(2.f * u);
  const float t = 1.f - 2.f / (e + 1.f);       // tanh(u), saturates correctly at +-inf
  return 0.5f * x * (1.f + t);
}

}  // namespace ronn
