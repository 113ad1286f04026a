// Token sampling on the device: repeat penalty -> temperature -> top-k -> softmax -> top-p -> draw, one CTA per row
// of fp32 logits, so a non-greedy decode step stays one CUDA-graph replay with no logits read-back.
//
// Pipeline and its order follow the sampler specification (docs/new/RONN-Llama-Branch-Prompt.md:1011-1116); the
// reference has no sampler code.  Nothing is sorted:
//   * top-k     the k-th largest logit is found by a 4-pass radix select over order-preserving 32-bit keys
//               (one 256-bin histogram in shared memory per pass); ties at the threshold are all kept
//   * top-p     a token is kept while the probability mass of the strictly larger tokens is <= top_p; that cut is
//               found by the same radix walk with probability mass in the bins instead of counts
//   * the draw  u in [0, 1) comes from a counter-based hash of (row seed, draw counter); the token is the first
//               index whose running mass (in index order, block-wide scan per 1024-token slab) reaches u * kept mass
// A row whose record sets `use_counter` mixes in a per-row draw counter that lives in device memory and is advanced
// by the kernel, so replays of a captured graph draw fresh numbers from one seed; a caller that supplies a new seed
// per step (the serving engine: seed = f(request seed, tokens generated)) leaves it off, and a request then draws
// the same tokens whatever row of whatever batch it occupies.
// Rows with temperature <= 0 return the arg max (lowest index on ties), penalty applied.
#include <float.h>

#include "common.cuh"

namespace ronn {

constexpr int SAMPLE_THREADS = 1024;

__device__ __forceinline__ uint32_t orderable(float f) {          // larger float <-> larger key
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float from_orderable(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}
__device__ __forceinline__ uint64_t mix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

struct SampleParams {                 // one record per row, 32 bytes
  float temperature, top_p, repeat_penalty;
  int top_k;
  unsigned long long seed;
  int n_recent, use_counter;
};

// logits: [rows, ld] fp32, modified in place (penalty).  recent: [rows, max_recent] token ids the penalty applies to.
// counters: [rows] draw counters (advanced).  out: [rows] sampled tokens.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(float* __restrict__ logits, long ld, int vocab, const SampleParams* __restrict__ params,
              const int* __restrict__ recent, int max_recent, unsigned long long* __restrict__ counters,
              int* __restrict__ out) {
  __shared__ float s_hist[256];
  __shared__ float s_red[32];
  __shared__ float s_f[2];
  __shared__ uint32_t s_u[2];
  __shared__ int s_i[2];
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x, tid = threadIdx.x;
  float* x = logits + long(row) * ld;
  const SampleParams p = params[row];

  // ---- repeat penalty on the set of recent tokens (a token listed twice is penalised once)
  if (p.repeat_penalty != 1.f && p.n_recent > 0) {
    const int* rec = recent + long(row) * max_recent;
    const int n = min(p.n_recent, max_recent);
    for (int j = tid; j < n; j += blockDim.x) {
      const int t = rec[j];
      if (t < 0 || t >= vocab) continue;
      bool first = true;
      for (int e = 0; e < j; ++e)
        if (rec[e] == t) { first = false; break; }
      if (first) {
        const float v = x[t];
        x[t] = v > 0.f ? v / p.repeat_penalty : v * p.repeat_penalty;
      }
    }
    __syncthreads();
  }

  // ---- arg max (also the greedy answer and the softmax shift)
  float best = -FLT_MAX;
  int best_i = 0x7fffffff;
  for (int i = tid; i < vocab; i += blockDim.x) {
    const float v = x[i];
    if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
  }
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
  }
  __shared__ float s_bv[32];
  __shared__ int s_bi[32];
  if ((tid & 31) == 0) { s_bv[tid >> 5] = best; s_bi[tid >> 5] = best_i; }
  __syncthreads();
  if (tid < 32) {
    best = tid < (blockDim.x >> 5) ? s_bv[tid] : -FLT_MAX;
    best_i = tid < (blockDim.x >> 5) ? s_bi[tid] : 0x7fffffff;
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (tid == 0) { s_f[0] = best; s_i[0] = best_i; }
  }
  __syncthreads();
  const float xmax = s_f[0];
  if (p.temperature <= 0.f) {
    if (tid == 0) out[row] = s_i[0];
    return;
  }
  const float inv_t = 1.f / p.temperature;

  // ---- top-k: key of the k-th largest logit (radix select, most significant byte first)
  uint32_t kth_key = 0;                                   // keep everything by default
  if (p.top_k > 0 && p.top_k < vocab) {
    uint32_t prefix = 0, mask = 0;
    int want = p.top_k;                                   // rank (1 = largest) still to be located inside the prefix
    for (int shift = 24; shift >= 0; shift -= 8) {
      if (tid < 256) s_hist[tid] = 0.f;
      __syncthreads();
      for (int i = tid; i < vocab; i += blockDim.x) {
        const uint32_t k = orderable(x[i]);
        if ((k & mask) == prefix) atomicAdd(&s_hist[(k >> shift) & 255u], 1.f);
      }
      __syncthreads();
      if (tid == 0) {
        int acc = 0, b = 255;
        for (; b > 0; --b) {                              // walk from the largest byte value down
          const int c = int(s_hist[b]);
          if (acc + c >= want) break;
          acc += c;
        }
        s_u[0] = uint32_t(b);
        s_i[1] = want - acc;
      }
      __syncthreads();
      prefix |= s_u[0] << shift;
      mask |= 255u << shift;
      want = s_i[1];
      __syncthreads();
    }
    kth_key = prefix;
  }

  // ---- softmax mass of the kept tokens
  float sum = 0.f;
  for (int i = tid; i < vocab; i += blockDim.x) {
    const float v = x[i];
    if (orderable(v) >= kth_key) sum += __expf((v - xmax) * inv_t);
  }
  const float total = block_sum(sum, s_red);

  // ---- top-p: smallest key such that the mass of strictly larger keys is <= top_p * total
  uint32_t cut_key = kth_key;
  float kept = total;
  if (p.top_p < 1.f) {
    const float budget = p.top_p * total;
    uint32_t prefix = 0, mask = 0;
    float above = 0.f;                                    // mass of keys known to be larger than every key in the prefix
    for (int shift = 24; shift >= 0; shift -= 8) {
      if (tid < 256) s_hist[tid] = 0.f;
      __syncthreads();
      for (int i = tid; i < vocab; i += blockDim.x) {
        const float v = x[i];
        const uint32_t k = orderable(v);
        if (k >= kth_key && (k & mask) == prefix) atomicAdd(&s_hist[(k >> shift) & 255u], __expf((v - xmax) * inv_t));
      }
      __syncthreads();
      if (tid == 0) {
        float acc = above;
        int b = 255;
        for (; b > 0; --b) {
          if (acc + s_hist[b] > budget) break;           // the cut lies inside this bin
          acc += s_hist[b];
        }
        s_u[0] = uint32_t(b);
        s_f[1] = acc;
      }
      __syncthreads();
      prefix |= s_u[0] << shift;
      mask |= 255u << shift;
      above = s_f[1];
      __syncthreads();
    }
    cut_key = prefix > kth_key ? prefix : kth_key;
    // every token whose key equals the cut is kept (the first one always is: the mass above the maximum is 0)
    float s2 = 0.f;
    for (int i = tid; i < vocab; i += blockDim.x) {
      const float v = x[i];
      if (orderable(v) >= cut_key) s2 += __expf((v - xmax) * inv_t);
    }
    kept = block_sum(s2, s_red);
  }

  // ---- the draw
  unsigned long long ctr = 0;
  if (tid == 0) {
    if (p.use_counter) {
      ctr = counters[row];
      counters[row] = ctr + 1;
    }
    const uint64_t h = mix64(mix64(p.seed) + 0xD1B54A32D192ED03ull * ctr);
    s_f[0] = float(h >> 40) * (1.f / 16777216.f) * kept;   // 24 random bits -> [0, kept)
    s_i[0] = -1;
    s_i[1] = best_i;                                       // fallback: rounding left the target above the last slab
  }
  __syncthreads();
  const float target = s_f[0];
  float carried = 0.f;
  for (int base = 0; base < vocab; base += blockDim.x) {
    const int i = base + tid;
    float m = 0.f;
    if (i < vocab) {
      const float v = x[i];
      if (orderable(v) >= cut_key) m = __expf((v - xmax) * inv_t);
    }
    // inclusive scan of the slab: warp scan, then the warp totals
    float incl = m;
    for (int o = 1; o < 32; o <<= 1) {
      const float t = __shfl_up_sync(0xffffffffu, incl, o);
      if ((tid & 31) >= o) incl += t;
    }
    __syncthreads();
    if ((tid & 31) == 31) s_red[tid >> 5] = incl;
    __syncthreads();
    float warp_base = 0.f;
    for (int w = 0; w < (tid >> 5); ++w) warp_base += s_red[w];
    const float upto = carried + warp_base + incl;
    if (m > 0.f && upto > target && upto - m <= target) atomicCAS(&s_i[0], -1, i);
    float slab = 0.f;
    for (int w = 0; w < (blockDim.x >> 5); ++w) slab += s_red[w];
    carried += slab;
    __syncthreads();
    if (s_i[0] >= 0) break;
  }
  if (tid == 0) out[row] = s_i[0] >= 0 ? s_i[0] : s_i[1];
}

}  // namespace ronn

using namespace ronn;

// params: rows records of {float temperature, top_p, repeat_penalty; int top_k; uint64 seed; int n_recent, use_counter}.
extern "C" int ronn_sample(float* logits, long ld, int vocab, long rows, const void* params, const int* recent,
                           int max_recent, unsigned long long* counters, int* out, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0 || ld < vocab || params == nullptr || counters == nullptr || out == nullptr) return -1;
  cudaError_t err = launch(sample_kernel, dim3(unsigned(rows)), dim3(SAMPLE_THREADS), 0, stream, logits, ld, vocab,
                           static_cast<const SampleParams*>(params), recent, max_recent, counters, out);
  return (err == cudaSuccess && cudaGetLastError() == cudaSuccess) ? 0 : -100;
}
