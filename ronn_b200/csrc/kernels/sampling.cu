// Token sampling on the device: repeat penalty -> temperature -> top-k -> softmax -> top-p -> draw, one CTA per row
// of fp32 logits, so a non-greedy decode step stays one CUDA-graph replay with no logits read-back.
//
// Pipeline and its order follow the sampler specification (docs/new/RONN-Llama-Branch-Prompt.md:1011-1116); the
// reference has no sampler code.  Nothing is sorted:
//   * top-k     the k-th largest logit is found by a 4-pass radix select over order-preserving 32-bit keys
//               (256-bin histograms in shared memory); ties at the threshold are all kept.  Logits cluster in a
//               handful of bins and same-address shared-memory atomics serialise, so a warp groups its lanes by bin
//               (one match instruction), sums a group with one warp-reduce instruction and issues ONE atomic per
//               distinct bin, on one of eight histogram copies; probability mass travels as 2^-26 fixed point so that
//               the integer reduce applies; the walk over the 256 bins is a warp scan, not a serial loop
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

constexpr int HIST_COPIES = 8;
constexpr float MASS_SCALE = 67108864.f;               // 2^26: a warp's 32 fixed-point masses (each <= 1) sum below 2^32

// Adds `amount` (a fixed-point mass, MASS) or 1 (counts) to bin `bin` of `hist` for every active lane.  The lanes of a
// warp that share a bin are found with one match instruction, summed with one warp-reduce instruction, and their
// leader issues one atomic.  Must be called by all 32 lanes.
template <bool MASS>
__device__ __forceinline__ void hist_add(unsigned long long* hist, uint32_t bin, uint32_t amount, bool active) {
  const int lane = threadIdx.x & 31;
  if (__ballot_sync(0xffffffffu, active) == 0u) return;         // later radix levels: most warps see no candidate
  const unsigned grp = __match_any_sync(0xffffffffu, active ? bin : 0xffffffffu);
  uint32_t s;
  if (MASS) s = __reduce_add_sync(grp, active ? amount : 0u);
  else s = uint32_t(__popc(grp));
  if (active && lane == __ffs(grp) - 1) atomicAdd(&hist[bin], (unsigned long long)s);
}

// Sums the histogram copies into `binf` as floats (value * scale); all threads, ends with a barrier.
__device__ __forceinline__ void hist_merge(const unsigned long long* hist, float* binf, float scale) {
  __syncthreads();
  if (threadIdx.x < 256) {
    unsigned long long t = 0;
#pragma unroll
    for (int c = 0; c < HIST_COPIES; ++c) t += hist[c * 256 + threadIdx.x];
    binf[threadIdx.x] = float(t) * scale;
  }
  __syncthreads();
}
__device__ __forceinline__ void hist_clear(unsigned long long* hist) {
  for (int i = threadIdx.x; i < HIST_COPIES * 256; i += blockDim.x) hist[i] = 0ull;
  __syncthreads();
}

// Walk from bin 255 down: the first bin b >= 1 at which the running sum `acc` (of the bins above it, starting at
// `start`) satisfies STRICT ? acc + hist[b] > limit : acc + hist[b] >= limit; bin 0 if none does.  Returns the bin
// and the sum of the bins above it through `acc_out`.  Warp 0 computes (a scan over 8 bins per lane), everybody gets
// the answer; contains barriers.
template <bool STRICT>
__device__ __forceinline__ uint32_t hist_walk(const float* hist, float start, float limit, float* acc_out, float* s_f,
                                              uint32_t* s_u) {
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    float c[8], tot = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      c[j] = hist[255 - (8 * lane + j)];
      tot += c[j];
    }
    float incl = tot;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    float acc = start + incl - tot;                  // sum of the bins above this lane's first bin
    int hit = -1;
    float acc_at = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int rb = 8 * lane + j;
      const bool cond = STRICT ? (acc + c[j] > limit) : (acc + c[j] >= limit);
      if (hit < 0 && rb < 255 && cond) {
        hit = rb;
        acc_at = acc;
      }
      if (rb < 255) acc += c[j];
    }
    const unsigned m = __ballot_sync(0xffffffffu, hit >= 0);
    const int src = m ? __ffs(m) - 1 : 31;           // no hit: lane 31 holds the sum of bins 255..1 in `acc`
    hit = __shfl_sync(0xffffffffu, m ? hit : 255, src);
    acc_at = __shfl_sync(0xffffffffu, m ? acc_at : acc, src);
    if (lane == 0) {
      s_u[0] = uint32_t(255 - hit);
      s_f[1] = acc_at;
    }
  }
  __syncthreads();
  const uint32_t b = s_u[0];
  *acc_out = s_f[1];
  __syncthreads();
  return b;
}

struct SampleParams {                 // one record per row, 32 bytes
  float temperature, top_p, repeat_penalty;
  int top_k;
  unsigned long long seed;
  int n_recent, use_counter;
};

// Visits every element of the row: f(index, value, valid) is called by ALL threads the same number of times (the
// histogram updates are warp collectives), `valid` false past the end.  Eight loads per thread are in flight at a
// time: a pass whose every iteration waits for one load from L2 took 11 us for 50 K logits, this form 1.5 us.
template <class F>
__device__ __forceinline__ void for_each_logit(const float* __restrict__ x, int vocab, F f) {
  constexpr int U = 8;
  const int tid = threadIdx.x, n = blockDim.x;
  for (int base = 0; base < vocab; base += U * n) {
    float v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = base + u * n + tid;
      v[u] = i < vocab ? x[i] : 0.f;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = base + u * n + tid;
      f(i, v[u], i < vocab);
    }
  }
}

// First radix level without a histogram.  The top byte of a key is the sign and the upper exponent bits, so the
// candidates of top-k / top-p sit in the bin of the row maximum or just below it: every thread keeps the count (or the
// probability mass) of the four bins from the maximum's down and of everything below in registers, and five block sums
// replace ~50 K histogram updates.  c[j]: bin (bmax - j), c[4]: the rest.  Only keys >= min_key take part.
template <bool MASS>
__device__ __forceinline__ void top_bins(const float* __restrict__ x, int vocab, uint32_t bmax, uint32_t min_key, float xmax,
                                         float inv_t, float (&c)[5], float* s_red) {
  float t[5] = {0.f, 0.f, 0.f, 0.f, 0.f};
  for_each_logit(x, vocab, [&](int, float v, bool valid) {
    const uint32_t k = orderable(v);
    if (valid && k >= min_key) {
      const float w = MASS ? __expf((v - xmax) * inv_t) : 1.f;
      const uint32_t d = bmax - (k >> 24);
#pragma unroll
      for (int j = 0; j < 4; ++j) t[j] += d == uint32_t(j) ? w : 0.f;
      t[4] += d >= 4u ? w : 0.f;
    }
  });
#pragma unroll
  for (int j = 0; j < 5; ++j) c[j] = block_sum(t[j], s_red);
}

// logits: [rows, ld] fp32, modified in place (penalty).  recent: [rows, max_recent] token ids the penalty applies to.
// counters: [rows] draw counters (advanced).  out: [rows] sampled tokens.
// STAGED: the row (after the penalty) is copied into shared memory once and every later sweep reads it there; the
// launcher picks it when the vocabulary fits (about 51 K tokens).  A sweep from L2 costs ~12 K cycles, from shared
// memory ~2 K (more when most elements update a histogram).  Sweeps: arg max + copy, four top-k levels, four top-p
// levels (the first also yields the total mass, the last the kept mass), the draw.
template <bool STAGED>
__global__ void __launch_bounds__(SAMPLE_THREADS, 1)
sample_kernel(float* __restrict__ logits, long ld, int vocab, const SampleParams* __restrict__ params,
              const int* __restrict__ recent, int max_recent, unsigned long long* __restrict__ counters,
              int* __restrict__ out) {
  extern __shared__ float s_row[];
  __shared__ unsigned long long s_hist[HIST_COPIES * 256];
  __shared__ float s_binf[256];
  __shared__ float s_red[32];
  __shared__ float s_f[2];
  __shared__ uint32_t s_u[2];
  __shared__ int s_i[2];
  __shared__ float s_bv[32];
  __shared__ int s_bi[32];
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float* xg = logits + long(row) * ld;
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
        const float v = xg[t];
        xg[t] = v > 0.f ? v / p.repeat_penalty : v * p.repeat_penalty;
      }
    }
    __syncthreads();
  }
  const bool sampled = p.temperature > 0.f;
  const bool use_top_k = sampled && p.top_k > 0 && p.top_k < vocab;
  unsigned long long* my_hist = s_hist + (warp & (HIST_COPIES - 1)) * 256;

  // ---- first sweep (from global memory): arg max (the greedy answer and the softmax shift) and the copy into
  // shared memory
  float best = -FLT_MAX;
  int best_i = 0x7fffffff;
  for_each_logit(xg, vocab, [&](int i, float v, bool valid) {
    if (valid && (v > best || (v == best && i < best_i))) { best = v; best_i = i; }
    if (STAGED && valid) s_row[i] = v;
  });
  const float* x = STAGED ? s_row : xg;
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
  }
  if (lane == 0) { s_bv[warp] = best; s_bi[warp] = best_i; }
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
  const int arg_max = s_i[0];
  if (!sampled) {
    if (tid == 0) out[row] = arg_max;
    return;
  }
  __syncthreads();                                        // s_f / s_i are reused below
  const float inv_t = 1.f / p.temperature;
  const uint32_t bmax = orderable(xmax) >> 24;

  // ---- top-k: key of the k-th largest logit (radix select, most significant byte first)
  uint32_t kth_key = 0;                                   // keep everything by default
  if (use_top_k) {
    uint32_t prefix = 0, mask = 0;
    int want = p.top_k;                                   // rank (1 = largest) still to be located inside the prefix
    int first_shift = 24;
    {
      float c[5];
      top_bins<false>(x, vocab, bmax, 0u, xmax, inv_t, c, s_red);
      float acc = 0.f;
      for (int j = 0; j < 4 && first_shift == 24; ++j) {
        if (acc + c[j] >= float(want) && bmax >= uint32_t(j)) {
          prefix = (bmax - uint32_t(j)) << 24;
          mask = 255u << 24;
          want -= int(acc);
          first_shift = 16;
        }
        acc += c[j];
      }
    }
    for (int shift = first_shift; shift >= 0; shift -= 8) {      // from 24 only if the rank lies below the four top bins
      hist_clear(s_hist);
      for_each_logit(x, vocab, [&](int, float v, bool valid) {
        const uint32_t k = orderable(v);
        hist_add<false>(my_hist, (k >> shift) & 255u, 0u, valid && (k & mask) == prefix);
      });
      hist_merge(s_hist, s_binf, 1.f);
      float above;
      const uint32_t b = hist_walk<false>(s_binf, 0.f, float(want), &above, s_f, s_u);
      prefix |= b << shift;
      mask |= 255u << shift;
      want -= int(above);
    }
    kth_key = prefix;
  }

  // ---- top-p: smallest key such that the mass of strictly larger keys is <= top_p * (mass of the kept tokens).
  // The first level's bins add up to that mass; at the last level a bin is one key, so the bin of the cut plus
  // everything above it is the mass that stays.  Without top-p one sweep sums the mass.
  uint32_t cut_key = kth_key;
  float kept;
  if (p.top_p < 1.f) {
    uint32_t prefix = 0, mask = 0;
    float above = 0.f, budget = 0.f, cut_bin = 0.f;       // above: mass of keys larger than every key in the prefix
    int first_shift = 24;
    {
      float c[5];
      top_bins<true>(x, vocab, bmax, kth_key, xmax, inv_t, c, s_red);
      const float total = c[0] + c[1] + c[2] + c[3] + c[4];
      float acc = 0.f;
      for (int j = 0; j < 4 && first_shift == 24; ++j) {
        if (acc + c[j] > p.top_p * total && bmax >= uint32_t(j)) {
          prefix = (bmax - uint32_t(j)) << 24;
          mask = 255u << 24;
          above = acc;
          cut_bin = c[j];
          budget = p.top_p * total;
          first_shift = 16;
        }
        acc += c[j];
      }
    }
    for (int shift = first_shift; shift >= 0; shift -= 8) {      // from 24 only if the cut lies below the four top bins
      hist_clear(s_hist);
      for_each_logit(x, vocab, [&](int, float v, bool valid) {
        const uint32_t k = orderable(v);
        const bool act = valid && k >= kth_key && (k & mask) == prefix;
        const uint32_t m = act ? __float2uint_rn(__expf((v - xmax) * inv_t) * MASS_SCALE) : 0u;
        hist_add<true>(my_hist, (k >> shift) & 255u, m, act);
      });
      hist_merge(s_hist, s_binf, 1.f / MASS_SCALE);
      if (shift == 24) {
        const float t = block_sum(tid < 256 ? s_binf[tid] : 0.f, s_red);
        budget = p.top_p * t;
      }
      const uint32_t b = hist_walk<true>(s_binf, above, budget, &above, s_f, s_u);   // the cut lies inside bin b
      cut_bin = s_binf[b];
      __syncthreads();                                    // s_binf is rewritten by the next level
      prefix |= b << shift;
      mask |= 255u << shift;
    }
    cut_key = prefix > kth_key ? prefix : kth_key;
    // every token whose key equals the cut is kept (the first one always is: the mass above the maximum is 0)
    kept = above + cut_bin;
  } else {
    float sum = 0.f;
    for_each_logit(x, vocab, [&](int, float v, bool valid) {
      if (valid && orderable(v) >= kth_key) sum += __expf((v - xmax) * inv_t);
    });
    kept = block_sum(sum, s_red);
  }

  // ---- the draw: the first index whose running mass (index order) exceeds u * kept.  A thread owns 8 consecutive
  // tokens of a slab of 8 x blockDim; thread totals are scanned across the block, the owner scans its own eight.
  if (tid == 0) {
    unsigned long long ctr = 0;
    if (p.use_counter) {
      ctr = counters[row];
      counters[row] = ctr + 1;
    }
    const uint64_t h = mix64(mix64(p.seed) + 0xD1B54A32D192ED03ull * ctr);
    s_f[0] = float(h >> 40) * (1.f / 16777216.f) * kept;   // 24 random bits -> [0, kept)
    s_i[0] = -1;
  }
  __syncthreads();
  const float target = s_f[0];
  float carried = 0.f;
  constexpr int PER = 8;
  for (int base = 0; base < vocab; base += PER * blockDim.x) {
    const int i0 = base + tid * PER;
    float m[PER], mine = 0.f;
#pragma unroll
    for (int u = 0; u < PER; ++u) {
      const int i = i0 + u;
      const float v = i < vocab ? x[i] : -FLT_MAX;
      m[u] = (i < vocab && orderable(v) >= cut_key) ? __expf((v - xmax) * inv_t) : 0.f;
      mine += m[u];
    }
    float incl = mine;                                    // inclusive scan of the thread totals: warp, then warp totals
    for (int o = 1; o < 32; o <<= 1) {
      const float t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    if (lane == 31) s_red[warp] = incl;
    __syncthreads();
    float wt = lane < (blockDim.x >> 5) ? s_red[lane] : 0.f;       // every warp scans the 32 warp totals itself
    float wincl = wt;
    for (int o = 1; o < 32; o <<= 1) {
      const float t = __shfl_up_sync(0xffffffffu, wincl, o);
      if (lane >= o) wincl += t;
    }
    const float warp_base = __shfl_sync(0xffffffffu, wincl - wt, warp);
    const float slab = __shfl_sync(0xffffffffu, wincl, 31);
    float upto = carried + warp_base + incl - mine;       // mass before this thread's first token
    if (mine > 0.f && upto + mine > target && upto <= target) {
      int pick = -1;
#pragma unroll
      for (int u = 0; u < PER; ++u) {
        if (pick < 0 && m[u] > 0.f && upto + m[u] > target) pick = i0 + u;
        upto += m[u];
      }
      if (pick >= 0) atomicCAS(&s_i[0], -1, pick);
    }
    carried += slab;
    __syncthreads();
    if (s_i[0] >= 0) break;
  }
  // rounding can leave the target at or above the last kept token's running mass: the arg max is always kept
  if (tid == 0) out[row] = s_i[0] >= 0 ? s_i[0] : arg_max;
}

}  // namespace ronn

using namespace ronn;

// params: rows records of {float temperature, top_p, repeat_penalty; int top_k; uint64 seed; int n_recent, use_counter}.
extern "C" int ronn_sample(float* logits, long ld, int vocab, long rows, const void* params, const int* recent,
                           int max_recent, unsigned long long* counters, int* out, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0 || ld < vocab || params == nullptr || counters == nullptr || out == nullptr) return -1;
  // the row is staged in shared memory when it fits beside the kernel's ~18 KB of static shared memory
  const size_t row_bytes = size_t(vocab) * sizeof(float);
  const bool staged = row_bytes <= 200 * 1024;
  cudaError_t err;
  if (staged) {
    static bool configured[MAX_DEVICES] = {false};
    if (first_use_on_device(configured) &&
        cudaFuncSetAttribute(sample_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
      return -10;
    err = launch(sample_kernel<true>, dim3(unsigned(rows)), dim3(SAMPLE_THREADS), row_bytes, stream, logits, ld, vocab,
                 static_cast<const SampleParams*>(params), recent, max_recent, counters, out);
  } else {
    err = launch(sample_kernel<false>, dim3(unsigned(rows)), dim3(SAMPLE_THREADS), 0, stream, logits, ld, vocab,
                 static_cast<const SampleParams*>(params), recent, max_recent, counters, out);
  }
  return (err == cudaSuccess && cudaGetLastError() == cudaSuccess) ? 0 : -100;
}
