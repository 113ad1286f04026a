// Device and host pieces shared by the kernels that end in the low-latency two-phase all-reduce (gemm_ll.cu: bf16 / fp16
// GEMM; bitnet.cu: ternary x int8 BitLinear): the argument block, the scatter of a 32 x 32 accumulator chunk to the row
// owners (phase A), the owner-side reduce + broadcast (phase B) and the unpack + norm (phase C).
#pragma once
#include "comm_ptx.cuh"
#include "common.cuh"
#include "gemm_epilogue.cuh"
#include "gemm_ll.h"
#include "ptx_sm100.cuh"
#include "umma_persistent.cuh"

namespace ronn {

constexpr int LL_MAX_RANKS = RONN_LL_MAX_RANKS;
// The epoch word is 64 bits wide and the CTAs of a call add up to exactly one unit on it, so the call count (and with
// it the sequence number carried by the words on the wire) only repeats after 2^32 calls: a word left in an area by
// an old call of another shape can never be mistaken for current data.
constexpr unsigned long long LL_UNIT = 1ull << 16;

struct LLArgs {
  uint8_t* scatter_peer[LL_MAX_RANKS];   // phase-A receive area of every rank: [2 parities][W sources][owner_rows * N] values, 4 bytes each
  uint8_t* scatter_local;
  uint8_t* result_peer[LL_MAX_RANKS];    // phase-B result area of every rank: [2 parities][M * N] values, 4 bytes each
  uint8_t* result_mc;                    // its multicast address (NVLS) or null
  uint8_t* result_local;
  long scatter_parity_stride, result_parity_stride;   // bytes
  unsigned long long* state;             // [0] epoch word
  void* out;                             // X [M, ld_out], local
  void* norm_out;                        // H, or null
  const void* bias;
  const void* residual;                  // [M, ld_res]; a row is read by its owner only
  const void* gamma;
  const void* beta;
  unsigned long long* trace;
  int8_t* quant_out;                     // norm_mode 3
  float* quant_scale;
  unsigned long long wait_ns;
  long ld_out, ld_res;
  float eps;
  int M, N, rank, world, owner_rows, row_begin, row_end;
  int norm_mode, nvls, wpr, phases;
  int S, kb_per, num_kb;                 // K slices per rank: every (rank, slice) pair is one source of phase A
};

// The call's sequence number and parity offset, from the epoch word (read after the dependency wait).
__device__ __forceinline__ void ll_resolve(const LLArgs& a, uint32_t& seq, size_t& scatter_parity_off) {
  const unsigned long long epoch = *reinterpret_cast<volatile unsigned long long*>(a.state) / LL_UNIT;
  seq = uint32_t(epoch) + 1u;
  if (seq == 0u) seq = 1u;
  scatter_parity_off = size_t(epoch & 1u) * a.scatter_parity_stride;
}

// Phase A for one chunk: row `gm` (this lane's) x 32 columns from `gn` of fp32 values -> 16-bit pairs -> {data, sequence}
// words in the owners' receive areas, source slot `src`.  Called by a whole warp whose lanes hold 32 consecutive rows
// (lane l: row gm - l + l); `stage`: 32 x 80 bytes of shared memory owned by the warp.  N % 32 == 0.
template <class T>
__device__ __forceinline__ void ll_scatter_chunk(const LLArgs& a, uint32_t seq, size_t parity_off, int src, int gm, int gn,
                                                 const float (&f)[32], uint8_t* stage) {
  const int M = a.M, N = a.N;
  if (gn >= N) return;                          // uniform across the warp (N % 32 == 0)
  const int lane = threadIdx.x & 31;
  if (gm < M) {
    uint8_t* mine = stage + lane * 80;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float g[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) g[i] = f[j * 8 + i];
      *reinterpret_cast<Vec8*>(mine + j * 16) = pack8<T>(g);
    }
  }
  __syncwarp();
  // lane l sends 16-byte piece (l % 4) of rows (l / 4) + 8 i: four lanes cover 128 contiguous bytes of a row's words
  const int base_row = gm - lane, piece = lane & 3;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int rr = (lane >> 2) + 8 * i;
    const int grow = base_row + rr;
    if (grow < M) {
      const int owner = grow / a.owner_rows;
      const int lrow = grow - owner * a.owner_rows;
      const Vec8 pk = *reinterpret_cast<const Vec8*>(stage + rr * 80 + piece * 16);
      uint8_t* dst = a.scatter_peer[owner] + parity_off +
                     ((size_t(src) * a.owner_rows + lrow) * N + gn + piece * 8) * 4;
      st_volatile_u4(dst, pk.w[0], seq, pk.w[1], seq);
      st_volatile_u4(dst + 16, pk.w[2], seq, pk.w[3], seq);
    }
  }
  __syncwarp();                                 // the stage is free for the warp's next chunk
}

// Two 16-byte loads of {data, seq, data, seq}: true when all four words carry `seq`; the 8 values land in `pk`.
__device__ __forceinline__ bool ll_load8(const uint8_t* p, uint32_t seq, Vec8& pk) {
  const uint4 lo = ld_volatile_u4(p), hi = ld_volatile_u4(p + 16);
  pk.w[0] = lo.x;
  pk.w[1] = lo.z;
  pk.w[2] = hi.x;
  pk.w[3] = hi.z;
  return lo.y == seq && lo.w == seq && hi.y == seq && hi.w == seq;
}

template <class T, bool NVLS>
__device__ __forceinline__ void ll_phases(const LLArgs& a, uint32_t* status, float* s_red) {
  pdl_wait();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = int(gridDim.x);
  const unsigned long long epoch = *reinterpret_cast<volatile unsigned long long*>(a.state) / LL_UNIT;
  uint32_t seq = uint32_t(epoch) + 1u;
  if (seq == 0u) seq = 1u;
  const size_t pa = size_t(epoch & 1u) * a.scatter_parity_stride;
  const size_t pb = size_t(epoch & 1u) * a.result_parity_stride;
  unsigned long long* tr = (a.trace && tid == 0) ? a.trace + size_t(blockIdx.x) * 8 : nullptr;
  if (tr) tr[1] = globaltimer_ns();
  const unsigned long long deadline = globaltimer_ns() + a.wait_ns;
  bool alive = true;
  const int N = a.N, n8 = N >> 3;
  const T* bias = reinterpret_cast<const T*>(a.bias);
  const T* res = reinterpret_cast<const T*>(a.residual);

  // ---- phase B: owned rows, one warp per (row, 32 chunks of 8 values); units are dealt to the CTAs round-robin
  if (a.phases & 2) {
    const int R = a.row_end - a.row_begin;
    const int segs = (n8 + 31) / 32;
    const int units = R * segs;
    const int nsrc = a.world * a.S;               // at most LL_MAX_RANKS (checked by the launcher)
    for (int u = int(blockIdx.x) + G * warp; u < units; u += G * (PG_THREADS / 32)) {
      const int r = u / segs, c8 = (u - r * segs) * 32 + lane;
      if (c8 >= n8) continue;
      const int gr = a.row_begin + r;
      Vec8 pbias, pres;
      if (bias) pbias = *reinterpret_cast<const Vec8*>(bias + c8 * 8);
      if (res) pres = *reinterpret_cast<const Vec8*>(res + size_t(gr) * a.ld_res + c8 * 8);
      Vec8 pk[LL_MAX_RANKS];
      uint32_t polls = 0;
      bool ready;
      do {                                        // every load of a round is issued before the first check
        ready = true;
#pragma unroll
        for (int src = 0; src < LL_MAX_RANKS; ++src)
          if (src < nsrc)
            ready = ll_load8(a.scatter_local + pa + ((size_t(src) * a.owner_rows + r) * N + c8 * 8) * 4, seq, pk[src]) && ready;
        if (!ready && (++polls & 63u) == 0u && globaltimer_ns() > deadline) {
          if (status) atomicCAS(status, 0u, uint32_t(STATUS_WAIT_PEER));
          alive = false;
        }
      } while (!ready && alive);
      float acc[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] = 0.f;
#pragma unroll
      for (int src = 0; src < LL_MAX_RANKS; ++src)
        if (src < nsrc) {
          float f[8];
          unpack8<T>(pk[src], f);
#pragma unroll
          for (int k = 0; k < 8; ++k) acc[k] += f[k];
        }
      if (bias) {
        float f[8];
        unpack8<T>(pbias, f);
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] += f[k];
      }
      if (res) {
        float f[8];
        unpack8<T>(pres, f);
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] += f[k];
      }
      const Vec8 o = pack8<T>(acc);
      const size_t off = pb + (size_t(gr) * N + c8 * 8) * 4;
      if (NVLS) {
        multimem_st_u4(a.result_mc + off, o.w[0], seq, o.w[1], seq);
        multimem_st_u4(a.result_mc + off + 16, o.w[2], seq, o.w[3], seq);
      } else {
#pragma unroll
        for (int p = 0; p < LL_MAX_RANKS; ++p)
          if (p < a.world) {
            st_volatile_u4(a.result_peer[p] + off, o.w[0], seq, o.w[1], seq);
            st_volatile_u4(a.result_peer[p] + off + 16, o.w[2], seq, o.w[3], seq);
          }
      }
    }
  }
  if (tr) tr[3] = globaltimer_ns();

  // ---- phase C: all rows; a group of `wpr` warps takes a row, unpacks X and normalises it
  if (warp < 8 && (a.phases & 4)) {
    const int wpr = a.wpr, gpc = 8 / wpr, grp = warp / wpr, L = wpr * 32, l = (warp % wpr) * 32 + lane;
    T* out = reinterpret_cast<T*>(a.out);
    T* nout = reinterpret_cast<T*>(a.norm_out);
    const T* gamma = reinterpret_cast<const T*>(a.gamma);
    const T* beta = reinterpret_cast<const T*>(a.beta);
    float* slot = s_red + grp * 16;
    auto group_sum = [&](float x, float* sl) -> float {
      x = warp_sum(x);
      if (wpr == 1) return x;
      if (lane == 0) sl[warp % wpr] = x;
      bar_sync_named(1 + grp, L);
      float t = 0.f;
      for (int k = 0; k < wpr; ++k) t += sl[k];
      return t;
    };
    for (int r = int(blockIdx.x) + G * grp; r < a.M; r += G * gpc) {
      float v[4][8];
      Vec8 pk[4];
      uint32_t polls = 0;
      bool ready;
      do {
        ready = true;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int c8 = l + L * i;
          if (c8 < n8) ready = ll_load8(a.result_local + pb + (size_t(r) * N + c8 * 8) * 4, seq, pk[i]) && ready;
        }
        if (!ready && (++polls & 63u) == 0u && globaltimer_ns() > deadline) {
          if (status) atomicCAS(status, 0u, uint32_t(STATUS_WAIT_PEER));
          alive = false;
        }
      } while (!ready && alive);
      float s1 = 0.f, s2 = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int c8 = l + L * i;
        if (c8 < n8) {
          *reinterpret_cast<Vec8*>(out + size_t(r) * a.ld_out + c8 * 8) = pk[i];
          unpack8<T>(pk[i], v[i]);
#pragma unroll
          for (int k = 0; k < 8; ++k) { s1 += v[i][k]; s2 += v[i][k] * v[i][k]; }
        }
      }
      if (a.norm_mode == 3) {
        // RMSNorm * gamma, rounded through the storage type, then the row's int8 quantisation: the next BitLinear
        // layer reads (quant_out, quant_scale) directly
        const float inv = rsqrtf(group_sum(s2, slot) / float(N) + a.eps);
        float m = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int c8 = l + L * i;
          if (c8 < n8) {
            float g[8];
            unpack8<T>(*reinterpret_cast<const Vec8*>(gamma + c8 * 8), g);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              v[i][k] = Cvt<T>::to_f(Cvt<T>::from_f(v[i][k] * inv * g[k]));
              m = fmaxf(m, fabsf(v[i][k]));
            }
          }
        }
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (wpr > 1) {
          float* sl = slot + 8;
          if (lane == 0) sl[warp % wpr] = m;
          bar_sync_named(1 + grp, L);
          m = 0.f;
          for (int k = 0; k < wpr; ++k) m = fmaxf(m, sl[k]);
        }
        m = fmaxf(m, 1e-5f);
        const float qs = __fdiv_rn(127.f, m);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int c8 = l + L * i;
          if (c8 < n8) {
            alignas(8) int8_t o8[8];
#pragma unroll
            for (int k = 0; k < 8; ++k)
              o8[k] = int8_t(int(fminf(fmaxf(rintf(__fmul_rn(v[i][k], qs)), -127.f), 127.f)));
            *reinterpret_cast<uint2*>(a.quant_out + size_t(r) * N + c8 * 8) = *reinterpret_cast<const uint2*>(o8);
          }
        }
        if (l == 0) a.quant_scale[r] = __fdiv_rn(m, 127.f);
      } else if (a.norm_mode != 0) {
        float mean = 0.f, inv;
        if (a.norm_mode == 2) {
          inv = rsqrtf(group_sum(s2, slot) / float(N) + a.eps);
          if (wpr > 1) bar_sync_named(1 + grp, L);           // the slot is free for the next row
        } else {
          mean = group_sum(s1, slot) / float(N);
          float q = 0.f;
#pragma unroll
          for (int i = 0; i < 4; ++i)
            if (l + L * i < n8) {
#pragma unroll
              for (int k = 0; k < 8; ++k) { const float d = v[i][k] - mean; q += d * d; }
            }
          inv = rsqrtf(group_sum(q, slot + 8) / float(N) + a.eps);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int c8 = l + L * i;
          if (c8 < n8) {
            float g[8], b[8], o[8];
            if (gamma) unpack8<T>(*reinterpret_cast<const Vec8*>(gamma + c8 * 8), g);
            if (beta) unpack8<T>(*reinterpret_cast<const Vec8*>(beta + c8 * 8), b);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              float t = (v[i][k] - mean) * inv;
              if (gamma) t *= g[k];
              if (beta) t += b[k];
              o[k] = t;
            }
            *reinterpret_cast<Vec8*>(nout + size_t(r) * a.ld_out + c8 * 8) = pack8<T>(o);
          }
        }
      }
    }
  }
  if (tr) tr[4] = globaltimer_ns();

  // ---- epoch: the CTAs of a call add up to exactly LL_UNIT; no value is read back and nobody waits on the word (the
  // next call reads it after its dependency wait, when this grid has completed)
  __syncthreads();
  if (tid == 0 && (a.phases & 4)) {
    red_add_gpu_u64(a.state, blockIdx.x == 0 ? LL_UNIT - (unsigned long long)(G - 1) : 1ull);
    if (tr) tr[7] = globaltimer_ns();
  }
}

// ---------------------------------------------------------------------------------------------- host side
// Fills the device argument block from the C parameters (everything but the K-slice fields) after checking them.
// Returns 0 or a negative code.
inline int ll_fill_args(const RonnGemmLLParams* p, LLArgs& a) {
  const int M = p->M, N = p->N, world = p->world, rank = p->rank;
  if (M <= 0 || N <= 0 || world < 2 || world > LL_MAX_RANKS || rank < 0 || rank >= world) return -1;
  if ((N & 31) || (p->ld_out & 7) || (p->residual && (p->ld_res & 7))) return -2;
  if (p->norm_mode < 0 || p->norm_mode > 3) return -5;
  if ((p->norm_mode == 1 || p->norm_mode == 2) && p->norm_out == nullptr) return -5;
  if (p->norm_mode == 3 && (!p->quant_out || !p->quant_scale || !p->gamma || (N & 7))) return -5;
  if (p->out == nullptr || p->state == nullptr) return -6;
  const int owner_rows = (M + world - 1) / world;
  for (int r = 0; r < world; ++r)
    if (!p->scatter_area[r] || !p->result_area[r]) return -6;
  if (p->nvls && !p->result_mc) return -7;
  for (int r = 0; r < LL_MAX_RANKS; ++r) {
    a.scatter_peer[r] = r < world ? static_cast<uint8_t*>(p->scatter_area[r]) : nullptr;
    a.result_peer[r] = r < world ? static_cast<uint8_t*>(p->result_area[r]) : nullptr;
  }
  a.scatter_local = a.scatter_peer[rank];
  a.result_local = a.result_peer[rank];
  a.result_mc = static_cast<uint8_t*>(p->result_mc);
  a.scatter_parity_stride = p->scatter_parity_stride;
  a.result_parity_stride = p->result_parity_stride;
  a.state = static_cast<unsigned long long*>(p->state);
  a.out = p->out;
  a.norm_out = p->norm_out;
  a.bias = p->bias;
  a.residual = p->residual;
  a.gamma = p->gamma;
  a.beta = p->beta;
  a.trace = static_cast<unsigned long long*>(p->trace);
  a.quant_out = static_cast<int8_t*>(p->quant_out);
  a.quant_scale = p->quant_scale;
  a.wait_ns = static_cast<unsigned long long>(p->wait_seconds * 1e9);
  a.ld_out = p->ld_out;
  a.ld_res = p->ld_res;
  a.eps = p->eps;
  a.M = M;
  a.N = N;
  a.rank = rank;
  a.world = world;
  a.owner_rows = owner_rows;
  a.row_begin = rank * owner_rows < M ? rank * owner_rows : M;
  a.row_end = a.row_begin + owner_rows < M ? a.row_begin + owner_rows : M;
  a.norm_mode = p->norm_mode;
  a.nvls = p->nvls ? 1 : 0;
  a.wpr = 1;
  a.phases = (p->phases & 7) ? (p->phases & 7) : 7;
  a.S = 1;
  a.kb_per = 0;
  a.num_kb = 0;
  return 0;
}

// Warps per row of phase C: a lane keeps at most 4 chunks of 8 values; more warps when rows alone leave the grid idle.
// Returns 0 when a row does not fit.
inline int ll_pick_wpr(int M, int N, int grid) {
  const int n8 = N >> 3;
  int wpr = 1;
  while (wpr < 8 && n8 > 128 * wpr) wpr <<= 1;
  if (n8 > 128 * wpr) return 0;
  while (wpr < 8 && wpr * 32 < n8 && long(M) * (wpr * 2) <= 8l * grid) wpr <<= 1;
  return wpr;
}

}  // namespace ronn
