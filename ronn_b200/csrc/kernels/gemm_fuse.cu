// Skinny GEMM fused with everything that follows it, in ONE kernel:
//
//   X = sum over K-slices and over ranks of A[M, K] * W[N, K]^T + bias (+ activation) + residual
//   H = LayerNorm / RMSNorm(X) * gamma (+ beta)                                   (optional)
//
// Phase 1 is the persistent tcgen05 GEMM (TMA -> shared memory -> tcgen05.mma -> TMEM).  The K range is cut into S
// slices and every (row tile, column tile, slice) is one tile of the grid, so a decode-sized problem (M = 256) still
// puts a short K chain on every SM; the epilogue stores fp32 partial sums into a scratch area.  When the tiles of a
// CTA are stored it raises a counter per 128-row tile.
//
// Phase 2 runs in the same CTAs.  Every output row has ONE owner (a group of 1-8 warps): it waits (bounded) until the
// counters of its row tile are complete, sums the S slices in a fixed order, applies bias / activation / residual,
// writes the row, computes the row statistics and writes the normalised row.
//
// Across GPUs (tensor parallel, world W > 1) the same two phases form a two-shot all-reduce over NVLink, still
// inside the kernel: the scratch area, the counters and the outputs live in symmetric memory; rank r owns rows
// [r M / W, (r + 1) M / W).  Counters are raised on every rank, the owner sums the partials of all ranks and stores
// the finished rows into every rank's output; a second counter tells each rank when all owners have delivered.
//   NVLS mode: counters are raised with multimem.red, partials are summed inside the switch by multimem.ld_reduce,
//              finished rows are broadcast by multimem.st  (one instruction each, whatever the world size).
//   P2P mode : the same steps with W remote atomics, W peer loads and W peer stores.
// Every rank therefore moves 1/W of the result instead of W - 1 whole copies, bias / residual / norm are computed
// once per row instead of once per rank, and all ranks hold the same bits because only the owner computes a row.
// A reduce-scatter form (owner keeps its rows, nothing is broadcast) serves sequence-parallel activations.
//
// Counters only ever count up (compared modulo 2^32) and every one of them advances by the same amount per call, so
// the value a call waits for follows from one epoch word in local device memory and CUDA-graph replays need no host
// arguments.  No TMA multicast is used; all waits are bounded and report STATUS_WAIT_PEER through the status word.
//
// The reference has no collective and no fused projection (crates/ronn-providers/src/gpu/provider.rs:226-249 picks
// one device per sub-graph; crates/ronn-core/src/ops/matrix.rs:27-60 is a library matmul).
#include "gemm_fuse.h"

#include "gemm_epilogue.cuh"
#include "tma_desc.cuh"
#include "umma_persistent.cuh"

namespace ronn {

constexpr int FUSE_MAX_RANKS = RONN_FUSE_MAX_RANKS;
constexpr int FUSE_MAX_MT = RONN_FUSE_MAX_ROW_TILES;
// Every counter advances by exactly FUSE_UNIT per call: the arrivals of a call are 1 each except one designated
// arrival that carries the remainder, and counters a call does not use are advanced by its CTA 0.  A waiter therefore
// needs no per-counter bookkeeping: the value to wait for is (epoch word rounded down to a unit) + FUSE_UNIT.
constexpr uint32_t FUSE_UNIT = 1u << 16;             // more than the arrivals of any one call on one counter
// state (uint32, local): [0] epoch word, advanced by FUSE_UNIT per call by the leaving CTAs
// flag block (uint32, symmetric): [0, MAX_MT) "ready" counters per 128-row tile, [MAX_MT] "delivered" counter
constexpr int FL_DONE = FUSE_MAX_MT;

enum : int { FUSE_LOCAL = 0, FUSE_P2P = 1, FUSE_NVLS = 2 };

struct FuseArgs {
  float* part_local;                       // scratch: [2 parities][S][M][N] fp32
  const float* part_peer[FUSE_MAX_RANKS];  // the same area on every rank (P2P mode)
  const float* part_mc;                    // its multicast address (NVLS mode)
  long parity_stride;                      // floats between the two parities
  uint32_t* flag_local;
  uint32_t* flag_peer[FUSE_MAX_RANKS];
  uint32_t* flag_mc;
  uint32_t* state;
  uint8_t* out_peer[FUSE_MAX_RANKS];       // X on every rank ([0] = the local output when world == 1)
  uint8_t* out_mc;
  uint8_t* norm_peer[FUSE_MAX_RANKS];      // H on every rank, or null
  uint8_t* norm_mc;
  const void* bias;
  const void* residual;                    // rows aligned with X (all-reduce) or with the owned shard (scatter)
  const void* gamma;
  const void* beta;
  unsigned long long* trace;               // optional: 8 timestamps per CTA
  unsigned long long wait_ns;
  long ld_out, ld_res;
  float eps;
  int M, N, S, kb_per, num_kb;
  int rank, world;
  int row_begin, row_end;                  // rows this rank owns
  int owner_rows;                          // rows per owner (ceil(M / world)), for the delivered count
  int scatter;                             // 1: owned rows only, written locally with row 0 = row_begin
  int norm_mode;                           // 0 none, 1 LayerNorm, 2 RMSNorm
  int act;                                 // 0 none, 1 relu, 2 gelu(tanh): applied before the residual
  int wpr;                                 // warps per row in phase 2 (1, 2, 4 or 8); 0: flat (no whole rows)
};

// ------------------------------------------------------------------------------------------------ PTX helpers
__device__ __forceinline__ uint32_t ld_acquire_u32(const uint32_t* p, bool sys) {
  uint32_t v;
  if (sys) asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  else asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_add_sys(uint32_t* p, uint32_t v) {
  asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_add_gpu(uint32_t* p, uint32_t v) {
  asm volatile("red.relaxed.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void multimem_red_add(uint32_t* mc, uint32_t v) {
  asm volatile("multimem.red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(mc), "r"(v) : "memory");
}
__device__ __forceinline__ float4 multimem_ld_reduce_f32x4(const float* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_16(void* mc, const Vec8& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "r"(v.w[0]), "r"(v.w[1]),
               "r"(v.w[2]), "r"(v.w[3])
               : "memory");
}
__device__ __forceinline__ float4 ld_volatile_f4(const float* p) {
  float4 v;
  asm volatile("ld.volatile.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_global_16(void* p, const Vec8& v) {
  asm volatile("st.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.w[0]), "r"(v.w[1]), "r"(v.w[2]), "r"(v.w[3]) : "memory");
}
__device__ __forceinline__ void bar_sync_named(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// ------------------------------------------------------------------------------------------------ phase 1
template <int BN, class T>
struct FuseProblem {
  static constexpr bool kForceStage = false;
  const CUtensorMap* map_a;
  const CUtensorMap* map_b;
  const FuseArgs* a;
  int m_tiles, n_tiles;
  mutable float* part;             // resolved by the epilogue after the dependency wait

  __device__ __forceinline__ int num_tiles() const { return m_tiles * n_tiles * a->S; }
  __device__ __forceinline__ void tile(int t, int& m0, int& n0, int& kb0, int& nkb) const {
    const int per_z = m_tiles * n_tiles;
    const int z = t / per_z, r = t - z * per_z;
    m0 = (r % m_tiles) * PG_BM;
    n0 = (r / m_tiles) * BN;
    kb0 = z * a->kb_per;
    nkb = min(a->kb_per, a->num_kb - kb0);
  }
  __device__ __forceinline__ void load_a(uint8_t* smem, uint64_t* bar, int k_elem, int m0) const {
    tma_load_2d(smem, map_a, bar, k_elem, m0);
  }
  __device__ __forceinline__ void load_b(uint8_t* smem, uint64_t* bar, int k_elem, int n0) const {
    tma_load_2d(smem, map_b, bar, k_elem, n0);
  }
  __device__ __forceinline__ void epilogue(int t, int m0, int n0, int row, int col, uint32_t (&r)[32], uint8_t*) const {
    if (part == nullptr) {
      const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(a->state) / FUSE_UNIT;
      part = a->part_local + size_t(epoch & 1u) * a->parity_stride;
    }
    const int gm = m0 + row, gn = n0 + col;
    const int M = a->M, N = a->N;
    if (gn >= N || gm >= M) return;
    const int z = t / (m_tiles * n_tiles);
    float* dst = part + (size_t(z) * M + gm) * N + gn;
    if (gn + 32 <= N) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        *reinterpret_cast<float4*>(dst + j * 4) =
            make_float4(__uint_as_float(r[j * 4]), __uint_as_float(r[j * 4 + 1]), __uint_as_float(r[j * 4 + 2]),
                        __uint_as_float(r[j * 4 + 3]));
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (gn + i < N) dst[i] = __uint_as_float(r[i]);
    }
  }
};

// ------------------------------------------------------------------------------------------------ phase 2
// Sum of the S slices (and of all ranks) of 8 consecutive values at float offset `off` of the parity slot, in a
// fixed order (slice-major, rank-minor).  Up to eight 32-byte loads are in flight before the first one is used.
template <int MODE>
__device__ __forceinline__ void fuse_gather8(const FuseArgs& a, size_t off, float (&acc)[8]) {
  const size_t slice = size_t(a.M) * a.N;
  const int total = MODE == FUSE_P2P ? a.S * a.world : a.S;
#pragma unroll
  for (int k = 0; k < 8; ++k) acc[k] = 0.f;
  for (int base = 0; base < total; base += 8) {
    float4 lo[8], hi[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int idx = base + j;
      if (idx < total) {
        if (MODE == FUSE_NVLS) {
          const float* p = a.part_mc + off + size_t(idx) * slice;
          lo[j] = multimem_ld_reduce_f32x4(p);
          hi[j] = multimem_ld_reduce_f32x4(p + 4);
        } else {
          const float* p = MODE == FUSE_P2P ? a.part_peer[idx % a.world] + off + size_t(idx / a.world) * slice
                                            : a.part_local + off + size_t(idx) * slice;
          lo[j] = ld_volatile_f4(p);
          hi[j] = ld_volatile_f4(p + 4);
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (base + j < total) {
        acc[0] += lo[j].x; acc[1] += lo[j].y; acc[2] += lo[j].z; acc[3] += lo[j].w;
        acc[4] += hi[j].x; acc[5] += hi[j].y; acc[6] += hi[j].z; acc[7] += hi[j].w;
      }
  }
}

// The same sums for CH chunks of one row at once.  A peer load is a round trip of several microseconds under load:
// the loads of all chunks of a source are issued before the first value is used, 2 CH 16-byte loads in flight per
// lane, where chunk-after-chunk gathers made a row cost CH round trips (measured: 80 us for the
// owner-side reduction of 4096 x 1024 rows at two ranks).
template <int MODE, int CH>
__device__ __forceinline__ void fuse_gather_multi(const FuseArgs& a, const size_t (&off)[CH], const bool (&valid)[CH],
                                                  float (&acc)[CH][8]) {
  const size_t slice = size_t(a.M) * a.N;
  const int total = MODE == FUSE_P2P ? a.S * a.world : a.S;
#pragma unroll
  for (int i = 0; i < CH; ++i)
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[i][k] = 0.f;
  for (int idx = 0; idx < total; ++idx) {
    float4 lo[CH], hi[CH];
#pragma unroll
    for (int i = 0; i < CH; ++i)
      if (valid[i]) {
        if (MODE == FUSE_NVLS) {
          const float* p = a.part_mc + off[i] + size_t(idx) * slice;
          lo[i] = multimem_ld_reduce_f32x4(p);
          hi[i] = multimem_ld_reduce_f32x4(p + 4);
        } else {
          const float* p = MODE == FUSE_P2P ? a.part_peer[idx % a.world] + off[i] + size_t(idx / a.world) * slice
                                            : a.part_local + off[i] + size_t(idx) * slice;
          lo[i] = ld_volatile_f4(p);
          hi[i] = ld_volatile_f4(p + 4);
        }
      }
#pragma unroll
    for (int i = 0; i < CH; ++i)
      if (valid[i]) {
        acc[i][0] += lo[i].x; acc[i][1] += lo[i].y; acc[i][2] += lo[i].z; acc[i][3] += lo[i].w;
        acc[i][4] += hi[i].x; acc[i][5] += hi[i].y; acc[i][6] += hi[i].z; acc[i][7] += hi[i].w;
      }
  }
}

// 16 bytes of an output row: the local copy, or one copy per rank.
template <int MODE>
__device__ __forceinline__ void fuse_store16(const FuseArgs& a, uint8_t* const (&peer)[FUSE_MAX_RANKS], uint8_t* mc,
                                             size_t byte_off, const Vec8& v) {
  if (MODE == FUSE_LOCAL || a.scatter) {
    st_global_16(peer[MODE == FUSE_LOCAL ? 0 : a.rank] + byte_off, v);
  } else if (MODE == FUSE_NVLS) {
    multimem_st_16(mc + byte_off, v);
  } else {
#pragma unroll
    for (int p = 0; p < FUSE_MAX_RANKS; ++p)
      if (p < a.world) st_global_16(peer[p] + byte_off, v);
  }
}

// bias, activation, residual on 8 summed values; stores the 16-byte result and returns it as stored (rounded).
template <class T, int MODE>
__device__ __forceinline__ void fuse_finish8(const FuseArgs& a, float (&acc)[8], const Vec8& bias, const Vec8& res,
                                             int out_row, int c, float (&v)[8]) {
  if (a.bias) {
    float f[8];
    unpack8<T>(bias, f);
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] += f[k];
  }
  if (a.act == 1) {
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = fmaxf(acc[k], 0.f);
  } else if (a.act == 2) {
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = gelu_tanh_f(acc[k]);
  }
  if (a.residual) {
    float f[8];
    unpack8<T>(res, f);
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] += f[k];
  }
  const Vec8 o = pack8<T>(acc);
  fuse_store16<MODE>(a, a.out_peer, a.out_mc, (size_t(out_row) * a.ld_out + c) * sizeof(T), o);
  unpack8<T>(o, v);                              // the norm sees exactly what the residual stream stores
}

// Whole rows: a group of `wpr` warps owns a row and keeps it in registers (CH chunks of 8 values per lane) for the
// norm.  The operands that do not depend on the GEMM (bias, residual, scale, shift) of a group's first row are
// fetched by `prefetch` before the wait, so the wait hides their latency.
template <class T, int MODE, int CH>
struct FuseRows {
  int wpr, gpc, grp, L, l, n8, r, R, G;

  __device__ __forceinline__ void init(const FuseArgs& a) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    wpr = a.wpr;
    gpc = 8 / wpr;
    grp = warp / wpr;
    L = wpr * 32;
    l = (warp % wpr) * 32 + lane;
    n8 = a.N >> 3;
    R = a.row_end - a.row_begin;
    G = int(gridDim.x);
    r = warp < 8 ? int(blockIdx.x) + G * grp : R;
  }
  // CH == 1 (decode: the group's lanes cover the row once) keeps the side operands in registers across the wait;
  // wider rows fetch them where they are used, which keeps the kernel at one register allocation for all paths
  static constexpr bool PRE = CH == 1;
  Vec8 pb[PRE ? CH : 1], pr[PRE ? CH : 1], pg[PRE ? CH : 1], pt[PRE ? CH : 1];
  __device__ __forceinline__ void prefetch(const FuseArgs& a) {
    if (!PRE || r >= R) return;
    const T* bias = reinterpret_cast<const T*>(a.bias);
    const T* res = reinterpret_cast<const T*>(a.residual);
    const T* gamma = reinterpret_cast<const T*>(a.gamma);
    const T* beta = reinterpret_cast<const T*>(a.beta);
    const int out_row = a.scatter ? r : a.row_begin + r;
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      const int c8 = l + L * i;
      if (c8 < n8) {
        if (bias) pb[i] = *reinterpret_cast<const Vec8*>(bias + c8 * 8);
        if (res) pr[i] = *reinterpret_cast<const Vec8*>(res + size_t(out_row) * a.ld_res + c8 * 8);
        if (a.norm_mode != 0 && gamma) pg[i] = *reinterpret_cast<const Vec8*>(gamma + c8 * 8);
        if (a.norm_mode != 0 && beta) pt[i] = *reinterpret_cast<const Vec8*>(beta + c8 * 8);
      }
    }
  }
  __device__ __forceinline__ void run(const FuseArgs& a, size_t parity_off, float* s_red) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* slot = s_red + grp * 16;              // [8] first exchange, [8] second exchange
    auto group_sum = [&](float x, float* sl) -> float {
      x = warp_sum(x);
      if (wpr == 1) return x;
      if (lane == 0) sl[warp % wpr] = x;
      bar_sync_named(1 + grp, L);
      float t = 0.f;
      for (int k = 0; k < wpr; ++k) t += sl[k];
      return t;
    };
    while (r < R) {
      const int gr = a.row_begin + r;
      const int out_row = a.scatter ? r : gr;
      float v[CH][8];
      float s1 = 0.f, s2 = 0.f;
      if (CH == 1) {
        const int c8 = l;
        if (c8 < n8) {
          float acc[8];
          fuse_gather8<MODE>(a, parity_off + size_t(gr) * a.N + c8 * 8, acc);
          fuse_finish8<T, MODE>(a, acc, pb[0], pr[0], out_row, c8 * 8, v[0]);
#pragma unroll
          for (int k = 0; k < 8; ++k) { s1 += v[0][k]; s2 += v[0][k] * v[0][k]; }
        }
      } else {
        // wide rows: the partial sums of all chunks and the side operands are requested together
        size_t off[CH];
        bool valid[CH];
        Vec8 lb[CH], lr[CH];
#pragma unroll
        for (int i = 0; i < CH; ++i) {
          const int c8 = l + L * i;
          valid[i] = c8 < n8;
          off[i] = parity_off + size_t(gr) * a.N + c8 * 8;
          if (valid[i]) {
            if (a.bias) lb[i] = *reinterpret_cast<const Vec8*>(reinterpret_cast<const T*>(a.bias) + c8 * 8);
            if (a.residual)
              lr[i] = *reinterpret_cast<const Vec8*>(reinterpret_cast<const T*>(a.residual) + size_t(out_row) * a.ld_res + c8 * 8);
          }
        }
        float acc[CH][8];
        fuse_gather_multi<MODE, CH>(a, off, valid, acc);
#pragma unroll
        for (int i = 0; i < CH; ++i)
          if (valid[i]) {
            fuse_finish8<T, MODE>(a, acc[i], lb[i], lr[i], out_row, (l + L * i) * 8, v[i]);
#pragma unroll
            for (int k = 0; k < 8; ++k) { s1 += v[i][k]; s2 += v[i][k] * v[i][k]; }
          }
      }
      if (a.norm_mode != 0) {
        float mean = 0.f, inv;
        if (a.norm_mode == 2) {
          inv = rsqrtf(group_sum(s2, slot) / float(a.N) + a.eps);
          if (wpr > 1) bar_sync_named(1 + grp, L);         // the slot is free for the next row
        } else {
          mean = group_sum(s1, slot) / float(a.N);
          float q = 0.f;
#pragma unroll
          for (int i = 0; i < CH; ++i)
            if (l + L * i < n8) {
#pragma unroll
              for (int k = 0; k < 8; ++k) { const float d = v[i][k] - mean; q += d * d; }
            }
          inv = rsqrtf(group_sum(q, slot + 8) / float(a.N) + a.eps);
        }
#pragma unroll
        for (int i = 0; i < CH; ++i) {
          const int c8 = l + L * i;
          if (c8 < n8) {
            float g[8], b[8], o[8];
            if (a.gamma) unpack8<T>(PRE ? pg[i] : *reinterpret_cast<const Vec8*>(reinterpret_cast<const T*>(a.gamma) + c8 * 8), g);
            if (a.beta) unpack8<T>(PRE ? pt[i] : *reinterpret_cast<const Vec8*>(reinterpret_cast<const T*>(a.beta) + c8 * 8), b);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              float t = (v[i][k] - mean) * inv;
              if (a.gamma) t *= g[k];
              if (a.beta) t += b[k];
              o[k] = t;
            }
            fuse_store16<MODE>(a, a.norm_peer, a.norm_mc, (size_t(out_row) * a.ld_out + c8 * 8) * sizeof(T), pack8<T>(o));
          }
        }
      }
      r += G * gpc;
      prefetch(a);                               // residual of the group's next row (bias, scale, shift: same values)
    }
  }
};

// CTAs of a rank that own rows in phase 2: a function of (rows, grid, path) only, so every rank can count the
// "delivered" arrivals to expect from every other rank.
__device__ __forceinline__ uint32_t fuse_owner_ctas(const FuseArgs& a, int rows, int G) {
  const long n8 = a.N >> 3;
  const long c = a.wpr > 0 ? long(rows) : (long(rows) * n8 + PG_THREADS - 1) / PG_THREADS;
  return uint32_t(c < G ? c : G);
}

template <class T, int MODE>
__device__ __forceinline__ void fuse_phase2(const FuseArgs& a, int m_tiles, int n_tiles, uint32_t* status,
                                            float* s_red) {
  pdl_wait();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = int(gridDim.x);
  // every counter has advanced by FUSE_UNIT per completed call, the epoch word included; CTAs of THIS call that have
  // already left add less than a unit in total, so rounding down gives the value at the start of the call
  const uint32_t base = *reinterpret_cast<volatile uint32_t*>(a.state) & ~(FUSE_UNIT - 1u);
  const uint32_t want = base + FUSE_UNIT;
  const size_t parity_off = size_t((base / FUSE_UNIT) & 1u) * a.parity_stride;
  unsigned long long* tr = (a.trace && tid == 0) ? a.trace + size_t(blockIdx.x) * 8 : nullptr;
  if (tr) tr[1] = globaltimer_ns();
  const int R = a.row_end - a.row_begin;
  const int n8 = a.N >> 3;

  // ---- operands of the first row that do not depend on the GEMM: in flight before the wait
  FuseRows<T, MODE, 1> rows1;
  FuseRows<T, MODE, 4> rows4;
  const bool one_chunk = a.wpr > 0 && n8 <= a.wpr * 32;
  if (a.wpr > 0) {
    if (one_chunk) { rows1.init(a); rows1.prefetch(a); }
    else { rows4.init(a); rows4.prefetch(a); }
  }

  // ---- publish: the tiles of this CTA are stored (the GEMM's closing barrier has passed).  The arrivals of a call
  // add up to exactly FUSE_UNIT per counter: one designated tile per row tile carries the remainder.
  if (tid == 0) {
    if (MODE == FUSE_LOCAL) __threadfence(); else __threadfence_system();
    const int per_z = m_tiles * n_tiles, ntiles = per_z * a.S;
    const uint32_t count = uint32_t(a.world * n_tiles * a.S);
    for (int t = blockIdx.x; t < ntiles; t += G) {
      const int mt = (t % per_z) % m_tiles;
      const uint32_t inc = (a.rank == 0 && t < m_tiles) ? FUSE_UNIT - (count - 1u) : 1u;
      if (MODE == FUSE_LOCAL) {
        red_add_gpu(a.flag_local + mt, inc);
      } else if (MODE == FUSE_NVLS) {
        multimem_red_add(a.flag_mc + mt, inc);
      } else {
        for (int p = 0; p < a.world; ++p) red_add_sys(a.flag_peer[p] + mt, inc);
      }
    }
    if (tr) tr[2] = globaltimer_ns();
  }
  // counters this call does not use advance too (local copies only: nobody else touches them in this call)
  if (blockIdx.x == 0 && tid < FUSE_MAX_MT + 1) {
    const bool unused = tid < FUSE_MAX_MT ? tid >= m_tiles : (MODE == FUSE_LOCAL || a.scatter);
    if (unused) red_add_gpu(a.flag_local + tid, FUSE_UNIT);
  }

  // ---- wait (bounded) until the row tiles that hold this rank's rows are complete on every rank
  const unsigned long long deadline = globaltimer_ns() + a.wait_ns;
  if (warp == 0 && R > 0) {
    const int mt_lo = a.row_begin / PG_BM, mt_hi = (a.row_end - 1) / PG_BM;
    for (int mt = mt_lo + lane; mt <= mt_hi; mt += 32) {
      uint32_t polls = 0;
      while (int32_t(ld_acquire_u32(a.flag_local + mt, MODE != FUSE_LOCAL) - want) < 0) {
        if ((++polls & 63u) == 0u && globaltimer_ns() > deadline) {
          if (status) atomicCAS(status, 0u, uint32_t(STATUS_WAIT_PEER));
          break;
        }
      }
    }
  }
  __syncthreads();
  if (tr) tr[3] = globaltimer_ns();

  if (a.wpr > 0) {
    if (one_chunk) rows1.run(a, parity_off, s_red);
    else rows4.run(a, parity_off, s_red);
  } else {
    // ---- flat: 16-byte pieces of the owned rows, no row statistics
    const T* bias = reinterpret_cast<const T*>(a.bias);
    const T* res = reinterpret_cast<const T*>(a.residual);
    const long vecs = long(R) * n8;
    for (long i = long(blockIdx.x) * blockDim.x + tid; i < vecs; i += long(G) * blockDim.x) {
      const int r = int(i / n8), c = int(i - long(r) * n8) * 8;
      const int gr = a.row_begin + r;
      const int out_row = a.scatter ? r : gr;
      Vec8 pb, pr;
      if (bias) pb = *reinterpret_cast<const Vec8*>(bias + c);
      if (res) pr = *reinterpret_cast<const Vec8*>(res + size_t(out_row) * a.ld_res + c);
      float acc[8], v[8];
      fuse_gather8<MODE>(a, parity_off + size_t(gr) * a.N + c, acc);
      fuse_finish8<T, MODE>(a, acc, pb, pr, out_row, c, v);
    }
  }
  if (tr) tr[4] = globaltimer_ns();

  // ---- delivered: every owner CTA tells every rank once its rows are stored there; one thread of the grid waits
  // until all owners of all ranks have done so, which makes the kernel's completion mean "all rows are here"
  if (MODE != FUSE_LOCAL && !a.scatter) {
    __syncthreads();
    if (tid == 0) {
      uint32_t expect = 0;
      for (int p = 0; p < a.world; ++p) {
        const int rb = min(p * a.owner_rows, a.M), re = min(rb + a.owner_rows, a.M);
        expect += fuse_owner_ctas(a, re - rb, G);
      }
      if (uint32_t(blockIdx.x) < fuse_owner_ctas(a, R, G)) {
        __threadfence_system();
        const uint32_t inc = (a.rank == 0 && blockIdx.x == 0) ? FUSE_UNIT - (expect - 1u) : 1u;
        if (MODE == FUSE_NVLS) {
          multimem_red_add(a.flag_mc + FL_DONE, inc);
        } else {
          for (int p = 0; p < a.world; ++p) red_add_sys(a.flag_peer[p] + FL_DONE, inc);
        }
        if (tr) tr[5] = globaltimer_ns();
      }
      if (blockIdx.x == 0) {
        uint32_t polls = 0;
        while (int32_t(ld_acquire_u32(a.flag_local + FL_DONE, true) - want) < 0) {
          if ((++polls & 63u) == 0u && globaltimer_ns() > deadline) {
            if (status) atomicCAS(status, 0u, uint32_t(STATUS_WAIT_PEER));
            break;
          }
        }
        if (tr) tr[6] = globaltimer_ns();
      }
    }
  }

  // ---- epoch: the CTAs of a call add up to exactly FUSE_UNIT (no value is read back, nobody waits on it; the next
  // call reads the word after its dependency wait, when this grid has completed)
  __syncthreads();
  if (tid == 0) {
    red_add_gpu(a.state, blockIdx.x == 0 ? FUSE_UNIT - uint32_t(G - 1) : 1u);
    if (tr) tr[7] = globaltimer_ns();
  }
}

template <int BN, int STAGES, class T, int MODE>
__global__ void __launch_bounds__(PG_THREADS)
gemm_fuse_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ FuseArgs args, uint32_t idesc, uint32_t* status) {
  extern __shared__ uint8_t dyn_smem[];
  __shared__ float s_red[8 * 16];
  if (args.trace && threadIdx.x == 0) args.trace[size_t(blockIdx.x) * 8] = globaltimer_ns();
  FuseProblem<BN, T> prob;
  prob.map_a = &map_a;
  prob.map_b = &map_b;
  prob.a = &args;
  prob.m_tiles = (args.M + PG_BM - 1) / PG_BM;
  prob.n_tiles = (args.N + BN - 1) / BN;
  prob.part = nullptr;
  gemm_persistent<BN, STAGES, 0, FuseProblem<BN, T>>(dyn_smem, prob, 64, idesc, status);
  fuse_phase2<T, MODE>(args, prob.m_tiles, prob.n_tiles, status, s_red);
}

static int fuse_sm_count() { return device_sm_count(); }

// Grid of a (BN, STAGES) variant: every CTA must be resident at once because phase 2 waits on the whole grid.
template <int BN, int STAGES, class T, int MODE>
static int fuse_grid(int tiles, int* grid_out) {
  using L = PGemmSmem<BN, STAGES>;
  auto kern = gemm_fuse_kernel<BN, STAGES, T, MODE>;
  static bool configured[MAX_DEVICES] = {false};
  if (first_use_on_device(configured)) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYN_SMEM) != cudaSuccess) return -10;
  }
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, PG_THREADS, L::DYN_SMEM) != cudaSuccess || per_sm < 1)
    return -12;
  if (per_sm > 2) per_sm = 2;
  if (512u / L::TMEM_COLS < unsigned(per_sm)) per_sm = int(512u / L::TMEM_COLS);      // TMEM columns per SM
  const int resident = fuse_sm_count() * per_sm;
  *grid_out = tiles < resident ? tiles : resident;
  return 0;
}

template <int BN, int STAGES, class T, int MODE>
static int fuse_launch(const CUtensorMap& ma, const CUtensorMap& mb, FuseArgs& a, int grid, int is_bf16,
                       uint32_t* status, cudaStream_t stream) {
  using L = PGemmSmem<BN, STAGES>;
  auto kern = gemm_fuse_kernel<BN, STAGES, T, MODE>;
  const uint32_t idesc = umma_idesc(PG_BM, BN, is_bf16 ? 1u : 0u, 1u);
  cudaError_t err = launch(kern, dim3(grid), dim3(PG_THREADS), size_t(L::DYN_SMEM), stream, ma, mb, a, idesc, status);
  return (err == cudaSuccess && cudaGetLastError() == cudaSuccess) ? 0 : -11;
}

// Warps per row of phase 2: enough that a lane keeps at most 4 chunks of 8 values, more when the owned rows alone
// would leave most of the grid idle (decode), never more than the row has 16-byte chunks for.
static int pick_wpr(int rows, int n8, int grid) {
  int need = 1;
  while (need < 8 && n8 > 128 * need) need <<= 1;
  if (n8 > 128 * need) return -1;                // rows wider than 8192 values are not kept in registers
  int useful = 1;
  while (useful < 8 && useful * 32 < n8) useful <<= 1;
  int wpr = need;
  while (wpr < useful && long(rows) * (wpr * 2) <= 8l * grid) wpr <<= 1;
  return wpr;
}

template <int BN, int STAGES, class T>
static int fuse_dispatch(const CUtensorMap& ma, const CUtensorMap& mb, FuseArgs& a, int mode, int want_rows,
                         int is_bf16, uint32_t* status, cudaStream_t stream) {
  const int tiles = ((a.N + BN - 1) / BN) * ((a.M + PG_BM - 1) / PG_BM) * a.S;
  int grid = 0, rc;
  if (mode == FUSE_LOCAL) rc = fuse_grid<BN, STAGES, T, FUSE_LOCAL>(tiles, &grid);
  else if (mode == FUSE_P2P) rc = fuse_grid<BN, STAGES, T, FUSE_P2P>(tiles, &grid);
  else rc = fuse_grid<BN, STAGES, T, FUSE_NVLS>(tiles, &grid);
  if (rc) return rc;
  a.wpr = 0;
  if (want_rows) {
    a.wpr = pick_wpr(a.owner_rows, a.N >> 3, grid);
    if (a.wpr < 0) return -5;
  }
  if (mode == FUSE_LOCAL) return fuse_launch<BN, STAGES, T, FUSE_LOCAL>(ma, mb, a, grid, is_bf16, status, stream);
  if (mode == FUSE_P2P) return fuse_launch<BN, STAGES, T, FUSE_P2P>(ma, mb, a, grid, is_bf16, status, stream);
  return fuse_launch<BN, STAGES, T, FUSE_NVLS>(ma, mb, a, grid, is_bf16, status, stream);
}

}  // namespace ronn

using namespace ronn;

extern "C" int ronn_gemm_fuse(const RonnGemmFuseParams* p, uint32_t* status, cudaStream_t stream) {
  if (!p) return -1;
  const int M = p->M, N = p->N, K = p->K, world = p->world, rank = p->rank;
  if (M <= 0 || N <= 0 || K <= 0 || world < 1 || world > FUSE_MAX_RANKS || rank < 0 || rank >= world) return -1;
  if ((K & 7) || (p->lda & 7) || (p->ldw & 7) || (N & 7) || (p->ld_out & 7) || (p->residual && (p->ld_res & 7))) return -2;
  const int m_tiles = (M + PG_BM - 1) / PG_BM;
  if (m_tiles > FUSE_MAX_MT) return -4;
  if (p->norm_mode != 0 && (p->norm_out[0] == nullptr || p->norm_mode > 2)) return -5;
  if (p->part[0] == nullptr || p->flags[0] == nullptr || p->state == nullptr || p->out[0] == nullptr) return -6;
  int mode = FUSE_LOCAL;
  if (world > 1) {
    mode = p->nvls ? FUSE_NVLS : FUSE_P2P;
    for (int r = 0; r < world; ++r) {
      if (!p->part[r] || !p->flags[r]) return -6;
      if (!p->scatter && (!p->out[r] || (p->norm_mode && !p->norm_out[r]))) return -6;
    }
    if (mode == FUSE_NVLS && (!p->part_mc || !p->flags_mc || (!p->scatter && (!p->out_mc || (p->norm_mode && !p->norm_mc)))))
      return -7;
  }
  const int num_kb = (K + 63) / 64;
  int S = p->splitk < 1 ? 1 : p->splitk;
  if (S > num_kb) S = num_kb;
  const int kb_per = (num_kb + S - 1) / S;
  S = (num_kb + kb_per - 1) / kb_per;              // every slice non-empty
  if (long(S) * M * N > p->parity_stride) return -8;

  FuseArgs a;
  a.part_local = static_cast<float*>(p->part[world > 1 ? rank : 0]);
  a.flag_local = static_cast<uint32_t*>(p->flags[world > 1 ? rank : 0]);
  for (int r = 0; r < FUSE_MAX_RANKS; ++r) {
    const bool in = r < world;
    a.part_peer[r] = in ? static_cast<const float*>(p->part[r]) : nullptr;
    a.flag_peer[r] = in ? static_cast<uint32_t*>(p->flags[r]) : nullptr;
    a.out_peer[r] = in ? static_cast<uint8_t*>(p->out[r]) : nullptr;
    a.norm_peer[r] = in ? static_cast<uint8_t*>(p->norm_out[r]) : nullptr;
  }
  a.part_mc = static_cast<const float*>(p->part_mc);
  a.flag_mc = static_cast<uint32_t*>(p->flags_mc);
  a.out_mc = static_cast<uint8_t*>(p->out_mc);
  a.norm_mc = static_cast<uint8_t*>(p->norm_mc);
  a.parity_stride = p->parity_stride;
  a.state = static_cast<uint32_t*>(p->state);
  a.bias = p->bias;
  a.residual = p->residual;
  a.gamma = p->gamma;
  a.beta = p->beta;
  a.trace = static_cast<unsigned long long*>(p->trace);
  a.wait_ns = static_cast<unsigned long long>(p->wait_seconds * 1e9);
  a.ld_out = p->ld_out;
  a.ld_res = p->ld_res;
  a.eps = p->eps;
  a.M = M;
  a.N = N;
  a.S = S;
  a.kb_per = kb_per;
  a.num_kb = num_kb;
  a.rank = rank;
  a.world = world;
  a.owner_rows = (M + world - 1) / world;
  a.row_begin = world > 1 ? (rank * a.owner_rows < M ? rank * a.owner_rows : M) : 0;
  a.row_end = world > 1 ? (a.row_begin + a.owner_rows < M ? a.row_begin + a.owner_rows : M) : M;
  a.scatter = (world > 1 && p->scatter) ? 1 : 0;
  a.norm_mode = p->norm_mode;
  a.act = p->act;
  a.wpr = 0;
  const int want_rows = p->norm_mode != 0 || (N >> 3) <= 512;     // rows of up to 4096 values take the row path

  int bn = p->bn & 0xfff;
  if (bn == 0) {
    // narrow tiles until the grid has about one CTA per SM; the K slices multiply the tile count
    bn = 128;
    while (bn > 32 && long(m_tiles) * ((N + bn - 1) / bn) * S < 120) bn >>= 1;
  }
  if (long(world) * ((N + bn - 1) / bn) * S >= long(FUSE_UNIT)) return -9;      // arrivals per counter and call
  const int tiles = m_tiles * ((N + bn - 1) / bn) * S;
  const int deep = (p->bn & 0x1000) ? 1 : ((p->bn & 0x2000) ? 0 : (tiles <= fuse_sm_count() ? 1 : 0));
  CUtensorMap ma, mb;
  int rc = make_tmap_2d(&ma, p->A, uint64_t(M), uint64_t(K), uint64_t(p->lda), PG_BM, 64, 2);
  if (rc) return rc - 20;
  rc = make_tmap_2d(&mb, p->W, uint64_t(N), uint64_t(K), uint64_t(p->ldw), uint32_t(bn), 64, 2);
  if (rc) return rc - 30;
  const int bf = p->dtype == 0;
#define RONN_DISPATCH(BN_, ST_)                                                                         \
  return bf ? fuse_dispatch<BN_, ST_, __nv_bfloat16>(ma, mb, a, mode, want_rows, 1, status, stream)     \
            : fuse_dispatch<BN_, ST_, __half>(ma, mb, a, mode, want_rows, 0, status, stream)
  switch (deep ? -bn : bn) {
    case 128: RONN_DISPATCH(128, 3);
    case 64: RONN_DISPATCH(64, 4);
    case 32: RONN_DISPATCH(32, 5);
    case -128: RONN_DISPATCH(128, 6);
    case -64: RONN_DISPATCH(64, 8);
    case -32: RONN_DISPATCH(32, 10);
    default: return -3;
  }
#undef RONN_DISPATCH
}

extern "C" int ronn_gemm_fuse_state_ints(void) { return 8; }
extern "C" int ronn_gemm_fuse_flag_ints(void) { return FUSE_MAX_MT + 8; }
