// Row-parallel GEMM fused with its collective, in ONE kernel, over NVLink peer memory.
//
//   Y = reduce_over_ranks( A_r[M, K_r] * W_r[N, K_r]^T ) + bias + residual
//
// Every rank runs the same kernel.  Phase 1 is the persistent tcgen05 GEMM; its epilogue writes
// the rank's partial products (bf16) into the rank's own slot of a symmetric buffer.  When the last
// CTA of a rank has stored its tiles, that rank raises a per-call flag on every peer with a remote
// system-scope atomic.  Phase 2 runs in the same CTAs: each waits (bounded) until all ranks have
// flagged, then reads the partials of every rank straight from peer memory with 16-byte loads, sums
// them in fp32 in rank order (so every rank obtains bit-identical results), adds bias and residual
// and writes the rows it owns:
//     all-reduce mode      rows [0, M)          -> replicated activations (decode, small M)
//     reduce-scatter mode  this rank's row shard -> sequence-parallel activations (prefill)
//
// Buffers alternate between two parities per call; a rank can never run two calls ahead of a peer
// (phase 2 of call k needs every peer's phase 1 of call k), so two slots are enough.  Flags only ever
// count up (one increment per call and source rank), so nothing is reset between calls and CUDA-graph
// replays need no host-side arguments: the call counter lives in device memory.
//
// No TMA multicast is used anywhere; remote data is read with plain loads, flags are written with
// remote atomics.  All waits are bounded: on expiry the kernel records STATUS_WAIT_PEER and returns.
//
// The reference has no collective of any kind (its only multi-GPU code picks one device per sub-graph,
// crates/ronn-providers/src/gpu/provider.rs:226-249).
#include "gemm_epilogue.cuh"
#include "tma_desc.cuh"
#include "umma_persistent.cuh"

namespace ronn {

constexpr int MAX_RANKS = 8;

struct CommArgs {
  uint8_t* peer_part[MAX_RANKS];   // base of every rank's partial buffer (two parities back to back)
  int* peer_flags[MAX_RANKS];      // every rank's flag array: [2 parities][MAX_RANKS sources]
  long part_stride;                // bytes between the two parity slots
  int* state;                      // local, 8 ints: [0] calls completed, [1] phase-1 CTA counter, [2] phase-2 CTA
                                   // counter, [4 + parity] flag (pull-mode) calls completed on that parity
  int rank, world;
  int row_begin, row_end;          // rows this rank reduces and writes
  void* out;                       // [row_end - row_begin, N]
  long ld_out;
  const void* bias;                // [N] or null
  const void* residual;            // rows aligned with `out`, or null
  long ld_res;
  unsigned long long wait_ns;      // limit of the peer wait
  void* norm_out;                  // optional: norm(result) * gamma (+ beta), rows aligned with `out`
  const void* gamma;
  const void* beta;
  float eps;
  int norm_mode;                   // 0 none, 1 LayerNorm, 2 RMSNorm (needs N <= 1024)
  // Push mode (small results, N <= 1024): the epilogue stores every partial tile into the receive area of EVERY rank,
  // slot [parity][source rank], as 8-byte words {two 16-bit values, call sequence number}.  A word is written
  // atomically, so a reader that sees the current sequence number in a word also sees its data: no fence, no flag
  // round trip, no atomics; the reduction polls local memory only.  A slot holds M * N / 2 words (4 bytes per value).
  uint8_t* peer_recv[MAX_RANKS];   // base of every rank's receive area, or all null (pull mode)
  long recv_parity_stride;         // bytes between the two parities of a receive area
  long recv_src_stride;            // bytes between source slots
  int push;
};

__device__ __forceinline__ Vec8 ld_volatile_16(const void* p) {
  Vec8 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3])
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void st_volatile_16(void* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint4 ld_volatile_u4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

template <int BN, class T, bool PUSH>
struct PartialProblem {
  static constexpr bool kForceStage = true;      // the push epilogue re-shapes its stores through the stage
  const CUtensorMap* map_a;
  const CUtensorMap* map_b;
  const CommArgs* comm;
  int M, N, m_tiles, n_tiles, num_kb;
  mutable T* part;                 // resolved lazily by the epilogue (after the dependency wait)
  mutable int parity;
  mutable uint32_t seq;             // sequence number of this call (push mode)

  __device__ __forceinline__ int num_tiles() const { return m_tiles * n_tiles; }
  __device__ __forceinline__ void tile(int t, int& m0, int& n0, int& kb0, int& nkb) const {
    m0 = (t % m_tiles) * PG_BM;
    n0 = (t / m_tiles) * BN;
    kb0 = 0;
    nkb = num_kb;
  }
  __device__ __forceinline__ void load_a(uint8_t* smem, uint64_t* bar, int k_elem, int m0) const {
    tma_load_2d(smem, map_a, bar, k_elem, m0);
  }
  __device__ __forceinline__ void load_b(uint8_t* smem, uint64_t* bar, int k_elem, int n0) const {
    tma_load_2d(smem, map_b, bar, k_elem, n0);
  }
  __device__ __forceinline__ void epilogue(int, int m0, int n0, int row, int col, uint32_t (&r)[32], uint8_t* stage) const {
    if (part == nullptr) {
      const int total = *reinterpret_cast<volatile int*>(comm->state);
      parity = total & 1;
      seq = uint32_t(total) + 1u;
      part = reinterpret_cast<T*>(comm->peer_part[comm->rank] + size_t(parity) * comm->part_stride);
    }
    const int gm = m0 + row, gn = n0 + col;
    if (gn >= N) return;                          // uniform across the warp
    if (PUSH) {                                   // launcher guarantees N % 32 == 0 in this mode
      // 64 bytes of this lane's row -> stage; then every rank's receive slot gets the chunk as {data, sequence} words,
      // 4 lanes covering 128 contiguous bytes of a row per store pair
      const int lane = threadIdx.x & 31;
      if (gm < M) {
        uint8_t* mine = stage + lane * 80;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float f[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(r[j * 8 + i]);
          *reinterpret_cast<Vec8*>(mine + j * 16) = pack8<T>(f);
        }
      }
      __syncwarp();
      const int base_row = gm - lane, piece = lane & 3;
      const size_t slot = size_t(parity) * comm->recv_parity_stride + size_t(comm->rank) * comm->recv_src_stride;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int rr = (lane >> 2) + 8 * i;
        if (base_row + rr < M) {
          const Vec8 pk = *reinterpret_cast<const Vec8*>(stage + rr * 80 + piece * 16);
          const size_t off = slot + (size_t(base_row + rr) * N + gn + piece * 8) * 4;     // 4 bytes per value
#pragma unroll 1
          for (int p = 0; p < comm->world; ++p) {
            st_volatile_16(comm->peer_recv[p] + off, pk.w[0], seq, pk.w[1], seq);
            st_volatile_16(comm->peer_recv[p] + off + 16, pk.w[2], seq, pk.w[3], seq);
          }
        }
      }
      __syncwarp();
      return;
    }
    if (gm >= M) return;
    T* dst = part + size_t(gm) * N + gn;
    if (gn + 32 <= N) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float f[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(r[j * 8 + i]);
        *reinterpret_cast<Vec8*>(dst + j * 8) = pack8<T>(f);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (gn + i < N) dst[i] = Cvt<T>::from_f(__uint_as_float(r[i]));
    }
  }
};

// Tail of a reduced 8-value chunk: bias, residual, store, and the row statistics of the stored (rounded) values.
template <class T>
__device__ __forceinline__ void finish_chunk(const CommArgs& comm, float (&acc)[8], int r, int c, T* out, const T* bias,
                                             const T* res, float (&vrow)[8], float& s1, float& s2) {
  if (bias) {
    float f[8];
    unpack8<T>(*reinterpret_cast<const Vec8*>(bias + c), f);
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] += f[k];
  }
  if (res) {
    float f[8];
    unpack8<T>(*reinterpret_cast<const Vec8*>(res + size_t(r) * comm.ld_res + c), f);
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] += f[k];
  }
  const Vec8 o = pack8<T>(acc);
  *reinterpret_cast<Vec8*>(out + size_t(r) * comm.ld_out + c) = o;
  unpack8<T>(o, vrow);                           // normalise exactly what the residual stream stores
#pragma unroll
  for (int k = 0; k < 8; ++k) { s1 += vrow[k]; s2 += vrow[k] * vrow[k]; }
}

// Chunks I0 .. I0 + G - 1 (32 x 16 bytes each) of row r: sum the partials of all ranks in rank order, add bias and
// residual, store the row and keep it (as stored) in v for the norm.
// LL = false: partials are read from the peers' buffers; all peer loads are issued before any is used.
// LL = true : the sources are this rank's receive slots in {data, sequence} words (push mode); the words of a chunk
//             are re-read until every one carries `seq` (bounded by `deadline`; `alive` goes false when it passes).
template <class T, int I0, int G, int W, bool LL>
__device__ __forceinline__ void reduce_row_chunks(const CommArgs& comm, const uint8_t* const (&src_base)[W], int r, int lane,
                                                  int n8, int N, T* out,
                                                  const T* bias, const T* res, float (&v)[4][8], float& s1, float& s2,
                                                  uint32_t seq, unsigned long long deadline, bool& alive,
                                                  uint32_t* status) {
  if (LL) {
    // one polling round covers all G chunks: every load of the round is issued before the first check, so a row costs
    // one local round trip when the data has already landed (the usual case: it arrived during the GEMM)
    float acc[G][8];
    uint32_t polls = 0;
    bool ready;
    do {
      ready = true;
#pragma unroll
      for (int i = 0; i < G; ++i) {
        const int c8 = lane + 32 * (I0 + i);
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[i][k] = 0.f;
        if (c8 < n8) {
          const size_t off = (size_t(comm.row_begin + r) * N + c8 * 8) * 4;
#pragma unroll
          for (int src = 0; src < W; ++src)
            if (src < comm.world) {
              const uint4 lo = ld_volatile_u4(src_base[src] + off);
              const uint4 hi = ld_volatile_u4(src_base[src] + off + 16);
              ready = ready && lo.y == seq && lo.w == seq && hi.y == seq && hi.w == seq;
              Vec8 t;
              t.w[0] = lo.x;
              t.w[1] = lo.z;
              t.w[2] = hi.x;
              t.w[3] = hi.z;
              float f[8];
              unpack8<T>(t, f);
#pragma unroll
              for (int k = 0; k < 8; ++k) acc[i][k] += f[k];
            }
        }
      }
      if (!ready && (++polls & 63u) == 0u && globaltimer_ns() > deadline) {
        if (status) atomicCAS(status, 0u, uint32_t(STATUS_WAIT_PEER));
        alive = false;
      }
    } while (!ready && alive);
#pragma unroll
    for (int i = 0; i < G; ++i) {
      const int c8 = lane + 32 * (I0 + i);
      if (c8 < n8) finish_chunk<T>(comm, acc[i], r, c8 * 8, out, bias, res, v[I0 + i], s1, s2);
    }
  } else {
    Vec8 pk[G][W];                              // W: compile-time bound of the world size (registers)
#pragma unroll
    for (int i = 0; i < G; ++i) {
      const int c8 = lane + 32 * (I0 + i);
      if (c8 < n8) {
        const size_t off = (size_t(comm.row_begin + r) * N + c8 * 8) * sizeof(T);
#pragma unroll
        for (int src = 0; src < W; ++src)
          if (src < comm.world) pk[i][src] = ld_volatile_16(src_base[src] + off);
      }
    }
#pragma unroll
    for (int i = 0; i < G; ++i) {
      const int c8 = lane + 32 * (I0 + i);
      if (c8 < n8) {
        float acc[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] = 0.f;
#pragma unroll
        for (int src = 0; src < W; ++src)
          if (src < comm.world) {
            float f[8];
            unpack8<T>(pk[i][src], f);
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[k] += f[k];
          }
        finish_chunk<T>(comm, acc, r, c8 * 8, out, bias, res, v[I0 + i], s1, s2);
      }
    }
  }
}

// Cross-rank phase shared by the fused GEMM kernel and the stand-alone reduction kernel.  On entry every thread of the
// CTA has issued its stores of this rank's partial result (and passed a CTA barrier).  All CTAs of the grid must be
// resident at once: the phase waits on work of the whole grid and of the peers.
template <class T, int W, bool PUSH>
__device__ __forceinline__ void cross_rank_phase(const CommArgs& comm, int M, int N, uint32_t* status, int& s_flag) {
  pdl_wait();
  const int total = *reinterpret_cast<volatile int*>(comm.state);
  const int parity = total & 1;
  // flag value this call waits for: the flag calls (pull mode) completed on this parity, plus one; push-mode calls do
  // not touch the flags, so they are not counted
  const int want = PUSH ? 0 : *reinterpret_cast<volatile int*>(comm.state + 4 + parity) + 1;
  const uint32_t seq = uint32_t(total) + 1u;
  const unsigned long long deadline = globaltimer_ns() + comm.wait_ns;
  bool alive = true;
  if (PUSH) {
    // push mode: the data words carry the sequence number themselves; nothing to signal and nothing to wait for here
    if (threadIdx.x == 0) s_flag = 1;
  } else if (threadIdx.x == 0) {
    __threadfence_system();
    const int done = atomicAdd(comm.state + 1, 1);
    if (done == int(gridDim.x) - 1) {            // last CTA of this rank: tell every rank our partials are complete
      comm.state[1] = 0;
      __threadfence_system();
      for (int p = 0; p < comm.world; ++p)
        atomicAdd_system(comm.peer_flags[p] + parity * MAX_RANKS + comm.rank, 1);
    }
    // ---- phase 2: wait for the partials of every rank (bounded)
    const int* flags = comm.peer_flags[comm.rank] + parity * MAX_RANKS;
    const unsigned long long t0 = globaltimer_ns();
    int ok = 1;
    for (int src = 0; src < comm.world && ok; ++src) {
      unsigned polls = 0;
      while (ld_acquire_sys(flags + src) < want) {
        if ((++polls & 63u) == 0u && globaltimer_ns() - t0 > comm.wait_ns) {
          if (status) atomicCAS(status, 0u, uint32_t(STATUS_WAIT_PEER));
          ok = 0;
          break;
        }
      }
    }
    s_flag = ok;
  }
  __syncthreads();
  if (s_flag) {
    const int rows = comm.row_end - comm.row_begin;
    const int n8 = N >> 3;
    // where the partials of source rank `src` are read from: this rank's receive slots (push) or the peers' buffers
    const uint8_t* src_base[W];
#pragma unroll
    for (int src = 0; src < W; ++src) {
      src_base[src] = nullptr;
      if (src < comm.world)
        src_base[src] = PUSH ? comm.peer_recv[comm.rank] + size_t(parity) * comm.recv_parity_stride +
                                        size_t(src) * comm.recv_src_stride
                                  : comm.peer_part[src] + size_t(parity) * comm.part_stride;
    }
    T* out = reinterpret_cast<T*>(comm.out);
    const T* bias = reinterpret_cast<const T*>(comm.bias);
    const T* res = reinterpret_cast<const T*>(comm.residual);
    if (n8 <= 32 * 4) {
      // ---- one warp per row: the whole row stays in registers, so the norm of the next block is applied here too
      const int lane = threadIdx.x & 31;
      const int warps = int(gridDim.x) * (PG_THREADS / 32);
      const T* gamma = reinterpret_cast<const T*>(comm.gamma);
      const T* beta = reinterpret_cast<const T*>(comm.beta);
      T* nout = reinterpret_cast<T*>(comm.norm_out);
      for (int r = int(blockIdx.x) * (PG_THREADS / 32) + (threadIdx.x >> 5); r < rows; r += warps) {
        float v[4][8];
        float s1 = 0.f, s2 = 0.f;
        // Peer loads cost an NVLink round trip each: every load of a group of chunks (all ranks) is issued before the
        // first one is used, so a row pays one or two round trips instead of one per chunk.
        if (PUSH) {
          if (W <= 4) {
            reduce_row_chunks<T, 0, 4, W, true>(comm, src_base, r, lane, n8, N, out, bias, res, v, s1, s2, seq, deadline, alive, status);
          } else {
            reduce_row_chunks<T, 0, 2, W, true>(comm, src_base, r, lane, n8, N, out, bias, res, v, s1, s2, seq, deadline, alive, status);
            reduce_row_chunks<T, 2, 2, W, true>(comm, src_base, r, lane, n8, N, out, bias, res, v, s1, s2, seq, deadline, alive, status);
          }
        } else if (W <= 4) {
          reduce_row_chunks<T, 0, 4, W, false>(comm, src_base, r, lane, n8, N, out, bias, res, v, s1, s2, seq, deadline, alive, status);
        } else {
          reduce_row_chunks<T, 0, 2, W, false>(comm, src_base, r, lane, n8, N, out, bias, res, v, s1, s2, seq, deadline, alive, status);
          reduce_row_chunks<T, 2, 2, W, false>(comm, src_base, r, lane, n8, N, out, bias, res, v, s1, s2, seq, deadline, alive, status);
        }
        if (comm.norm_mode != 0) {
          float mean = 0.f, inv;
          if (comm.norm_mode == 2) {
            inv = rsqrtf(warp_sum(s2) / float(N) + comm.eps);
          } else {
            mean = warp_sum(s1) / float(N);
            float q = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i)
              if (lane + 32 * i < n8) {
#pragma unroll
                for (int k = 0; k < 8; ++k) { const float d = v[i][k] - mean; q += d * d; }
              }
            inv = rsqrtf(warp_sum(q) / float(N) + comm.eps);
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int c8 = lane + 32 * i;
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
              *reinterpret_cast<Vec8*>(nout + size_t(r) * comm.ld_out + c8 * 8) = pack8<T>(o);
            }
          }
        }
      }
    } else {
      const long vecs = long(rows) * n8;
      for (long v = long(blockIdx.x) * blockDim.x + threadIdx.x; v < vecs; v += long(gridDim.x) * blockDim.x) {
        const int r = int(v / n8), c = int(v - long(r) * n8) * 8;
        const size_t off = (size_t(comm.row_begin + r) * N + c) * sizeof(T);
        Vec8 pk[W];
#pragma unroll
        for (int src = 0; src < W; ++src)
          if (src < comm.world) pk[src] = ld_volatile_16(src_base[src] + off);
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0.f;
#pragma unroll
        for (int src = 0; src < W; ++src)
          if (src < comm.world) {
            float f[8];
            unpack8<T>(pk[src], f);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] += f[i];
          }
        if (bias) {
          float f[8];
          unpack8<T>(*reinterpret_cast<const Vec8*>(bias + c), f);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] += f[i];
        }
        if (res) {
          float f[8];
          unpack8<T>(*reinterpret_cast<const Vec8*>(res + size_t(r) * comm.ld_res + c), f);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] += f[i];
        }
        *reinterpret_cast<Vec8*>(out + size_t(r) * comm.ld_out + c) = pack8<T>(acc);
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const int done = atomicAdd(comm.state + 2, 1);
    if (done == int(gridDim.x) - 1) {            // last CTA: the call is complete on this rank
      comm.state[2] = 0;
      if (!PUSH) comm.state[4 + parity] = want;
      __threadfence();
      *reinterpret_cast<volatile int*>(comm.state) = total + 1;
    }
  }
}

// W: compile-time bound of the world size (2, 4 or 8); it sizes the register arrays of the reduction phase.
template <int BN, int STAGES, class T, int W, bool PUSH>
__global__ void __launch_bounds__(PG_THREADS)
gemm_reduce_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                   const __grid_constant__ CommArgs comm, int M, int N, int K, uint32_t idesc, uint32_t* status) {
  extern __shared__ uint8_t dyn_smem[];
  __shared__ int s_flag;
  PartialProblem<BN, T, PUSH> prob;
  prob.map_a = &map_a;
  prob.map_b = &map_b;
  prob.comm = &comm;
  prob.M = M;
  prob.N = N;
  prob.m_tiles = (M + PG_BM - 1) / PG_BM;
  prob.n_tiles = (N + BN - 1) / BN;
  prob.num_kb = (K + 63) / 64;
  prob.part = nullptr;
  gemm_persistent<BN, STAGES, 0, PartialProblem<BN, T, PUSH>>(dyn_smem, prob, 64, idesc, status);
  // ---- end of phase 1: every thread of this CTA has issued its partial stores (teardown barrier passed)
  cross_rank_phase<T, W, PUSH>(comm, M, N, status, s_flag);
}

// Reduction of partial results that another kernel of this rank (e.g. the ternary BitLinear GEMM) has written into the
// current parity slot of this rank's partial buffer: flags, bounded wait, rank-ordered sum from peer memory, bias,
// residual and optional norm.  grid <= resident CTAs.
template <class T, int W>
__global__ void __launch_bounds__(PG_THREADS)
peer_reduce_kernel(const __grid_constant__ CommArgs comm, int M, int N, uint32_t* status) {
  __shared__ int s_flag;
  pdl_wait();                                    // the producer of the partials is the previous kernel in the stream
  pdl_trigger();
  __syncthreads();
  cross_rank_phase<T, W, false>(comm, M, N, status, s_flag);
}

static int comm_sm_count() { return device_sm_count(); }

template <int BN, int STAGES, class T, int W, bool PUSH>
static int launch_reduce_w(const CUtensorMap& ma, const CUtensorMap& mb, const CommArgs& comm, int M, int N, int K,
                           int is_bf16, uint32_t* status, cudaStream_t stream) {
  using L = PGemmSmem<BN, STAGES, true>;
  auto kern = gemm_reduce_kernel<BN, STAGES, T, W, PUSH>;
  static bool configured[MAX_DEVICES] = {false};
  if (first_use_on_device(configured)) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYN_SMEM) != cudaSuccess) return -10;
  }
  const int tiles = ((N + BN - 1) / BN) * ((M + PG_BM - 1) / PG_BM);
  // every CTA must be resident at once (phase 2 waits on work of the whole grid): never exceed one wave
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, PG_THREADS, L::DYN_SMEM) != cudaSuccess || per_sm < 1)
    return -12;
  if (per_sm > 2) per_sm = 2;
  const int resident = comm_sm_count() * per_sm;
  dim3 grid(tiles < resident ? tiles : resident);
  uint32_t idesc = umma_idesc(PG_BM, BN, is_bf16 ? 1u : 0u, 1u);
  cudaError_t err = launch(kern, grid, dim3(PG_THREADS), size_t(L::DYN_SMEM), stream, ma, mb, comm, M, N, K, idesc, status);
  return (err == cudaSuccess && cudaGetLastError() == cudaSuccess) ? 0 : -11;
}

template <int BN, int STAGES, class T>
static int launch_reduce(const CUtensorMap& ma, const CUtensorMap& mb, const CommArgs& comm, int M, int N, int K,
                         int is_bf16, uint32_t* status, cudaStream_t stream) {
  if (comm.push) {
    if (comm.world <= 2) return launch_reduce_w<BN, STAGES, T, 2, true>(ma, mb, comm, M, N, K, is_bf16, status, stream);
    if (comm.world <= 4) return launch_reduce_w<BN, STAGES, T, 4, true>(ma, mb, comm, M, N, K, is_bf16, status, stream);
    return launch_reduce_w<BN, STAGES, T, 8, true>(ma, mb, comm, M, N, K, is_bf16, status, stream);
  }
  if (comm.world <= 2) return launch_reduce_w<BN, STAGES, T, 2, false>(ma, mb, comm, M, N, K, is_bf16, status, stream);
  if (comm.world <= 4) return launch_reduce_w<BN, STAGES, T, 4, false>(ma, mb, comm, M, N, K, is_bf16, status, stream);
  return launch_reduce_w<BN, STAGES, T, 8, false>(ma, mb, comm, M, N, K, is_bf16, status, stream);
}

}  // namespace ronn

using namespace ronn;

// peer_part / peer_flags: `world` pointers each.  part_stride: bytes between the two parity slots of a partial
// buffer (>= M * N * 2).  state: eight zero-initialised ints in local device memory, shared by all calls on this
// rank.  Rows [row_begin, row_end) of the reduced result (+ bias + residual) are written to `out`.
// With norm_mode 1 (LayerNorm) / 2 (RMSNorm) and N <= 1024 the normalised rows are also written to norm_out.
// dtype 0 bf16, 1 fp16.  N % 8 == 0.  Returns 0 on success.
static int gemm_reduce_impl(const void* A, const void* W, int M, int N, int K, int lda, int ldw,
                            void* const* peer_part, int* const* peer_flags, long part_stride, int* state,
                            int rank, int world, int row_begin, int row_end, void* out, long ld_out,
                            const void* bias, const void* residual, long ld_res, double wait_seconds, int dtype,
                            int bn, void* norm_out, const void* gamma, const void* beta, float eps, int norm_mode,
                            void* const* peer_recv, long recv_parity_stride, long recv_src_stride,
                            uint32_t* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || world < 1 || world > MAX_RANKS || rank < 0 || rank >= world) return -1;
  if ((K & 7) || (lda & 7) || (ldw & 7) || (N & 7) || (ld_out & 7) || (residual && (ld_res & 7))) return -2;
  if (norm_mode != 0 && (N > 1024 || norm_out == nullptr)) return -5;
  if (row_begin < 0 || row_end > M || row_begin > row_end || part_stride < long(M) * N * 2) return -4;
  if (bn == 0) {
    const int mt = (M + PG_BM - 1) / PG_BM;
    bn = 128;
    while (bn > 32 && mt * ((N + bn - 1) / bn) < 96) bn >>= 1;
  }
  CUtensorMap ma, mb;
  int rc = make_tmap_2d(&ma, A, uint64_t(M), uint64_t(K), uint64_t(lda), PG_BM, 64, 2);
  if (rc) return rc - 20;
  rc = make_tmap_2d(&mb, W, uint64_t(N), uint64_t(K), uint64_t(ldw), uint32_t(bn), 64, 2);
  if (rc) return rc - 30;
  CommArgs c;
  for (int p = 0; p < MAX_RANKS; ++p) {
    c.peer_part[p] = p < world ? static_cast<uint8_t*>(peer_part[p]) : nullptr;
    c.peer_flags[p] = p < world ? peer_flags[p] : nullptr;
  }
  c.push = peer_recv != nullptr ? 1 : 0;
  // push mode: a slot holds 4 bytes per value; whole 32-column chunks and the row-wise reduction (N <= 1024) only
  if (c.push && (recv_src_stride < long(M) * N * 4 || recv_parity_stride < recv_src_stride * world || (N & 31) ||
                 N > 1024))
    return -6;
  for (int p = 0; p < MAX_RANKS; ++p)
    c.peer_recv[p] = (c.push && p < world) ? static_cast<uint8_t*>(peer_recv[p]) : nullptr;
  c.recv_parity_stride = recv_parity_stride;
  c.recv_src_stride = recv_src_stride;
  c.part_stride = part_stride;
  c.state = state;
  c.rank = rank;
  c.world = world;
  c.row_begin = row_begin;
  c.row_end = row_end;
  c.out = out;
  c.ld_out = ld_out;
  c.bias = bias;
  c.residual = residual;
  c.ld_res = ld_res;
  c.wait_ns = static_cast<unsigned long long>(wait_seconds * 1e9);
  c.norm_out = norm_out;
  c.gamma = gamma;
  c.beta = beta;
  c.eps = eps;
  c.norm_mode = norm_mode;
  const int bf = dtype == 0;
#define RONN_DISPATCH(BN_, ST_)                                                                        \
  return bf ? launch_reduce<BN_, ST_, __nv_bfloat16>(ma, mb, c, M, N, K, 1, status, stream)           \
            : launch_reduce<BN_, ST_, __half>(ma, mb, c, M, N, K, 0, status, stream)
  switch (bn) {
    case 128: RONN_DISPATCH(128, 3);
    case 64: RONN_DISPATCH(64, 4);
    case 32: RONN_DISPATCH(32, 5);
    default: return -3;
  }
#undef RONN_DISPATCH
}

extern "C" int ronn_gemm_reduce(const void* A, const void* W, int M, int N, int K, int lda, int ldw,
                                void* const* peer_part, int* const* peer_flags, long part_stride, int* state,
                                int rank, int world, int row_begin, int row_end, void* out, long ld_out,
                                const void* bias, const void* residual, long ld_res, double wait_seconds, int dtype,
                                int bn, void* norm_out, const void* gamma, const void* beta, float eps, int norm_mode,
                                uint32_t* status, cudaStream_t stream) {
  return gemm_reduce_impl(A, W, M, N, K, lda, ldw, peer_part, peer_flags, part_stride, state, rank, world, row_begin,
                          row_end, out, ld_out, bias, residual, ld_res, wait_seconds, dtype, bn, norm_out, gamma, beta, eps,
                          norm_mode, nullptr, 0, 0, status, stream);
}

// Push variant for small results (N a multiple of 32, at most 1024): peer_recv[p] is rank p's receive area of
// 2 parities x `world` source slots (recv_parity_stride / recv_src_stride bytes apart, a slot holds 4 bytes per
// value).  Every partial tile is stored into all ranks' slots by the GEMM epilogue as {data, sequence} words; the
// reduction polls local memory only (no fence, no flags, no atomics between the ranks).
extern "C" int ronn_gemm_reduce_push(const void* A, const void* W, int M, int N, int K, int lda, int ldw,
                                     void* const* peer_part, int* const* peer_flags, long part_stride, int* state,
                                     int rank, int world, int row_begin, int row_end, void* out, long ld_out,
                                     const void* bias, const void* residual, long ld_res, double wait_seconds,
                                     int dtype, int bn, void* norm_out, const void* gamma, const void* beta, float eps,
                                     int norm_mode, void* const* peer_recv, long recv_parity_stride,
                                     long recv_src_stride, uint32_t* status, cudaStream_t stream) {
  if (peer_recv == nullptr) return -6;
  return gemm_reduce_impl(A, W, M, N, K, lda, ldw, peer_part, peer_flags, part_stride, state, rank, world, row_begin,
                          row_end, out, ld_out, bias, residual, ld_res, wait_seconds, dtype, bn, norm_out, gamma, beta, eps,
                          norm_mode, peer_recv, recv_parity_stride, recv_src_stride, status, stream);
}

// Cross-rank reduction of partial results that are already in the current parity slot of every rank's partial buffer
// (written by the previous kernel on the stream, e.g. ronn_bitlinear_to_slot).  Same arguments and semantics as the
// reduction half of ronn_gemm_reduce.
extern "C" int ronn_peer_reduce(int M, int N, void* const* peer_part, int* const* peer_flags, long part_stride, int* state,
                                int rank, int world, int row_begin, int row_end, void* out, long ld_out, const void* bias,
                                const void* residual, long ld_res, double wait_seconds, int dtype, void* norm_out,
                                const void* gamma, const void* beta, float eps, int norm_mode, uint32_t* status,
                                cudaStream_t stream) {
  if (M <= 0 || N <= 0 || world < 1 || world > MAX_RANKS || rank < 0 || rank >= world) return -1;
  if ((N & 7) || (ld_out & 7) || (residual && (ld_res & 7))) return -2;
  if (norm_mode != 0 && (N > 1024 || norm_out == nullptr)) return -5;
  if (row_begin < 0 || row_end > M || row_begin > row_end || part_stride < long(M) * N * 2) return -4;
  CommArgs c;
  for (int p = 0; p < MAX_RANKS; ++p) {
    c.peer_part[p] = p < world ? static_cast<uint8_t*>(peer_part[p]) : nullptr;
    c.peer_flags[p] = p < world ? peer_flags[p] : nullptr;
    c.peer_recv[p] = nullptr;
  }
  c.push = 0;
  c.recv_parity_stride = c.recv_src_stride = 0;
  c.part_stride = part_stride;
  c.state = state;
  c.rank = rank;
  c.world = world;
  c.row_begin = row_begin;
  c.row_end = row_end;
  c.out = out;
  c.ld_out = ld_out;
  c.bias = bias;
  c.residual = residual;
  c.ld_res = ld_res;
  c.wait_ns = static_cast<unsigned long long>(wait_seconds * 1e9);
  c.norm_out = norm_out;
  c.gamma = gamma;
  c.beta = beta;
  c.eps = eps;
  c.norm_mode = norm_mode;
  const int rows = row_end - row_begin;
  const int warps_per_cta = PG_THREADS / 32;
  int grid = N <= 1024 ? (rows + warps_per_cta - 1) / warps_per_cta : int((long(rows) * (N >> 3) + PG_THREADS - 1) / PG_THREADS);
  if (grid > comm_sm_count()) grid = comm_sm_count();         // every CTA resident at once
  if (grid < 1) grid = 1;
  cudaError_t err;
#define RONN_PR(T_, W_) err = launch(peer_reduce_kernel<T_, W_>, dim3(grid), dim3(PG_THREADS), 0, stream, c, M, N, status)
  if (dtype == 0) {
    if (world <= 2) RONN_PR(__nv_bfloat16, 2); else if (world <= 4) RONN_PR(__nv_bfloat16, 4); else RONN_PR(__nv_bfloat16, 8);
  } else {
    if (world <= 2) RONN_PR(__half, 2); else if (world <= 4) RONN_PR(__half, 4); else RONN_PR(__half, 8);
  }
#undef RONN_PR
  return (err == cudaSuccess && cudaGetLastError() == cudaSuccess) ? 0 : -11;
}

// Greedy token over vocabulary shards without a library collective: every rank stores its (max, index) pair of each row
// into every rank's exchange slot as two 8-byte words {max, sequence} {index, sequence}, then polls its own slots until
// the words of all ranks carry this call's sequence number and keeps the largest value (lowest index on ties), so all
// ranks pick the same token.  state: two zero-initialised ints in local memory ([0] calls completed, [1] block counter).
// Slot layout per rank: [2 parities][world sources][max_rows] records of 16 bytes.
struct ArgmaxExchangeArgs {
  uint8_t* peer_slots[MAX_RANKS];
  int* state;
  int rank, world, rows, max_rows;
  unsigned long long wait_ns;
};

__global__ void __launch_bounds__(256)
argmax_exchange_kernel(const __grid_constant__ ArgmaxExchangeArgs a, const int* __restrict__ idx,
                       const float* __restrict__ mx, int* __restrict__ tokens, uint32_t* status) {
  pdl_wait();
  pdl_trigger();
  const int total = *reinterpret_cast<volatile int*>(a.state);
  const uint32_t seq = uint32_t(total) + 1u;
  const size_t parity_off = size_t(total & 1) * a.world * a.max_rows * 16;
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b < a.rows) {
    const uint32_t vbits = __float_as_uint(mx[b]);
    const uint32_t ibits = uint32_t(idx[b]);
    const size_t mine = parity_off + (size_t(a.rank) * a.max_rows + b) * 16;
    for (int p = 0; p < a.world; ++p) st_volatile_16(a.peer_slots[p] + mine, vbits, seq, ibits, seq);
    const unsigned long long deadline = globaltimer_ns() + a.wait_ns;
    float best = -INFINITY;
    int best_idx = 0x7fffffff;
    bool alive = true;
    for (int src = 0; src < a.world && alive; ++src) {
      const uint8_t* slot = a.peer_slots[a.rank] + parity_off + (size_t(src) * a.max_rows + b) * 16;
      uint4 w = ld_volatile_u4(slot);
      uint32_t polls = 0;
      while (w.y != seq || w.w != seq) {
        if ((++polls & 63u) == 0u && globaltimer_ns() > deadline) {
          if (status) atomicCAS(status, 0u, uint32_t(STATUS_WAIT_PEER));
          alive = false;
          break;
        }
        w = ld_volatile_u4(slot);
      }
      const float v = __uint_as_float(w.x);
      const int i = int(w.z);
      if (alive && (v > best || (v == best && i < best_idx))) {
        best = v;
        best_idx = i;
      }
    }
    tokens[b] = alive ? best_idx : 0;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const int done = atomicAdd(a.state + 1, 1);
    if (done == int(gridDim.x) - 1) {
      a.state[1] = 0;
      __threadfence();
      *reinterpret_cast<volatile int*>(a.state) = total + 1;
    }
  }
}

// idx / mx: this rank's best index (global vocabulary index) and value per row; tokens: int32 [rows] result, the same
// on every rank.  peer_slots: `world` pointers to the ranks' exchange areas (2 * world * max_rows * 16 bytes each).
extern "C" int ronn_argmax_exchange(const int* idx, const float* mx, int* tokens, int rows, void* const* peer_slots,
                                    int max_rows, int* state, int rank, int world, double wait_seconds, uint32_t* status,
                                    cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (rows > max_rows || world < 1 || world > MAX_RANKS || rank < 0 || rank >= world) return -1;
  const int blocks = (rows + 255) / 256;
  if (blocks > comm_sm_count()) return -2;       // every block resident at once (they wait on the peers)
  ArgmaxExchangeArgs a;
  for (int p = 0; p < MAX_RANKS; ++p) a.peer_slots[p] = p < world ? static_cast<uint8_t*>(peer_slots[p]) : nullptr;
  a.state = state;
  a.rank = rank;
  a.world = world;
  a.rows = rows;
  a.max_rows = max_rows;
  a.wait_ns = static_cast<unsigned long long>(wait_seconds * 1e9);
  cudaError_t err = launch(argmax_exchange_kernel, dim3(blocks), dim3(256), 0, stream, a, idx, mx, tokens, status);
  return (err == cudaSuccess && cudaGetLastError() == cudaSuccess) ? 0 : -11;
}

// =====================================================================================================================
// Column-parallel all-gather -> GEMM in ONE kernel.
//
//   Y[T, N_local] = concat_r(X_r)[T, K] * W[N_local, K]^T (+ bias, activation)
//
// Every rank holds a row shard X_r [T / world, K] in a symmetric buffer.  The gathered activation matrix is never
// materialised: the TMA producer of each output tile reads the A rows it needs straight from the owning rank's
// buffer through a per-peer tensor map (plain cp.async.bulk.tensor loads, no multicast).  Before the first load from
// a peer it waits (bounded) for that peer's "shard ready" flag, so tiles whose rows are local start at once and the
// NVLink traffic of the remaining tiles overlaps their math.  Flags are raised by ronn_signal_peers, launched on the
// producing rank right after the kernel that wrote the shard.
//
// The symmetric shard buffer is single-buffered: a caller must put a cross-rank synchronising operation (the fused
// row-parallel GEMM above) between two gathers, which a transformer block does by construction.
namespace ronn {

struct GatherArgs {
  CUtensorMap map_a[MAX_RANKS];    // [rows_per_rank, K] view of every rank's shard buffer
  const int* flags;                // local: [MAX_RANKS] arrival counters, one per source rank
  int* state;                      // local: [0] gathers completed, [1] CTA counter
  int rows_per_rank, world, rank;
  unsigned long long wait_ns;
};

template <int BN, class T>
struct GatherProblem {
  static constexpr bool kForceStage = true;
  const GatherArgs* g;
  const CUtensorMap* map_b;
  DenseEpilogue e;
  int m_tiles, n_tiles, num_kb;
  uint32_t* status;
  mutable int ready_mask;          // peers whose shard has been seen ready by this thread
  mutable int want;

  __device__ __forceinline__ int num_tiles() const { return m_tiles * n_tiles; }
  __device__ __forceinline__ void tile(int t, int& m0, int& n0, int& kb0, int& nkb) const {
    // start with the tiles whose rows are local, then walk the peers round-robin from there
    const int per = m_tiles / g->world;              // m-tiles per rank (rows_per_rank % 128 == 0)
    const int mt = t % m_tiles;
    const int owner = (mt / per + g->rank) % g->world;
    m0 = (owner * per + mt % per) * PG_BM;
    n0 = (t / m_tiles) * BN;
    kb0 = 0;
    nkb = num_kb;
  }
  __device__ __forceinline__ void load_a(uint8_t* smem, uint64_t* bar, int k_elem, int m0) const {
    const int owner = m0 / g->rows_per_rank;
    if (!(ready_mask & (1 << owner))) {
      if (want < 0) want = *reinterpret_cast<volatile int*>(g->state) + 1;
      const unsigned long long t0 = globaltimer_ns();
      unsigned polls = 0;
      while (ld_acquire_sys(g->flags + owner) < want) {
        if ((++polls & 63u) == 0u && globaltimer_ns() - t0 > g->wait_ns) {
          if (status) atomicCAS(status, 0u, uint32_t(STATUS_WAIT_PEER));
          break;                                       // proceed: the result is flagged invalid through the status word
        }
      }
      ready_mask |= 1 << owner;
    }
    tma_load_2d(smem, &g->map_a[owner], bar, k_elem, m0 - owner * g->rows_per_rank);
  }
  __device__ __forceinline__ void load_b(uint8_t* smem, uint64_t* bar, int k_elem, int n0) const {
    tma_load_2d(smem, map_b, bar, k_elem, n0);
  }
  __device__ __forceinline__ void epilogue(int, int m0, int n0, int row, int col, uint32_t (&r)[32], uint8_t* stage) const {
    DenseEpilogue ep = e;
    ep.m0 = m0;
    ep.n0 = n0;
    ep.run<T>(row, col, r, stage);
  }
};

template <int BN, int STAGES, class T>
__global__ void __launch_bounds__(PG_THREADS)
ag_gemm_kernel(const __grid_constant__ GatherArgs g, const __grid_constant__ CUtensorMap map_b, DenseEpilogue epi,
               int K, uint32_t idesc, uint32_t* status) {
  extern __shared__ uint8_t dyn_smem[];
  GatherProblem<BN, T> prob;
  prob.g = &g;
  prob.map_b = &map_b;
  prob.e = epi;
  prob.m_tiles = (epi.M + PG_BM - 1) / PG_BM;
  prob.n_tiles = (epi.N + BN - 1) / BN;
  prob.num_kb = (K + 63) / 64;
  prob.status = status;
  prob.ready_mask = 0;
  prob.want = -1;
  gemm_persistent<BN, STAGES, 0, GatherProblem<BN, T>>(dyn_smem, prob, 64, idesc, status);
  if (threadIdx.x == 0) {
    const int done = atomicAdd(g.state + 1, 1);
    if (done == int(gridDim.x) - 1) {                  // last CTA: this gather is complete on this rank
      g.state[1] = 0;
      __threadfence();
      *reinterpret_cast<volatile int*>(g.state) = *reinterpret_cast<volatile int*>(g.state) + 1;
    }
  }
}

// One thread: make this rank's earlier writes visible system-wide, then bump its arrival counter on every rank.
struct PeerFlagPtrs {
  int* p[MAX_RANKS];
};
__global__ void signal_peers_kernel2(PeerFlagPtrs ptrs, int world, int rank) {
  pdl_wait();
  __threadfence_system();
  for (int p = 0; p < world; ++p) atomicAdd_system(ptrs.p[p] + rank, 1);
}

template <int BN, int STAGES, class T>
static int launch_ag(const GatherArgs& g, const CUtensorMap& mb, DenseEpilogue e, int M, int N, int K, int is_bf16,
                     uint32_t* status, cudaStream_t stream) {
  using L = PGemmSmem<BN, STAGES, true>;
  auto kern = ag_gemm_kernel<BN, STAGES, T>;
  static bool configured[MAX_DEVICES] = {false};
  if (first_use_on_device(configured)) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYN_SMEM) != cudaSuccess) return -10;
  }
  const int tiles = ((N + BN - 1) / BN) * ((M + PG_BM - 1) / PG_BM);
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, PG_THREADS, L::DYN_SMEM) != cudaSuccess || per_sm < 1)
    return -12;
  if (per_sm > 2) per_sm = 2;
  const int resident = comm_sm_count() * per_sm;
  dim3 grid(tiles < resident ? tiles : resident);
  uint32_t idesc = umma_idesc(PG_BM, BN, is_bf16 ? 1u : 0u, 1u);
  cudaError_t err = launch(kern, grid, dim3(PG_THREADS), size_t(L::DYN_SMEM), stream, g, mb, e, K, idesc, status);
  return (err == cudaSuccess && cudaGetLastError() == cudaSuccess) ? 0 : -11;
}

}  // namespace ronn

// peer_shards: `world` pointers to every rank's [rows_per_rank, K] shard (row stride ld_shard elements).
// flags: this rank's arrival counters (MAX_RANKS ints, symmetric memory); state: two zero-initialised local ints.
// rows_per_rank % 128 == 0.  Output C [world * rows_per_rank, N] (+bias, activation) in dtype (0 bf16, 1 fp16).
extern "C" int ronn_ag_gemm(void* const* peer_shards, int ld_shard, const void* W, int ldw, void* C, int ldc,
                            const void* bias, int rows_per_rank, int N, int K, int rank, int world, const int* flags,
                            int* state, int act, double wait_seconds, int dtype, int bn, uint32_t* status,
                            cudaStream_t stream) {
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world || rows_per_rank <= 0 || (rows_per_rank % PG_BM)) return -1;
  if ((K & 7) || (ld_shard & 7) || (ldw & 7) || (ldc & 7)) return -2;
  const int M = rows_per_rank * world;
  if (bn == 0) {
    const int mt = M / PG_BM;
    bn = 256;
    while (bn > 32 && (N < bn || mt * ((N + bn - 1) / bn) < 120)) bn >>= 1;
    if (bn > 128) bn = 128;
  }
  GatherArgs g;
  for (int p = 0; p < MAX_RANKS; ++p) {
    const void* base = peer_shards[p < world ? p : 0];
    int rc = make_tmap_2d(&g.map_a[p], base, uint64_t(rows_per_rank), uint64_t(K), uint64_t(ld_shard), PG_BM, 64, 2);
    if (rc) return rc - 20;
  }
  g.flags = flags;
  g.state = state;
  g.rows_per_rank = rows_per_rank;
  g.world = world;
  g.rank = rank;
  g.wait_ns = static_cast<unsigned long long>(wait_seconds * 1e9);
  CUtensorMap mb;
  int rc = make_tmap_2d(&mb, W, uint64_t(N), uint64_t(K), uint64_t(ldw), uint32_t(bn), 64, 2);
  if (rc) return rc - 30;
  DenseEpilogue e{C, bias, nullptr, M, N, ldc, 0, 0, act, 0, 0};
  const int bf = dtype == 0;
#define RONN_DISPATCH(BN_, ST_)                                                                  \
  return bf ? launch_ag<BN_, ST_, __nv_bfloat16>(g, mb, e, M, N, K, 1, status, stream)          \
            : launch_ag<BN_, ST_, __half>(g, mb, e, M, N, K, 0, status, stream)
  switch (bn) {
    case 128: RONN_DISPATCH(128, 3);
    case 64: RONN_DISPATCH(64, 4);
    case 32: RONN_DISPATCH(32, 5);
    default: return -3;
  }
#undef RONN_DISPATCH
}

// Raise this rank's "shard ready" counter on every rank (stream-ordered after the kernel that wrote the shard).
extern "C" int ronn_signal_peers(int* const* peer_flags, int rank, int world, cudaStream_t stream) {
  if (world < 1 || world > MAX_RANKS) return -1;
  PeerFlagPtrs ptrs;
  for (int p = 0; p < MAX_RANKS; ++p) ptrs.p[p] = p < world ? peer_flags[p] : nullptr;
  cudaError_t err = launch(signal_peers_kernel2, dim3(1), dim3(1), 0, stream, ptrs, world, rank);
  return err == cudaSuccess ? 0 : -100;
}
