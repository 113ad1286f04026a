// Row-parallel GEMM fused with a low-latency two-phase all-reduce over NVLink, bias, residual and LayerNorm /
// RMSNorm, in ONE kernel, for decode-sized results (tensor parallel, W ranks).
//
//   X = sum over ranks of A_r[M, K_r] * W_r[N, K_r]^T + bias + residual ,  H = norm(X) * gamma (+ beta)
//
// No fence, no flag and no atomic lies between the ranks: every 8-byte word that crosses NVLink carries two 16-bit
// values and the call's sequence number, a word is written atomically, and a reader polls its OWN memory until the
// words it needs carry the current number.  The latency chain of a call is therefore two one-way NVLink trips:
//
//   phase A  the GEMM epilogue (tcgen05 accumulators from TMEM) stores each partial row, as {data, sequence} words,
//            into the receive area of the rank that OWNS the row (rank r owns rows [r M / W, (r + 1) M / W)): each
//            rank sends (W - 1) / W of one result instead of W - 1 whole copies.  A rank may cut its K range into S
//            slices (S W <= 8): every (rank, slice) pair is then one source, the K chain of a CTA is S times shorter
//            and S times as many CTAs stream the weights
//   phase B  the owner polls its receive area, sums the W partials in rank order, adds bias and residual, and stores
//            the finished row of X, again as {data, sequence} words, into every rank's result area: one multimem.st
//            per 16 bytes through the NVSwitch (NVLS), or W peer stores
//   phase C  every rank polls its result area, unpacks X into its local output and computes H row by row
//
// All ranks hold the same bits because only the owner computes a row.  Areas alternate between two parities per
// call: a rank can be at most one call ahead of a peer (phase C of call k needs every owner's phase B of call k).
// The sequence number comes from an epoch word in local device memory that the leaving CTAs advance, so CUDA-graph
// replays need no host arguments.  Every poll is bounded and reports STATUS_WAIT_PEER through the status word.
// No TMA multicast is used; peer memory is only ever written (plain or multimem stores), never read.
//
// The reference has no collective of any kind (crates/ronn-providers/src/gpu/provider.rs:226-249).
#include "gemm_ll.h"

#include "comm_ptx.cuh"
#include "tma_desc.cuh"
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
  unsigned long long wait_ns;
  long ld_out, ld_res;
  float eps;
  int M, N, rank, world, owner_rows, row_begin, row_end;
  int norm_mode, nvls, wpr, phases;
  int S, kb_per, num_kb;                 // K slices per rank: every (rank, slice) pair is one source of phase A
};

template <int BN, class T>
struct LLProblem {
  static constexpr bool kForceStage = true;      // the epilogue re-shapes its stores through the per-warp stage
  const CUtensorMap* map_a;
  const CUtensorMap* map_b;
  const LLArgs* a;
  int m_tiles, n_tiles, num_kb;
  mutable uint32_t seq;                          // 0 = not resolved yet (sequence numbers start at 1)
  mutable size_t parity_off;

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
  // phase A: 32 rows x 32 columns of fp32 accumulators -> 16-bit pairs -> {data, sequence} words in the owners' areas
  __device__ __forceinline__ void epilogue(int t, int m0, int n0, int row, int col, uint32_t (&r)[32], uint8_t* stage) const {
    if (seq == 0u) {
      const unsigned long long epoch = *reinterpret_cast<volatile unsigned long long*>(a->state) / LL_UNIT;
      seq = uint32_t(epoch) + 1u;
      if (seq == 0u) seq = 1u;
      parity_off = size_t(epoch & 1u) * a->scatter_parity_stride;
    }
    const int gm = m0 + row, gn = n0 + col;
    const int M = a->M, N = a->N;
    if (gn >= N) return;                          // uniform across the warp (N % 32 == 0)
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
    // lane l sends 16-byte piece (l % 4) of rows (l / 4) + 8 i: four lanes cover 128 contiguous bytes of a row's words
    const int base_row = gm - lane, piece = lane & 3;
    const int src = a->rank * a->S + t / (m_tiles * n_tiles);        // (rank, K slice) -> source slot
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int rr = (lane >> 2) + 8 * i;
      const int grow = base_row + rr;
      if (grow < M) {
        const int owner = grow / a->owner_rows;
        const int lrow = grow - owner * a->owner_rows;
        const Vec8 pk = *reinterpret_cast<const Vec8*>(stage + rr * 80 + piece * 16);
        uint8_t* dst = a->scatter_peer[owner] + parity_off +
                       ((size_t(src) * a->owner_rows + lrow) * N + gn + piece * 8) * 4;
        st_volatile_u4(dst, pk.w[0], seq, pk.w[1], seq);
        st_volatile_u4(dst + 16, pk.w[2], seq, pk.w[3], seq);
      }
    }
    __syncwarp();                                 // the stage is free for the warp's next chunk
  }
};

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
      if (a.norm_mode != 0) {
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

template <int BN, int STAGES, class T, bool NVLS>
__global__ void __launch_bounds__(PG_THREADS)
gemm_ll_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ LLArgs args, int K, uint32_t idesc, uint32_t* status) {
  extern __shared__ uint8_t dyn_smem[];
  __shared__ float s_red[8 * 16];
  if (args.trace && threadIdx.x == 0) args.trace[size_t(blockIdx.x) * 8] = globaltimer_ns();
  LLProblem<BN, T> prob;
  prob.map_a = &map_a;
  prob.map_b = &map_b;
  prob.a = &args;
  prob.m_tiles = (args.M + PG_BM - 1) / PG_BM;
  prob.n_tiles = (args.N + BN - 1) / BN;
  prob.num_kb = args.num_kb;
  prob.seq = 0u;
  prob.parity_off = 0;
  if (args.phases & 1) gemm_persistent<BN, STAGES, 0, LLProblem<BN, T>>(dyn_smem, prob, 64, idesc, status);
  ll_phases<T, NVLS>(args, status, s_red);
}

static int ll_sm_count() { return device_sm_count(); }

template <int BN, int STAGES, class T, bool NVLS>
static int ll_launch(const CUtensorMap& ma, const CUtensorMap& mb, LLArgs& a, int K, int is_bf16, uint32_t* status,
                     cudaStream_t stream) {
  using L = PGemmSmem<BN, STAGES, true>;
  auto kern = gemm_ll_kernel<BN, STAGES, T, NVLS>;
  static bool configured[MAX_DEVICES] = {false};
  if (first_use_on_device(configured)) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYN_SMEM) != cudaSuccess) return -10;
  }
  // every CTA must be resident at once: phases B and C wait on work of the whole grid and of the peers
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, PG_THREADS, L::DYN_SMEM) != cudaSuccess || per_sm < 1)
    return -12;
  if (per_sm > 2) per_sm = 2;
  if (512u / L::TMEM_COLS < unsigned(per_sm)) per_sm = int(512u / L::TMEM_COLS);
  const int tiles = ((a.N + BN - 1) / BN) * ((a.M + PG_BM - 1) / PG_BM) * a.S;
  const int resident = ll_sm_count() * per_sm;
  const int grid = tiles < resident ? tiles : resident;
  // warps per row of phase C: a lane keeps at most 4 chunks of 8 values; more warps when rows alone leave the grid idle
  const int n8 = a.N >> 3;
  int wpr = 1;
  while (wpr < 8 && n8 > 128 * wpr) wpr <<= 1;
  if (n8 > 128 * wpr) return -5;
  while (wpr < 8 && wpr * 32 < n8 && long(a.M) * (wpr * 2) <= 8l * grid) wpr <<= 1;
  a.wpr = wpr;
  const uint32_t idesc = umma_idesc(PG_BM, BN, is_bf16 ? 1u : 0u, 1u);
  cudaError_t err = launch(kern, dim3(grid), dim3(PG_THREADS), size_t(L::DYN_SMEM), stream, ma, mb, a, K, idesc, status);
  return (err == cudaSuccess && cudaGetLastError() == cudaSuccess) ? 0 : -11;
}

}  // namespace ronn

using namespace ronn;

extern "C" int ronn_gemm_ll(const RonnGemmLLParams* p, uint32_t* status, cudaStream_t stream) {
  if (!p) return -1;
  const int M = p->M, N = p->N, K = p->K, world = p->world, rank = p->rank;
  if (M <= 0 || N <= 0 || K <= 0 || world < 2 || world > LL_MAX_RANKS || rank < 0 || rank >= world) return -1;
  if ((K & 7) || (p->lda & 7) || (p->ldw & 7) || (N & 31) || (p->ld_out & 7) || (p->residual && (p->ld_res & 7))) return -2;
  if (p->norm_mode != 0 && (p->norm_out == nullptr || p->norm_mode > 2)) return -5;
  if (p->out == nullptr || p->state == nullptr) return -6;
  const int owner_rows = (M + world - 1) / world;
  for (int r = 0; r < world; ++r)
    if (!p->scatter_area[r] || !p->result_area[r]) return -6;
  if (p->nvls && !p->result_mc) return -7;
  const int num_kb = (K + 63) / 64;
  int S = p->splitk < 1 ? 1 : p->splitk;
  if (S > num_kb) S = num_kb;
  while (S > 1 && S * world > LL_MAX_RANKS) --S;
  const int kb_per = (num_kb + S - 1) / S;
  S = (num_kb + kb_per - 1) / kb_per;              // every slice non-empty
  if (p->scatter_parity_stride < long(world) * S * owner_rows * N * 4 || p->result_parity_stride < long(M) * N * 4) return -8;

  LLArgs a;
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
  a.S = S;
  a.kb_per = kb_per;
  a.num_kb = num_kb;

  int bn = p->bn;
  const int m_tiles = (M + PG_BM - 1) / PG_BM;
  if (bn == 0) {
    bn = 128;
    while (bn > 32 && m_tiles * ((N + bn - 1) / bn) * S < 96) bn >>= 1;
  }
  CUtensorMap ma, mb;
  int rc = make_tmap_2d(&ma, p->A, uint64_t(M), uint64_t(K), uint64_t(p->lda), PG_BM, 64, 2);
  if (rc) return rc - 20;
  rc = make_tmap_2d(&mb, p->W, uint64_t(N), uint64_t(K), uint64_t(p->ldw), uint32_t(bn), 64, 2);
  if (rc) return rc - 30;
  const int bf = p->dtype == 0;
#define RONN_DISPATCH(BN_, ST_)                                                                              \
  do {                                                                                                       \
    if (a.nvls)                                                                                              \
      return bf ? ll_launch<BN_, ST_, __nv_bfloat16, true>(ma, mb, a, K, 1, status, stream)                  \
                : ll_launch<BN_, ST_, __half, true>(ma, mb, a, K, 0, status, stream);                        \
    return bf ? ll_launch<BN_, ST_, __nv_bfloat16, false>(ma, mb, a, K, 1, status, stream)                   \
              : ll_launch<BN_, ST_, __half, false>(ma, mb, a, K, 0, status, stream);                         \
  } while (0)
  switch (bn) {
    case 128: RONN_DISPATCH(128, 3);
    case 64: RONN_DISPATCH(64, 4);
    case 32: RONN_DISPATCH(32, 5);
    default: return -3;
  }
#undef RONN_DISPATCH
}
