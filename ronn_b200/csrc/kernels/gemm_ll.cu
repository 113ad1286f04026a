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
#include "gemm_ll_phases.cuh"
#include "tma_desc.cuh"

namespace ronn {

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
    if (seq == 0u) ll_resolve(*a, seq, parity_off);
    float f[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(r[i]);
    const int src = a->rank * a->S + t / (m_tiles * n_tiles);        // (rank, K slice) -> source slot
    ll_scatter_chunk<T>(*a, seq, parity_off, src, m0 + row, n0 + col, f, stage);
  }
};

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
  a.wpr = ll_pick_wpr(a.M, a.N, grid);
  if (a.wpr == 0) return -5;
  const uint32_t idesc = umma_idesc(PG_BM, BN, is_bf16 ? 1u : 0u, 1u);
  cudaError_t err = launch(kern, dim3(grid), dim3(PG_THREADS), size_t(L::DYN_SMEM), stream, ma, mb, a, K, idesc, status);
  return (err == cudaSuccess && cudaGetLastError() == cudaSuccess) ? 0 : -11;
}

}  // namespace ronn

using namespace ronn;

extern "C" int ronn_gemm_ll(const RonnGemmLLParams* p, uint32_t* status, cudaStream_t stream) {
  if (!p) return -1;
  const int M = p->M, N = p->N, K = p->K, world = p->world;
  if (K <= 0 || (K & 7) || (p->lda & 7) || (p->ldw & 7)) return K <= 0 ? -1 : -2;
  LLArgs a;
  if (const int rc = ll_fill_args(p, a)) return rc;
  const int owner_rows = a.owner_rows;
  const int num_kb = (K + 63) / 64;
  int S = p->splitk < 1 ? 1 : p->splitk;
  if (S > num_kb) S = num_kb;
  while (S > 1 && S * world > LL_MAX_RANKS) --S;
  const int kb_per = (num_kb + S - 1) / S;
  S = (num_kb + kb_per - 1) / kb_per;              // every slice non-empty
  if (p->scatter_parity_stride < long(world) * S * owner_rows * N * 4 || p->result_parity_stride < long(M) * N * 4) return -8;
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
