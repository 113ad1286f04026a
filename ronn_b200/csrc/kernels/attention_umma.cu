// Tensor-core attention over contiguous (non-paged) Q/K/V for whole-prompt prefill and encoder models:
// S = Q K^T and O += P V run on tcgen05 with the accumulators in TMEM, the softmax runs in registers.
//
// Kernel work-list item "prefill attention"; the reference computes attention through generic library matmul +
// softmax calls (crates/ronn-core/src/ops/neural_network.rs, attention section) and has no fused kernel.
//
// One CTA handles one (128-query tile, head, sequence):
//   warp 0      TMA producer: Q tile once, then K tiles [128 keys x D] (two buffers) and V^T tiles [D x 128 keys]
//               (two buffers for D = 128, one for D = 64), each buffer with its own full / empty barriers
//   warp 1      allocates TMEM and issues the MMAs: S = Q K^T (M 128, N 128, K = D) and PV = P V (M 128, N = D, K 128)
//   warps 2-9   masked online softmax over the S tile read from TMEM, P written to shared memory as the bf16/fp16 A
//               operand of the second MMA, O accumulated in registers from the PV tile.  Two threads share a query
//               row: warps 2-5 take keys 0-63 of the tile and the first half of the head dimension of O, warps 6-9
//               keys 64-127 and the second half; the two halves exchange their row maxima (and, at the end, their
//               row sums) through shared memory and an mbarrier.  With one thread per row the kernel was bound by
//               the issue rate of its four softmax warps.
// Both MMAs take K-major operands, so V is needed as V^T [D, keys]: ronn_transpose_v writes it (zero padded to whole
// key tiles, every sequence starting at a multiple of 128 columns, which also keeps every TMA x coordinate aligned).
// Two CTAs fit an SM for D = 64 (99 KB shared memory, 256 TMEM columns each), so the softmax of one overlaps the
// MMAs of the other.
#include "common.cuh"
#include "ptx_sm100.cuh"
#include "tma_desc.cuh"

namespace ronn {

constexpr int FA_THREADS = 320;
constexpr int FA_SOFTMAX_THREADS = 256;
constexpr int FA_BM = 128;     // queries per CTA
constexpr int FA_BN = 128;     // keys per tile

template <int D>
struct FaSmem {
  static constexpr int ATOMS = D / 64;                      // 128-byte-wide swizzle atoms along the head dimension
  static constexpr int Q_BYTES = FA_BM * D * 2;
  static constexpr int K_BYTES = FA_BN * D * 2;
  static constexpr int V_BYTES = D * FA_BN * 2;             // two atoms of [D rows x 128 B]
  static constexpr int P_BYTES = FA_BM * FA_BN * 2;         // two atoms of [128 rows x 128 B]
  // K tiles are double-buffered: K(j+1) is requested when S(j-1) has been computed, a whole key tile ahead of its
  // use (with one buffer the TMA round trip of K(j+1) sat between S(j) and S(j+1) and bounded the loop whatever the
  // softmax cost).  V^T is double-buffered where shared memory allows it (D = 128, one CTA per SM); for D = 64 two
  // CTAs share an SM and V(j+1) has the S MMA and the softmax of tile j+1 to land.
  static constexpr int K_STAGES = 2;
  static constexpr int V_STAGES = D == 64 ? 1 : 2;
  static constexpr int TILE_BYTES = Q_BYTES + K_STAGES * K_BYTES + V_STAGES * V_BYTES + P_BYTES;
  static constexpr int XCHG_BYTES = 2 * 2 * FA_BM * 4;      // [parity][column half][row] floats
  static constexpr int DYN_SMEM = TILE_BYTES + 16 * 8 + XCHG_BYTES + 1024;
  static constexpr uint32_t TMEM_COLS = 256;                // S: 128 columns, PV: D (<= 128) columns
};

struct FaArgs {
  const int* seq_start;    // first token row of each sequence in the qkv buffer
  const int* q_len;        // query rows of each sequence
  const int* kv_len;       // keys each sequence attends to (rows seq_start .. seq_start + kv_len)
  const int* vt_start;     // first column of each sequence in the V^T buffer (multiple of 128)
  void* out;
  long ld_o;
  int q_off, k_off;        // column of head 0 of Q / K in the qkv buffer
  int heads, kv_heads;
  int causal;
  float scale_log2;        // softmax scale * log2(e)
};

// 2^x on the special-function unit in one instruction (no range fix-up; inputs here are <= 0 or the result is masked)
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}


template <class T, int D>
__global__ void __launch_bounds__(FA_THREADS, D == 64 ? 2 : 1)
flash_attention_kernel(const __grid_constant__ CUtensorMap map_qk, const __grid_constant__ CUtensorMap map_vt, FaArgs a,
                       uint32_t idesc_s, uint32_t idesc_pv, uint32_t* status) {
  using L = FaSmem<D>;
  extern __shared__ uint8_t dyn_smem[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dyn_smem) + 1023) & ~uintptr_t(1023));
  uint8_t* sq = base;
  uint8_t* sk = sq + L::Q_BYTES;
  uint8_t* sv = sk + L::K_STAGES * L::K_BYTES;
  uint8_t* sp = sv + L::V_STAGES * L::V_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(base + L::TILE_BYTES);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;                               // [2]
  uint64_t* k_empty = bars + 3;                              // [2]
  uint64_t* v_full = bars + 5;                               // [2]
  uint64_t* v_empty = bars + 7;                              // [2]
  uint64_t* s_full = bars + 9;
  uint64_t* p_full = bars + 10;
  uint64_t* pv_full = bars + 11;
  uint64_t* x_full = bars + 12;                              // row-statistics exchange between the two column halves
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
  float* xbuf = reinterpret_cast<float*>(base + L::TILE_BYTES + 16 * 8);
  volatile uint32_t* abort = tmem_slot + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const int seq = blockIdx.z, head = blockIdx.y, qt = blockIdx.x;
  const int q_len = a.q_len[seq], kv_len = a.kv_len[seq];
  if (qt * FA_BM >= q_len || kv_len <= 0) return;            // uniform for the CTA, before any barrier or TMEM use
  const int row0 = a.seq_start[seq];
  const int kvh = head / (a.heads / a.kv_heads);
  const int shift = kv_len - q_len;                          // causal: query i sees keys j <= i + shift
  int n_kv = (kv_len + FA_BN - 1) / FA_BN;
  if (a.causal) {
    const int last_key = min(kv_len - 1, qt * FA_BM + FA_BM - 1 + shift);
    n_kv = last_key < 0 ? 0 : min(n_kv, last_key / FA_BN + 1);
  }

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(p_full, FA_SOFTMAX_THREADS);
    mbar_init(pv_full, 1);
    mbar_init(x_full, FA_SOFTMAX_THREADS);
    *abort = 0;
    mbar_fence_init();
    fence_proxy_async_smem();
  }
  __syncwarp();
  if (warp == 1) {
    tmem_alloc(tmem_slot, L::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base, tmem_pv = tmem_base + 128;

  if (warp == 0) {
    if (lane == 0) {
      pdl_wait();
      pdl_trigger();
      mbar_expect_tx(q_full, L::Q_BYTES);
#pragma unroll
      for (int at = 0; at < L::ATOMS; ++at)
        tma_load_2d(sq + at * (FA_BM * 128), &map_qk, q_full, a.q_off + head * D + at * 64, row0 + qt * FA_BM);
      const int vt0 = a.vt_start[seq];
      for (int j = 0; j < n_kv; ++j) {
        const int ks = j % L::K_STAGES, vs = j % L::V_STAGES;
        if (!mbar_wait(&k_empty[ks], ((j / L::K_STAGES) & 1) ^ 1, abort, status, STATUS_WAIT_SLOT)) break;
        mbar_expect_tx(&k_full[ks], L::K_BYTES);
        uint8_t* kdst = sk + ks * L::K_BYTES;
#pragma unroll
        for (int at = 0; at < L::ATOMS; ++at)
          tma_load_2d(kdst + at * (FA_BN * 128), &map_qk, &k_full[ks], a.k_off + kvh * D + at * 64, row0 + j * FA_BN);
        if (!mbar_wait(&v_empty[vs], ((j / L::V_STAGES) & 1) ^ 1, abort, status, STATUS_WAIT_SLOT)) break;
        mbar_expect_tx(&v_full[vs], L::V_BYTES);
        uint8_t* vdst = sv + vs * L::V_BYTES;
#pragma unroll
        for (int at = 0; at < 2; ++at)
          tma_load_2d(vdst + at * (D * 128), &map_vt, &v_full[vs], vt0 + j * FA_BN + at * 64, kvh * D);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = mbar_wait(q_full, 0, abort, status, STATUS_WAIT_TMA);
      const uint32_t aq = smem_u32(sq);
      // S(j) = Q K(j)^T into the single S accumulator; frees K's buffer for K(j+2)
      auto issue_s = [&](int j) -> bool {
        const int ks = j % L::K_STAGES;
        if (!mbar_wait(&k_full[ks], (j / L::K_STAGES) & 1, abort, status, STATUS_WAIT_TMA)) return false;
        tc_fence_after_sync();
        const uint32_t ak = smem_u32(sk + ks * L::K_BYTES);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = uint32_t(k / 4) * (FA_BM * 128) + uint32_t(k % 4) * 32;
          umma_f16(tmem_s, umma_desc_k128(aq + off), umma_desc_k128(ak + off), idesc_s, k != 0);
        }
        umma_commit(s_full);
        umma_commit(&k_empty[ks]);
        return true;
      };
      if (ok && n_kv > 0) ok = issue_s(0);
      for (int j = 0; j < n_kv && ok; ++j) {
        const int vs = j % L::V_STAGES;
        // P(j) is in shared memory and the softmax warps have finished reading S(j) and PV(j-1)
        if (!mbar_wait(p_full, j & 1, abort, status, STATUS_WAIT_EPI)) break;
        // S(j+1) goes first: the softmax of tile j+1 is the critical path (issuing an MMA costs 70-100 cycles, and
        // behind the eight instructions of PV(j) the next S was ready about 1000 cycles later); PV(j) then runs
        // during pass 1 of tile j+1, whose O update waits for it.  P has one buffer: it is rewritten in pass 2 of
        // tile j+1, after that wait.
        if (j + 1 < n_kv && !issue_s(j + 1)) break;
        if (!mbar_wait(&v_full[vs], (j / L::V_STAGES) & 1, abort, status, STATUS_WAIT_TMA)) break;
        tc_fence_after_sync();
        const uint32_t ap = smem_u32(sp);
        const uint32_t av = smem_u32(sv + vs * L::V_BYTES);
#pragma unroll
        for (int k = 0; k < FA_BN / 16; ++k) {
          const uint32_t offp = uint32_t(k / 4) * (FA_BM * 128) + uint32_t(k % 4) * 32;
          const uint32_t offv = uint32_t(k / 4) * (D * 128) + uint32_t(k % 4) * 32;
          umma_f16(tmem_pv, umma_desc_k128(ap + offp), umma_desc_k128(av + offv), idesc_pv, k != 0);
        }
        umma_commit(pv_full);
        umma_commit(&v_empty[vs]);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ softmax + output: two threads per query row
    pdl_wait();                                              // `out` may still be read by the previous kernel
    const int q = warp & 3;                                  // TMEM lane quarter of this warp
    const int half = (warp - 2) >> 2;                        // 0: keys 0-63 and O columns [0, D/2); 1: the rest
    const int r = q * 32 + lane;                             // row inside the tile
    const int qi = qt * FA_BM + r;                           // query index inside the sequence
    const uint32_t lane_addr = uint32_t(q * 32) << 16;
    const int limit = a.causal ? min(kv_len, qi + shift + 1) : kv_len;     // keys [0, limit) are visible
    const uint32_t sw = uint32_t(r & 7);
    constexpr int DH = D / 2;
    const int cbeg = half * (FA_BN / 2);
    float o[DH];
#pragma unroll
    for (int i = 0; i < DH; ++i) o[i] = 0.f;
    float m = -1e30f, l = 0.f;
    bool ok = true;
    uint32_t xphase = 0;
    // exchange a per-row value with the thread that owns the other column half of the row
    auto exchange = [&](float mine, float& other) -> bool {
      float* slot = xbuf + (xphase & 1u) * (2 * FA_BM);
      slot[half * FA_BM + r] = mine;
      mbar_arrive(x_full);
      bool good = mbar_wait(x_full, xphase & 1u, abort, status, STATUS_WAIT_EPI);
      good = __all_sync(0xffffffffu, good);
      if (good) other = slot[(half ^ 1) * FA_BM + r];
      ++xphase;
      return good;
    };
    for (int j = 0; j < n_kv; ++j) {
      ok = mbar_wait(s_full, j & 1, abort, status, STATUS_WAIT_ACCUM);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const int key0 = j * FA_BN;
      // Tiles whose 64 keys are visible to every row of the warp (all but the diagonal and the last tile) take a path
      // without per-key masks: the softmax warps are bound by instruction issue, and the mask costs about as much as
      // the arithmetic.
      const bool full = __all_sync(0xffffffffu, key0 + cbeg + FA_BN / 2 <= limit);
      // pass 1: row maximum of the visible keys of this half, then of the whole row.  S is read in 16-column pieces,
      // the next piece in flight while the current one is reduced (a TMEM load costs several hundred cycles).
      const uint32_t s_addr = tmem_s + lane_addr + uint32_t(cbeg);
      uint32_t va[16], vb[16];
      float mx = m;
      auto max16 = [&](const uint32_t (&v)[16], int c) {
        if (full) {
          float raw = __uint_as_float(v[0]);
#pragma unroll
          for (int i = 1; i < 16; ++i) raw = fmaxf(raw, __uint_as_float(v[i]));
          mx = fmaxf(mx, raw * a.scale_log2);                  // the scale is positive
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (key0 + cbeg + c + i < limit) mx = fmaxf(mx, __uint_as_float(v[i]) * a.scale_log2);
        }
      };
      tmem_ld_32x16(s_addr, va);
      tmem_ld_wait();
      tmem_ld_32x16(s_addr + 16, vb);
      max16(va, 0);
      tmem_ld_wait();
      tmem_ld_32x16(s_addr + 32, va);
      max16(vb, 16);
      tmem_ld_wait();
      tmem_ld_32x16(s_addr + 48, vb);
      max16(va, 32);
      tmem_ld_wait();
      max16(vb, 48);
      // the PV tile of the previous key tile joins O before O is rescaled to the new maximum; its load is in flight
      // while the two halves of the row exchange their maxima
      const uint32_t o_addr = tmem_pv + lane_addr + uint32_t(half * DH);
      if (j > 0) {
        ok = mbar_wait(pv_full, (j - 1) & 1, abort, status, STATUS_WAIT_ACCUM);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
        tmem_ld_32x16(o_addr, va);
      }
      float mx_other = mx;
      ok = exchange(mx, mx_other);
      if (!ok) break;
      mx = fmaxf(mx, mx_other);
      const float alpha = fast_exp2(m - mx);
      if (j > 0) {
        // O += PV in 16-column pieces, again with the next piece in flight
#pragma unroll
        for (int c = 0; c < DH; c += 32) {
          tmem_ld_wait();
          tmem_ld_32x16(o_addr + uint32_t(c + 16), vb);
#pragma unroll
          for (int i = 0; i < 16; ++i) o[c + i] += __uint_as_float(va[i]);
          tmem_ld_wait();
          if (c + 32 < DH) tmem_ld_32x16(o_addr + uint32_t(c + 32), va);
#pragma unroll
          for (int i = 0; i < 16; ++i) o[c + 16 + i] += __uint_as_float(vb[i]);
        }
      }
      tmem_ld_32x16(s_addr, va);                             // first piece of pass 2, in flight during the rescale
#pragma unroll
      for (int i = 0; i < DH; ++i) o[i] *= alpha;
      l *= alpha;
      m = mx;
      // pass 2: probabilities -> shared memory (A operand of the second MMA: K-major, 128-byte swizzle); the 64 keys
      // of this half are exactly one swizzle atom
      uint8_t* atom = sp + half * (FA_BM * 128) + r * 128;
      auto prob16 = [&](const uint32_t (&v)[16], int c) {
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          float p[8];
          if (full) {
#pragma unroll
            for (int i = 0; i < 8; ++i) p[i] = fast_exp2(fmaf(__uint_as_float(v[g * 8 + i]), a.scale_log2, -m));
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int key = key0 + cbeg + c + g * 8 + i;
              const float e = fast_exp2(fmaf(__uint_as_float(v[g * 8 + i]), a.scale_log2, -m));
              p[i] = key < limit ? e : 0.f;
            }
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) l += p[i];
          const uint32_t chunk = uint32_t(c / 8 + g);
          *reinterpret_cast<Vec8*>(atom + ((chunk ^ sw) << 4)) = pack8<T>(p);
        }
      };
      tmem_ld_wait();
      tmem_ld_32x16(s_addr + 16, vb);
      prob16(va, 0);
      tmem_ld_wait();
      tmem_ld_32x16(s_addr + 32, va);
      prob16(vb, 16);
      tmem_ld_wait();
      tmem_ld_32x16(s_addr + 48, vb);
      prob16(va, 32);
      tmem_ld_wait();
      prob16(vb, 48);
      tc_fence_before_sync();                                // TMEM reads of S and PV are done
      fence_proxy_async_smem();                              // P is visible to the tensor core
      mbar_arrive(p_full);
    }
    if (ok && n_kv > 0) {
      ok = mbar_wait(pv_full, (n_kv - 1) & 1, abort, status, STATUS_WAIT_ACCUM);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        tc_fence_after_sync();
#pragma unroll
        for (int c = 0; c < DH; c += 32) {
          uint32_t v[32];
          tmem_ld_32x32(tmem_pv + lane_addr + uint32_t(half * DH + c), v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[c + i] += __uint_as_float(v[i]);
        }
      }
    }
    if (ok) {
      float l_other = 0.f;
      ok = exchange(l, l_other);                             // the row sum is the sum of both halves
      l += l_other;
    }
    if (ok && qi < q_len) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      T* orow = reinterpret_cast<T*>(a.out) + long(row0 + qi) * a.ld_o + head * D + half * DH;
#pragma unroll
      for (int c = 0; c < DH; c += 8) {
        float f[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = o[c + i] * inv;
        *reinterpret_cast<Vec8*>(orow + c) = pack8<T>(f);
      }
    }
  }
  pdl_trigger();
  if (*abort) {
    const long long t0 = clock64();
    while (clock64() - t0 < 400000ll) { __nanosleep(1000); }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, L::TMEM_COLS);
  }
}

// V columns of the fused qkv buffer -> V^T [kv_heads * D, ld_vt], sequence s occupying columns
// [vt_start[s], vt_start[s] + round_up(kv_len[s], 128)), zero beyond kv_len.  grid = (key tiles, kv_heads, sequences).
template <class T, int D>
__global__ void __launch_bounds__(256)
transpose_v_kernel(const T* __restrict__ qkv, long ld, int v_off, const int* __restrict__ seq_start,
                   const int* __restrict__ kv_len, const int* __restrict__ vt_start, T* __restrict__ vt, long ld_vt) {
  // rows of D + 2 elements (an odd number of 32-bit words): a column read by consecutive key groups lands in
  // different banks, and the 4-byte stores of the first phase stay aligned
  __shared__ __align__(16) T tile[128][D + 2];
  pdl_wait();
  pdl_trigger();
  const int seq = blockIdx.z, kvh = blockIdx.y, kt = blockIdx.x;
  const int len = kv_len[seq];
  if (kt * 128 >= len) return;
  const int row0 = seq_start[seq] + kt * 128;
  constexpr int CPR = D / 8;                                  // 16-byte chunks per token row
  for (int i = threadIdx.x; i < 128 * CPR; i += blockDim.x) {
    const int t = i / CPR, c = i % CPR;
    Vec8 v = {};
    if (kt * 128 + t < len) v = *reinterpret_cast<const Vec8*>(qkv + long(row0 + t) * ld + v_off + kvh * D + c * 8);
    uint32_t* dst = reinterpret_cast<uint32_t*>(&tile[t][c * 8]);
    const uint32_t* src = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
    for (int k = 0; k < 4; ++k) dst[k] = src[k];
  }
  __syncthreads();
  const long col0 = long(vt_start[seq]) + kt * 128;
  // 8 consecutive lanes write 8 consecutive 16-byte chunks (8 keys each) of one V^T row: 128 contiguous bytes
  for (int i = threadIdx.x; i < D * 16; i += blockDim.x) {
    const int c = (i & 7) + 8 * (i / (8 * D)), d = (i >> 3) % D;
    alignas(16) T tmp[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) tmp[k] = tile[c * 8 + k][d];
    *reinterpret_cast<Vec8*>(vt + long(kvh * D + d) * ld_vt + col0 + c * 8) = *reinterpret_cast<const Vec8*>(tmp);
  }
}

template <class T, int D>
static int launch_fa(const CUtensorMap& mqk, const CUtensorMap& mvt, const FaArgs& a, int n_seq, int max_q_len,
                     int is_bf16, uint32_t* status, cudaStream_t stream) {
  using L = FaSmem<D>;
  auto kern = flash_attention_kernel<T, D>;
  static bool configured[MAX_DEVICES] = {false};
  if (first_use_on_device(configured)) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYN_SMEM) != cudaSuccess) return -10;
  }
  dim3 grid((max_q_len + FA_BM - 1) / FA_BM, a.heads, n_seq);
  const uint32_t fmt = is_bf16 ? 1u : 0u;
  cudaError_t err = launch(kern, grid, dim3(FA_THREADS), size_t(L::DYN_SMEM), stream, mqk, mvt, a,
                           umma_idesc(FA_BM, FA_BN, fmt, 1u), umma_idesc(FA_BM, D, fmt, 1u), status);
  return (err == cudaSuccess && cudaGetLastError() == cudaSuccess) ? 0 : -11;
}

}  // namespace ronn

using namespace ronn;



// qkv: [tokens, ld] with V of kv head h at columns v_off + h * head_dim.  vt: [kv_heads * head_dim, ld_vt].
// seq_start / kv_len / vt_start: device int32 [n_seq]; vt_start values are multiples of 128 and
// vt_start[s] + round_up(kv_len[s], 128) <= ld_vt.  max_kv_len bounds kv_len (grid size).  dtype 0 bf16, 1 fp16.
extern "C" int ronn_transpose_v(const void* qkv, long ld, int v_off, const int* seq_start, const int* kv_len,
                                const int* vt_start, void* vt, long ld_vt, int n_seq, int kv_heads, int head_dim,
                                int max_kv_len, int dtype, cudaStream_t stream) {
  if (n_seq <= 0 || max_kv_len <= 0) return 0;
  if ((ld & 7) || (ld_vt & 7) || (v_off & 7) || (head_dim != 64 && head_dim != 128)) return -2;
  dim3 grid((max_kv_len + 127) / 128, kv_heads, n_seq);
#define RONN_TV(T_, D_) launch(transpose_v_kernel<T_, D_>, grid, dim3(256), 0, stream, (const T_*)qkv, ld, v_off, seq_start, kv_len, vt_start, (T_*)vt, ld_vt)
  if (dtype == 0) { if (head_dim == 64) RONN_TV(__nv_bfloat16, 64); else RONN_TV(__nv_bfloat16, 128); }
  else { if (head_dim == 64) RONN_TV(__half, 64); else RONN_TV(__half, 128); }
#undef RONN_TV
  return cudaGetLastError() == cudaSuccess ? 0 : -100;
}

// Attention of n_seq sequences whose Q and K sit in the fused qkv buffer ([tokens, ld], head h of Q at column
// q_off + h * head_dim, kv head g of K at k_off + g * head_dim) and whose V^T was written by ronn_transpose_v.
// Query i of a sequence (row seq_start + i, i < q_len) attends to keys [0, kv_len), or with `causal` to keys
// j <= i + (kv_len - q_len).  out: [tokens, ld_o], head h at column h * head_dim.  total_rows: rows of the qkv
// buffer (TMA bound; rows past it read as zero).  head_dim 64 or 128; ld, ld_vt, offsets multiples of 8.
extern "C" int ronn_flash_attention(const void* qkv, long ld, long total_rows, int q_off, int k_off, const void* vt,
                                    long ld_vt, const int* seq_start, const int* q_len, const int* kv_len,
                                    const int* vt_start, void* out, long ld_o, int n_seq, int max_q_len, int heads,
                                    int kv_heads, int head_dim, int causal, float scale, int dtype, uint32_t* status,
                                    cudaStream_t stream) {
  if (n_seq <= 0 || max_q_len <= 0) return 0;
  if ((ld & 7) || (ld_vt & 7) || (ld_o & 7) || (q_off & 7) || (k_off & 7) || kv_heads <= 0 || heads % kv_heads) return -2;
  if (head_dim != 64 && head_dim != 128) return -3;
  CUtensorMap mqk, mvt;
  int rc = make_tmap_2d(&mqk, qkv, uint64_t(total_rows), uint64_t(ld), uint64_t(ld), 128, 64, 2);
  if (rc) return rc - 20;
  rc = make_tmap_2d(&mvt, vt, uint64_t(kv_heads) * head_dim, uint64_t(ld_vt), uint64_t(ld_vt), uint32_t(head_dim), 64, 2);
  if (rc) return rc - 30;
  FaArgs a{seq_start, q_len, kv_len, vt_start, out, ld_o, q_off, k_off, heads, kv_heads, causal,
           scale * 1.4426950408889634f};
  if (dtype == 0) {
    return head_dim == 64 ? launch_fa<__nv_bfloat16, 64>(mqk, mvt, a, n_seq, max_q_len, 1, status, stream)
                          : launch_fa<__nv_bfloat16, 128>(mqk, mvt, a, n_seq, max_q_len, 1, status, stream);
  }
  return head_dim == 64 ? launch_fa<__half, 64>(mqk, mvt, a, n_seq, max_q_len, 0, status, stream)
                        : launch_fa<__half, 128>(mqk, mvt, a, n_seq, max_q_len, 0, status, stream);
}
