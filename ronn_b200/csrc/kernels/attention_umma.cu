// Tensor-core attention for whole prompts, encoders and chunked prefill: S = Q K^T and PV = P V on tcgen05 with two alternating TMEM buffers, V read in
// its stored [keys, head_dim] layout (no transposed copy), K / V taken either from the fused qkv buffer (whole prompts,
// encoders) or from the paged KV cache through the block table (chunked prefill, prefix hits).
//
// Kernel work-list item "prefill attention"; the reference computes attention through generic library matmul +
// softmax calls (crates/ronn-core/src/ops/neural_network.rs, attention section) and has no fused kernel.
//
// One CTA handles one (128-query tile, head, sequence):
//   warp 0      TMA producer: Q tile once, then per key tile K [128 keys x D] (two buffers) and V [128 keys x D]
//               (two buffers for D = 128, one for D = 64).  Paged form: eight 16-key loads per tile and operand, one per
//               cache block, stacked into the same swizzled layout.
//   warp 1      allocates 256 TMEM columns = two buffers of 128 and issues the MMAs.  Buffer j & 1 first receives
//               S(j) = Q K(j)^T (M 128, N 128, K = D) and, once the softmax warps have turned it into P(j), the product
//               PV(j) = P(j) V(j) (M 128, N = D, K 128) in its first D columns.  S(j+1) sits in the other buffer while
//               tile j is in the softmax, so the softmax of consecutive tiles runs back to back; S(j+2) is issued as
//               soon as PV(j) has been read out.
//   warps 2-9   masked online softmax, two threads per query row (keys 0-63 / 64-127 of the tile, and the two halves
//               of the head dimension of O); the halves exchange row maxima through shared memory and a named barrier
//               of their two warps.  P goes to shared memory as the K-major A operand of the second MMA, O is
//               accumulated in registers from the PV tiles.
// The B operand of the second MMA is V as stored: keys are its K dimension and the head dimension is contiguous, so its
// shared-memory descriptor is MN-major (instruction-descriptor bit 16) over the same 128-byte-swizzled rows TMA writes.
// Rows of the qkv buffer past a sequence's keys (the next sequence, zero fill past the buffer) and cache slots past
// the context are multiplied by P = 0; they are finite because every row of the buffer is a GEMM output and the cache
// starts zeroed.
#include "common.cuh"
#include "ptx_sm100.cuh"
#include "tma_desc.cuh"

namespace ronn {

constexpr int FM_THREADS = 320;
constexpr int FM_SOFTMAX_WARPS = 8;
constexpr int FM_BM = 128;     // queries per CTA
constexpr int FM_BN = 128;     // keys per tile
constexpr int FM_BLOCK = 16;   // tokens per KV-cache block

template <int D>
struct FmSmem {
  static constexpr int ATOMS = D / 64;                      // 128-byte-wide swizzle atoms along the head dimension
  static constexpr int Q_BYTES = FM_BM * D * 2;
  static constexpr int K_BYTES = FM_BN * D * 2;
  static constexpr int V_BYTES = FM_BN * D * 2;
  static constexpr int P_BYTES = FM_BM * FM_BN * 2;         // two atoms of [128 rows x 128 B]
  static constexpr int K_STAGES = 2;
  static constexpr int V_STAGES = D == 64 ? 1 : 2;          // D = 64: two CTAs per SM
  static constexpr int TILE_BYTES = Q_BYTES + K_STAGES * K_BYTES + V_STAGES * V_BYTES + P_BYTES;
  static constexpr int XCHG_BYTES = 2 * 2 * FM_BM * 4;      // [parity][column half][row] floats
  static constexpr int DYN_SMEM = TILE_BYTES + 24 * 8 + XCHG_BYTES + 1024;
  static constexpr uint32_t TMEM_COLS = 256;
};

struct FmArgs {
  const int* seq_start;     // first token row of each sequence in the q buffer
  const int* q_len;         // query rows of each sequence
  const int* kv_len;        // keys each sequence attends to
  const int* block_tables;  // paged form: [*, max_blocks] cache block of every 16 keys
  const int* bt_row;        // paged form: row of block_tables per sequence (null: the sequence index)
  void* out;
  long ld_o;
  int max_blocks;
  int q_off, k_off, v_off;  // column of head 0 of Q (and, contiguous form, of K and V) in the buffer
  int heads, kv_heads;
  int causal;
  float scale_log2;         // softmax scale * log2(e)
};

__device__ __forceinline__ float fm_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Packed pairs of fp32 values in one 64-bit register: sm_100 adds, multiplies and fuses two lanes per instruction,
// which halves the issue slots of the softmax arithmetic (the softmax warps are bound by instruction issue).
__device__ __forceinline__ uint64_t pk2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ uint64_t pk2u(uint32_t lo, uint32_t hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ void upk2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// barrier of the two warps that share a set of query rows (ids 1-4; id 0 is __syncthreads)
__device__ __forceinline__ void pair_barrier(int id) {
  // literal ids: with the id in a register the compiler reserves all 16 barriers of the SM for one CTA
  switch (id) {
    case 1: asm volatile("bar.sync 1, 64;" ::: "memory"); break;
    case 2: asm volatile("bar.sync 2, 64;" ::: "memory"); break;
    case 3: asm volatile("bar.sync 3, 64;" ::: "memory"); break;
    default: asm volatile("bar.sync 4, 64;" ::: "memory"); break;
  }
}

// Shared-memory descriptor of an MN-major operand stored as rows of 128 bytes (64 values of the contiguous M/N
// dimension) per K index with the 128-byte swizzle: groups of 8 K indices are `sbo` bytes apart, blocks of 64 values
// along M/N `lbo` bytes apart.
__device__ __forceinline__ uint64_t umma_desc_mn128(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= uint64_t((smem_addr & 0x3FFFF) >> 4);
  d |= uint64_t(lbo >> 4) << 16;
  d |= uint64_t(sbo >> 4) << 32;
  d |= uint64_t(1) << 46;
  d |= uint64_t(2) << 61;
  return d;
}

template <class T, int D, bool PAGED>
__global__ void __launch_bounds__(FM_THREADS, D == 64 ? 2 : 1)
fmha_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
            const __grid_constant__ CUtensorMap map_v, FmArgs a, uint32_t idesc_s, uint32_t idesc_pv, uint32_t v_lbo,
            uint32_t v_sbo, uint32_t* status) {
  using L = FmSmem<D>;
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
  uint64_t* s_full = bars + 9;                               // [2] S(j) complete in buffer j & 1
  uint64_t* pv_full = bars + 11;                             // PV(j) complete
  uint64_t* p_full = bars + 12;                              // P(j) in shared memory, S(j) read out (one arrival per warp)
  uint64_t* buf_free = bars + 13;                            // [2] PV(j) read out of buffer j & 1 (one arrival per warp)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile uint32_t* abort = tmem_slot + 1;
  float* xbuf = reinterpret_cast<float*>(base + L::TILE_BYTES + 24 * 8);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // Query tiles are the slowest grid dimension, last tile first: the late tiles of a causal sequence have the most key
  // tiles, and with all of them at the head of the launch order the short CTAs fill the gaps at the end (in
  // sequence-major order a slot that drew three long CTAs set the kernel's duration).
  const int seq = blockIdx.y, head = blockIdx.x, qt = int(gridDim.z) - 1 - int(blockIdx.z);
  const int q_len = a.q_len[seq], kv_len = a.kv_len[seq];
  if (qt * FM_BM >= q_len || kv_len <= 0) return;            // uniform for the CTA, before any barrier or TMEM use
  const int row0 = a.seq_start[seq];
  const int kvh = head / (a.heads / a.kv_heads);
  const int shift = kv_len - q_len;                          // causal: query i sees keys j <= i + shift
  int n_kv = (kv_len + FM_BN - 1) / FM_BN;
  if (a.causal) {
    const int last_key = min(kv_len - 1, qt * FM_BM + FM_BM - 1 + shift);
    n_kv = last_key < 0 ? 0 : min(n_kv, last_key / FM_BN + 1);
  }

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&buf_free[i], FM_SOFTMAX_WARPS);
    }
    mbar_init(pv_full, 1);
    mbar_init(p_full, FM_SOFTMAX_WARPS);
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

  if (warp == 0) {
    if (lane == 0) {
      pdl_wait();
      pdl_trigger();
      mbar_expect_tx(q_full, L::Q_BYTES);
#pragma unroll
      for (int at = 0; at < L::ATOMS; ++at)
        tma_load_2d(sq + at * (FM_BM * 128), &map_q, q_full, a.q_off + head * D + at * 64, row0 + qt * FM_BM);
      const int* bt = PAGED ? a.block_tables + long(a.bt_row ? a.bt_row[seq] : seq) * a.max_blocks : nullptr;
      // one operand tile: a 128-row box of the qkv buffer, or eight 16-row boxes of the cache (blocks past the context
      // repeat the sequence's first block: their keys are masked, but the bytes have to arrive and be finite)
      auto load_tile = [&](uint8_t* dst, const CUtensorMap* map, uint64_t* bar, int col, int j) {
        if (!PAGED) {
#pragma unroll
          for (int at = 0; at < L::ATOMS; ++at)
            tma_load_2d(dst + at * (FM_BN * 128), map, bar, col + kvh * D + at * 64, row0 + j * FM_BN);
        } else {
#pragma unroll 1
          for (int i = 0; i < FM_BN / FM_BLOCK; ++i) {
            const int bi = j * (FM_BN / FM_BLOCK) + i;
            const int phys = bt[bi * FM_BLOCK < kv_len ? bi : 0];
            const int row = (phys * a.kv_heads + kvh) * FM_BLOCK;
#pragma unroll
            for (int at = 0; at < L::ATOMS; ++at)
              tma_load_2d(dst + at * (FM_BN * 128) + i * (FM_BLOCK * 128), map, bar, at * 64, row);
          }
        }
      };
      // order K(0) K(1) V(0) K(2) V(1) ...: the wait for V's buffer (PV(j-1) done) never holds back the K tile that
      // the next S needs
      for (int j = 0; j <= n_kv; ++j) {
        if (j < n_kv) {
          const int ks = j % L::K_STAGES;
          if (!mbar_wait(&k_empty[ks], ((j / L::K_STAGES) & 1) ^ 1, abort, status, STATUS_WAIT_SLOT)) break;
          mbar_expect_tx(&k_full[ks], L::K_BYTES);
          load_tile(sk + ks * L::K_BYTES, &map_k, &k_full[ks], a.k_off, j);
        }
        if (j >= 1) {
          const int i = j - 1, vs = i % L::V_STAGES;
          if (!mbar_wait(&v_empty[vs], ((i / L::V_STAGES) & 1) ^ 1, abort, status, STATUS_WAIT_SLOT)) break;
          mbar_expect_tx(&v_full[vs], L::V_BYTES);
          load_tile(sv + vs * L::V_BYTES, &map_v, &v_full[vs], a.v_off, i);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = mbar_wait(q_full, 0, abort, status, STATUS_WAIT_TMA);
      const uint32_t aq = smem_u32(sq);
      auto issue_s = [&](int j) -> bool {
        const int ks = j % L::K_STAGES;
        if (!mbar_wait(&k_full[ks], (j / L::K_STAGES) & 1, abort, status, STATUS_WAIT_TMA)) return false;
        tc_fence_after_sync();
        const uint32_t ak = smem_u32(sk + ks * L::K_BYTES);
        const uint32_t tmem_s = tmem_base + uint32_t(j & 1) * 128u;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = uint32_t(k / 4) * (FM_BM * 128) + uint32_t(k % 4) * 32;
          umma_f16(tmem_s, umma_desc_k128(aq + off), umma_desc_k128(ak + off), idesc_s, k != 0);
        }
        umma_commit(&s_full[j & 1]);
        umma_commit(&k_empty[ks]);
        return true;
      };
      if (ok && n_kv > 0) ok = issue_s(0);
      if (ok && n_kv > 1) ok = issue_s(1);
      for (int j = 0; j < n_kv && ok; ++j) {
        const int vs = j % L::V_STAGES;
        // P(j) is in shared memory and S(j) has left buffer j & 1
        if (!mbar_wait(p_full, j & 1, abort, status, STATUS_WAIT_EPI)) break;
        if (!mbar_wait(&v_full[vs], (j / L::V_STAGES) & 1, abort, status, STATUS_WAIT_TMA)) break;
        tc_fence_after_sync();
        const uint32_t ap = smem_u32(sp);
        const uint32_t av = smem_u32(sv + vs * L::V_BYTES);
        const uint32_t tmem_pv = tmem_base + uint32_t(j & 1) * 128u;
#pragma unroll
        for (int k = 0; k < FM_BN / 16; ++k) {
          const uint32_t offp = uint32_t(k / 4) * (FM_BM * 128) + uint32_t(k % 4) * 32;
          umma_f16(tmem_pv, umma_desc_k128(ap + offp), umma_desc_mn128(av + uint32_t(k) * (16 * 128), v_lbo, v_sbo),
                   idesc_pv, k != 0);
        }
        umma_commit(pv_full);
        umma_commit(&v_empty[vs]);
        if (j + 2 < n_kv) {
          // the softmax warps read PV(j) while they work on tile j + 1; then the buffer takes S(j+2)
          if (!mbar_wait(&buf_free[j & 1], (j >> 1) & 1, abort, status, STATUS_WAIT_EPI)) break;
          if (!issue_s(j + 2)) break;
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ softmax + output: two threads per query row
    // A failed wait does not leave the loop: the two warps of a pair meet at a named barrier in every iteration, so
    // all of them run every iteration to its end (waits return at once when the abort word is set) and `ok` only
    // gates the stores.
    pdl_wait();                                              // `out` may still be read by the previous kernel
    const int q = warp & 3;                                  // TMEM lane quarter of this warp
    const int half = (warp - 2) >> 2;                        // 0: keys 0-63 and O columns [0, D/2); 1: the rest
    const int r = q * 32 + lane;                             // row inside the tile
    const int qi = qt * FM_BM + r;                           // query index inside the sequence
    const uint32_t lane_addr = uint32_t(q * 32) << 16;
    const int limit = a.causal ? min(kv_len, qi + shift + 1) : kv_len;     // keys [0, limit) are visible
    const uint32_t sw = uint32_t(r & 7);
    constexpr int DH = D / 2;
    const int cbeg = half * (FM_BN / 2);
    uint64_t o2[DH / 2];                                     // O, two columns per register pair
#pragma unroll
    for (int i = 0; i < DH / 2; ++i) o2[i] = 0ull;
    float m = -1e30f;
    uint64_t l2 = 0ull;                                      // row sum, even and odd keys apart
    const uint64_t scale2 = pk2(a.scale_log2, a.scale_log2);
    bool ok = true;
    uint32_t xphase = 0;
    auto exchange = [&](float mine) -> float {
      float* slot = xbuf + (xphase & 1u) * (2 * FM_BM);
      slot[half * FM_BM + r] = mine;
      pair_barrier(1 + q);
      ++xphase;
      return slot[(half ^ 1) * FM_BM + r];
    };
    auto wait_all = [&](uint64_t* bar, uint32_t parity, uint32_t code) {
      const bool good = mbar_wait(bar, parity, abort, status, code);
      ok = __all_sync(0xffffffffu, good) && ok;
    };
    for (int j = 0; j < n_kv; ++j) {
      const uint32_t tmem_buf = tmem_base + uint32_t(j & 1) * 128u;
      wait_all(&s_full[j & 1], (j >> 1) & 1, STATUS_WAIT_ACCUM);
      tc_fence_after_sync();
      const int key0 = j * FM_BN;
      // tiles whose 64 keys are visible to every row of the warp take a path without per-key masks
      const bool full = __all_sync(0xffffffffu, key0 + cbeg + FM_BN / 2 <= limit);
      // pass 1: row maximum; S is read in 16-column pieces with the next piece in flight
      const uint32_t s_addr = tmem_buf + lane_addr + uint32_t(cbeg);
      uint32_t va[16], vb[16];
      float mx = m;
      auto max16 = [&](const uint32_t (&v)[16], int c) {
        if (full) {
          float raw = fmaxf(__uint_as_float(v[0]), __uint_as_float(v[1]));
#pragma unroll
          for (int i = 2; i < 16; i += 2) raw = fmax3(raw, __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
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
      // PV(j-1) (in the other buffer) joins O before O is rescaled.  It completes about 1100 cycles after P(j-1) was
      // handed over (the MMA thread needs 85 cycles per instruction it issues), so the wait for it comes as late as
      // possible: after pass 1 and the exchange of the maxima.
      const uint32_t o_addr = tmem_base + uint32_t((j - 1) & 1) * 128u + lane_addr + uint32_t(half * DH);
      mx = fmaxf(mx, exchange(mx));
      if (j > 0) {
        wait_all(pv_full, (j - 1) & 1, STATUS_WAIT_ACCUM);
        tc_fence_after_sync();
        tmem_ld_32x16(o_addr, va);
      }
      // The reference maximum moves only when the row maximum has grown by more than 8 (a factor 256 in P, well
      // inside bf16 / fp16 and the fp32 sums): after the first tiles of a row that is rare, and a tile in which no
      // row of the warp moved skips the rescale of O and l.
      const float m_new = mx > m + 8.f ? mx : m;
      const bool moved = __any_sync(0xffffffffu, m_new != m);
      const float alpha = fm_exp2(m - m_new);
      if (j > 0) {
#pragma unroll
        for (int c = 0; c < DH; c += 32) {
          tmem_ld_wait();
          tmem_ld_32x16(o_addr + uint32_t(c + 16), vb);
#pragma unroll
          for (int i = 0; i < 8; ++i) o2[c / 2 + i] = add2(o2[c / 2 + i], pk2u(va[2 * i], va[2 * i + 1]));
          tmem_ld_wait();
          if (c + 32 < DH) tmem_ld_32x16(o_addr + uint32_t(c + 32), va);
#pragma unroll
          for (int i = 0; i < 8; ++i) o2[c / 2 + 8 + i] = add2(o2[c / 2 + 8 + i], pk2u(vb[2 * i], vb[2 * i + 1]));
        }
        tc_fence_before_sync();                              // PV(j-1) has left its buffer: S(j+1) may follow
        __syncwarp();
        if (lane == 0) mbar_arrive(&buf_free[(j - 1) & 1]);
      }
      tmem_ld_32x16(s_addr, va);                             // first piece of pass 2, in flight during the rescale
      if (moved) {
        const uint64_t alpha2 = pk2(alpha, alpha);
#pragma unroll
        for (int i = 0; i < DH / 2; ++i) o2[i] = mul2(o2[i], alpha2);
        l2 = mul2(l2, alpha2);
      }
      m = m_new;
      const uint64_t negm2 = pk2(-m, -m);
      // pass 2: probabilities -> shared memory (A operand of the second MMA: K-major, 128-byte swizzle); the 64 keys
      // of this half are exactly one swizzle atom
      uint8_t* atom = sp + half * (FM_BM * 128) + r * 128;
      auto prob16 = [&](const uint32_t (&v)[16], int c) {
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          float p[8];
          if (full) {
#pragma unroll
            for (int i = 0; i < 8; i += 2) {
              float x0, x1;
              upk2(fma2(pk2u(v[g * 8 + i], v[g * 8 + i + 1]), scale2, negm2), x0, x1);
              p[i] = fm_exp2(x0);
              p[i + 1] = fm_exp2(x1);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int key = key0 + cbeg + c + g * 8 + i;
              const float e = fm_exp2(fmaf(__uint_as_float(v[g * 8 + i]), a.scale_log2, -m));
              p[i] = key < limit ? e : 0.f;
            }
          }
#pragma unroll
          for (int i = 0; i < 8; i += 2) l2 = add2(l2, pk2(p[i], p[i + 1]));
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
      tc_fence_before_sync();                                // S(j) has left its buffer
      fence_proxy_async_smem();                              // P is visible to the tensor core
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (n_kv > 0) {
      wait_all(pv_full, (n_kv - 1) & 1, STATUS_WAIT_ACCUM);
      tc_fence_after_sync();
      const uint32_t o_addr = tmem_base + uint32_t((n_kv - 1) & 1) * 128u + lane_addr + uint32_t(half * DH);
#pragma unroll
      for (int c = 0; c < DH; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(o_addr + uint32_t(c), v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; ++i) o2[c / 2 + i] = add2(o2[c / 2 + i], pk2u(v[2 * i], v[2 * i + 1]));
      }
    }
    float l, l_odd;
    upk2(l2, l, l_odd);
    l += l_odd;
    l += exchange(l);                                        // the row sum is the sum of both halves
    if (ok && qi < q_len) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      T* orow = reinterpret_cast<T*>(a.out) + long(row0 + qi) * a.ld_o + head * D + half * DH;
#pragma unroll
      for (int c = 0; c < DH; c += 8) {
        float f[8];
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
          upk2(o2[(c + i) / 2], f[i], f[i + 1]);
          f[i] *= inv;
          f[i + 1] *= inv;
        }
        *reinterpret_cast<Vec8*>(orow + c) = pack8<T>(f);
      }
    }
  }
  pdl_trigger();
  if (*abort) {
    // a wait was abandoned: give copies and MMAs still in flight time to land before shared memory and TMEM go
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

template <class T, int D, bool PAGED>
static int launch_fmha(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const FmArgs& a, int n_seq,
                       int max_q_len, int is_bf16, uint32_t* status, cudaStream_t stream) {
  using L = FmSmem<D>;
  auto kern = fmha_kernel<T, D, PAGED>;
  static bool configured[MAX_DEVICES] = {false};
  if (first_use_on_device(configured)) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYN_SMEM) != cudaSuccess) return -10;
  }
  dim3 grid(a.heads, n_seq, (max_q_len + FM_BM - 1) / FM_BM);
  const uint32_t fmt = is_bf16 ? 1u : 0u;
  const uint32_t idesc_pv = umma_idesc(FM_BM, D, fmt, 1u) | (1u << 16);          // B (= V) is MN-major
  // V rows of 128 bytes: groups of 8 keys 1024 bytes apart; the second 64 columns of a 128-wide head one atom further
  cudaError_t err = launch(kern, grid, dim3(FM_THREADS), size_t(L::DYN_SMEM), stream, mq, mk, mv, a,
                           umma_idesc(FM_BM, FM_BN, fmt, 1u), idesc_pv, uint32_t(FM_BN * 128), 1024u, status);
  return (err == cudaSuccess && cudaGetLastError() == cudaSuccess) ? 0 : -11;
}

template <bool PAGED>
static int dispatch_fmha(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const FmArgs& a,
                         int n_seq, int max_q_len, int head_dim, int dtype, uint32_t* status, cudaStream_t stream) {
  if (dtype == 0) {
    return head_dim == 64 ? launch_fmha<__nv_bfloat16, 64, PAGED>(mq, mk, mv, a, n_seq, max_q_len, 1, status, stream)
                          : launch_fmha<__nv_bfloat16, 128, PAGED>(mq, mk, mv, a, n_seq, max_q_len, 1, status, stream);
  }
  return head_dim == 64 ? launch_fmha<__half, 64, PAGED>(mq, mk, mv, a, n_seq, max_q_len, 0, status, stream)
                        : launch_fmha<__half, 128, PAGED>(mq, mk, mv, a, n_seq, max_q_len, 0, status, stream);
}

}  // namespace ronn

using namespace ronn;

// Attention of n_seq sequences whose Q, K and V sit in the fused qkv buffer ([total_rows, ld]; head h of Q at column
// q_off + h * head_dim, kv head g of K / V at k_off / v_off + g * head_dim).  Query i of a sequence (row
// seq_start + i, i < q_len) attends to keys [0, kv_len) (rows seq_start ..), or with `causal` to keys
// j <= i + (kv_len - q_len).  out: [total_rows, ld_o], head h at column h * head_dim.  head_dim 64 or 128; ld, ld_o
// and the offsets multiples of 8.  dtype 0 bf16, 1 fp16.
extern "C" int ronn_fmha(const void* qkv, long ld, long total_rows, int q_off, int k_off, int v_off,
                         const int* seq_start, const int* q_len, const int* kv_len, void* out, long ld_o, int n_seq,
                         int max_q_len, int heads, int kv_heads, int head_dim, int causal, float scale, int dtype,
                         uint32_t* status, cudaStream_t stream) {
  if (n_seq <= 0 || max_q_len <= 0) return 0;
  if (n_seq > 65535 || max_q_len > 65535 * FM_BM) return -2;
  if ((ld & 7) || (ld_o & 7) || (q_off & 7) || (k_off & 7) || (v_off & 7) || kv_heads <= 0 || heads % kv_heads) return -2;
  if (head_dim != 64 && head_dim != 128) return -3;
  CUtensorMap m;
  int rc = make_tmap_2d(&m, qkv, uint64_t(total_rows), uint64_t(ld), uint64_t(ld), FM_BN, 64, 2);
  if (rc) return rc - 20;
  FmArgs a{seq_start, q_len, kv_len, nullptr, nullptr, out, ld_o, 0, q_off, k_off, v_off, heads, kv_heads, causal,
           scale * 1.4426950408889634f};
  return dispatch_fmha<false>(m, m, m, a, n_seq, max_q_len, head_dim, dtype, status, stream);
}

// The same with K and V read from the paged cache ([n_blocks, kv_heads, 16, head_dim] each): key t of a sequence is
// slot t % 16 of block block_tables[row, t / 16], row = bt_row[seq] (or seq when bt_row is null).  The queries are the
// last q_len positions of the context (chunked prefill, prefix hits): q: [total_rows, ld_q], rows seq_start + i.
extern "C" int ronn_fmha_paged(const void* q, long ld_q, long total_rows, int q_off, const void* kcache,
                               const void* vcache, long n_blocks, const int* block_tables, int max_blocks,
                               const int* bt_row, const int* seq_start, const int* q_len, const int* kv_len, void* out,
                               long ld_o, int n_seq, int max_q_len, int heads, int kv_heads, int head_dim, int causal,
                               float scale, int dtype, uint32_t* status, cudaStream_t stream) {
  if (n_seq <= 0 || max_q_len <= 0) return 0;
  if (n_seq > 65535 || max_q_len > 65535 * FM_BM) return -2;
  if ((ld_q & 7) || (ld_o & 7) || (q_off & 7) || kv_heads <= 0 || heads % kv_heads || max_blocks <= 0) return -2;
  if (head_dim != 64 && head_dim != 128) return -3;
  CUtensorMap mq, mk, mv;
  int rc = make_tmap_2d(&mq, q, uint64_t(total_rows), uint64_t(ld_q), uint64_t(ld_q), FM_BM, 64, 2);
  if (rc) return rc - 20;
  const uint64_t cache_rows = uint64_t(n_blocks) * kv_heads * FM_BLOCK;
  rc = make_tmap_2d(&mk, kcache, cache_rows, uint64_t(head_dim), uint64_t(head_dim), FM_BLOCK, 64, 2);
  if (rc) return rc - 30;
  rc = make_tmap_2d(&mv, vcache, cache_rows, uint64_t(head_dim), uint64_t(head_dim), FM_BLOCK, 64, 2);
  if (rc) return rc - 40;
  FmArgs a{seq_start, q_len, kv_len, block_tables, bt_row, out, ld_o, max_blocks, q_off, 0, 0, heads, kv_heads, causal,
           scale * 1.4426950408889634f};
  return dispatch_fmha<true>(mq, mk, mv, a, n_seq, max_q_len, head_dim, dtype, status, stream);
}
