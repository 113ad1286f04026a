// Persistent warp-specialised tcgen05 GEMM mainloop.
//
// One CTA walks a list of output tiles (tile = blockIdx.x, += gridDim.x).  The TMA ring and its
// mbarrier phases run continuously across tiles; the accumulator is double-buffered in TMEM
// (two BN-column buffers), so the epilogue of tile j overlaps the MMAs of tile j + 1:
//
//   warp 0     TMA producer       waits empty[s]      -> expect_tx + A/B loads into stage s
//   warp 1     UMMA issuer        waits acc_empty[b], full[s] -> tcgen05.mma into buffer b,
//                                 tcgen05.commit -> empty[s]; after the tile: commit -> acc_full[b]
//   warps 2-9  epilogue           waits acc_full[b]   -> tcgen05.ld 32-column chunks -> functor,
//                                 then one arrival per warp on acc_empty[b].  Warp w reads TMEM lane quarter
//                                 w % 4; the two warps of a quarter drain one half of the columns each (with four
//                                 epilogue warps the epilogue of a 128 x 256 tile was as long as a 12-block main loop)
//
// Because every CTA of the grid is resident at once (grid <= SMs x CTAs/SM), a caller may add a
// grid-wide or cross-GPU phase after the tile loop without risking a scheduling deadlock.
//
// The `Problem` policy supplies the tile list and the I/O:
//   int  num_tiles() const
//   void tile(int t, int& m0, int& n0, int& kb0, int& nkb) const     k-block range of the tile
//   void load_a(uint8_t* smem, uint64_t* bar, int k_elem, int m0) const
//   void load_b(uint8_t* smem, uint64_t* bar, int k_elem, int n0) const
//   static constexpr bool kForceStage                                 true: `stage` below is never null
//   void epilogue(int t, int m0, int n0, int row, int col, uint32_t (&acc)[32], uint8_t* stage)   row/col within the
//        tile; stage: 32 x 80 bytes of shared memory owned by the calling warp (to re-shape its stores), or null
#pragma once
#include "common.cuh"
#include "ptx_sm100.cuh"

namespace ronn {

constexpr int PG_BM = 128;
constexpr int PG_EPI_WARPS = 8;                  // two warps per TMEM lane quarter, each drains half of the columns
constexpr int PG_THREADS = 64 + 32 * PG_EPI_WARPS;

// FORCE_STAGE: always reserve the per-warp store-staging area (kernels whose epilogue depends on it); otherwise only
// the deep-ring variants (one CTA per SM) carry it, so the shallow ones still fit two CTAs per SM.
// KA: 128-byte K atoms per stage.  A hand-over of a stage costs the MMA issuer ~220 cycles of barrier and fence
// traffic beside the ~70 cycles per MMA (four per atom), whatever the tile width: with two atoms per stage a skinny
// GEMM, whose CTAs are chains of K blocks, pays it half as often.
template <int BN, int STAGES, bool FORCE_STAGE = false, int KA = 1>
struct PGemmSmem {
  static constexpr int A_BYTES = PG_BM * 128;
  static constexpr int B_BYTES = BN * 128;
  static constexpr int ATOM_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGE_BYTES = KA * ATOM_BYTES;
  static constexpr int TILE_BYTES = STAGES * STAGE_BYTES;
  static constexpr int NUM_BARS = 2 * STAGES + 4;          // full, empty, acc_full[2], acc_empty[2]
  static constexpr int OUT_STAGE_ROW = 80;                 // 64 bytes of a row + padding against bank conflicts
  static constexpr int OUT_STAGE_BYTES =
      (FORCE_STAGE || STAGES * KA * (PG_BM * 128 + BN * 128) > 100 * 1024) ? PG_EPI_WARPS * 32 * OUT_STAGE_ROW : 0;   // per epilogue warp
  static constexpr int TOTAL = TILE_BYTES + NUM_BARS * 8 + 16 + OUT_STAGE_BYTES;
  static constexpr int DYN_SMEM = TOTAL + 1024;            // slack for manual 1024-byte alignment
  static constexpr uint32_t TMEM_COLS = (2 * BN <= 32) ? 32u : (2 * BN <= 64 ? 64u : (2 * BN <= 128 ? 128u : (2 * BN <= 256 ? 256u : 512u)));
};

// KIND: 0 = f16/bf16 operands, 1 = int8 operands.  k_elems: K elements per 128-byte smem row (64 or 128).
template <int BN, int STAGES, int KIND, class Problem, int KA = 1>
__device__ __forceinline__ void gemm_persistent(uint8_t* dyn_smem, Problem& prob, int k_elems, uint32_t idesc,
                                                uint32_t* status) {
  using L = PGemmSmem<BN, STAGES, Problem::kForceStage, KA>;
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dyn_smem) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(tiles + L::TILE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile uint32_t* abort = tmem_slot + 1;
  uint8_t* out_stage = reinterpret_cast<uint8_t*>(tmem_slot + 4);      // 16-byte aligned, behind the barriers
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], PG_EPI_WARPS);    // one arrival per epilogue warp
    }
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
  const int ntiles = prob.num_tiles();

  if (warp == 0) {
    if (lane == 0) {
      // Weights (B) never depend on the previous kernel in the stream: the first stages of the first tile are
      // requested before the programmatic-dependency wait, the activations (A) after it.
      // A stage holds KA atoms [A_0][B_0][A_1][B_1]...; the last stage of a tile may hold fewer.
      int pre = 0;
      if (int(blockIdx.x) < ntiles) {
        int m0, n0, kb0, nkb;
        prob.tile(blockIdx.x, m0, n0, kb0, nkb);
        const int nsb = (nkb + KA - 1) / KA;
        pre = nsb < STAGES ? nsb : STAGES;
        for (int sb = 0; sb < pre; ++sb) {
          const int na = min(KA, nkb - sb * KA);
          mbar_expect_tx(&full[sb], uint32_t(na * L::ATOM_BYTES));
          for (int a = 0; a < na; ++a)
            prob.load_b(tiles + sb * L::STAGE_BYTES + a * L::ATOM_BYTES + L::A_BYTES, &full[sb], (kb0 + sb * KA + a) * k_elems, n0);
        }
      }
      pdl_wait();
      pdl_trigger();                             // the predecessor is complete: let the successor launch and run its
                                                 // set-up (barriers, TMEM, weight prefetch) under this kernel
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < ntiles && ok; t += gridDim.x) {
        int m0, n0, kb0, nkb;
        prob.tile(t, m0, n0, kb0, nkb);
        const int nsb = (nkb + KA - 1) / KA;
        for (int sb = 0; sb < nsb; ++sb, ++it) {
          const int s = it % STAGES;
          const int na = min(KA, nkb - sb * KA);
          uint8_t* sa = tiles + s * L::STAGE_BYTES;
          if (it < uint32_t(pre)) {              // B already in flight, barrier already armed
            for (int a = 0; a < na; ++a) prob.load_a(sa + a * L::ATOM_BYTES, &full[s], (kb0 + sb * KA + a) * k_elems, m0);
            continue;
          }
          if (!mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1, abort, status, STATUS_WAIT_SLOT)) { ok = false; break; }
          mbar_expect_tx(&full[s], uint32_t(na * L::ATOM_BYTES));
          for (int a = 0; a < na; ++a) {
            prob.load_a(sa + a * L::ATOM_BYTES, &full[s], (kb0 + sb * KA + a) * k_elems, m0);
            prob.load_b(sa + a * L::ATOM_BYTES + L::A_BYTES, &full[s], (kb0 + sb * KA + a) * k_elems, n0);
          }
        }
      }
    }
    __syncwarp();
    pdl_trigger();
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t it = 0, j = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < ntiles && ok; t += gridDim.x, ++j) {
        int m0, n0, kb0, nkb;
        prob.tile(t, m0, n0, kb0, nkb);
        const uint32_t buf = j & 1;
        if (!mbar_wait(&acc_empty[buf], ((j >> 1) & 1) ^ 1, abort, status, STATUS_WAIT_EPI)) break;
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + buf * BN;
        const int nsb = (nkb + KA - 1) / KA;
        // a barrier poll takes ~90 cycles to answer: the next stage is probed before this stage's MMAs are issued
        bool ready = false;
        for (int sb = 0; sb < nsb; ++sb, ++it) {
          const int s = it % STAGES;
          if (!ready && !mbar_wait(&full[s], (it / STAGES) & 1, abort, status, STATUS_WAIT_TMA)) { ok = false; break; }
          tc_fence_after_sync();
          ready = sb + 1 < nsb && mbar_try_wait(&full[(it + 1) % STAGES], ((it + 1) / STAGES) & 1);
          const int na = min(KA, nkb - sb * KA);
          const uint32_t sa = smem_u32(tiles + s * L::STAGE_BYTES);
#pragma unroll
          for (int a = 0; a < KA; ++a) {
            if (a < na) {
              const uint64_t adesc = umma_desc_k128(sa + a * L::ATOM_BYTES);
              const uint64_t bdesc = umma_desc_k128(sa + a * L::ATOM_BYTES + L::A_BYTES);
#pragma unroll
              for (int k = 0; k < 4; ++k) {      // 4 x 32 bytes of K per 128-byte row
                const uint32_t acc = (sb | a | k) != 0;
                if (KIND == 0) umma_f16(tmem_d, adesc + 2 * k, bdesc + 2 * k, idesc, acc);
                else umma_i8(tmem_d, adesc + 2 * k, bdesc + 2 * k, idesc, acc);
              }
            }
          }
          umma_commit(&empty[s]);                // frees the stage once these MMAs have read it
        }
        if (ok) umma_commit(&acc_full[buf]);
      }
    }
    __syncwarp();
    pdl_trigger();
  } else {
    const int q = warp & 3;                      // TMEM lane quarter this warp may read
    const int half = (warp - 2) >> 2;            // which half of the columns this warp drains
    uint8_t* stage_w = L::OUT_STAGE_BYTES ? out_stage + (warp - 2) * (32 * L::OUT_STAGE_ROW) : nullptr;
    pdl_wait();                                  // the epilogue reads residuals and writes buffers the predecessor may use
    uint32_t j = 0;
    for (int t = blockIdx.x; t < ntiles; t += gridDim.x, ++j) {
      int m0, n0, kb0, nkb;
      prob.tile(t, m0, n0, kb0, nkb);
      const uint32_t buf = j & 1;
      // the accumulator hand-over is on the critical path of a skinny GEMM (one tile per CTA): every lane polls
      bool ok = mbar_wait(&acc_full[buf], (j >> 1) & 1, abort, status, STATUS_WAIT_ACCUM);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const int row = q * 32 + lane;
      const uint32_t tacc = tmem_base + (uint32_t(q * 32) << 16) + buf * BN;
      // TMEM loads are long-latency: the load of the next 32 columns is in flight while this chunk is converted and
      // stored.  The accumulator buffer is handed back as soon as its last load has landed.
      if (BN == 32) {
        if (half == 0) {
          uint32_t r0[32];
          tmem_ld_32x32(tacc, r0);
          tmem_ld_wait();
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty[buf]);
          prob.epilogue(t, m0, n0, row, 0, r0, stage_w);
        } else {
          if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
      } else {
        constexpr int HALF = BN / 2;
        const int c0 = half * HALF;
        uint32_t r0[32], r1[32];
        tmem_ld_32x32(tacc + uint32_t(c0), r0);
        if (HALF == 32) {
          tmem_ld_wait();
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty[buf]);
          prob.epilogue(t, m0, n0, row, c0, r0, stage_w);
        } else {
#pragma unroll 1
          for (int col = c0; col < c0 + HALF; col += 64) {
            tmem_ld_wait();
            tmem_ld_32x32(tacc + uint32_t(col + 32), r1);
            prob.epilogue(t, m0, n0, row, col, r0, stage_w);
            tmem_ld_wait();
            if (col + 64 < c0 + HALF) {
              tmem_ld_32x32(tacc + uint32_t(col + 64), r0);
            } else {
              tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) mbar_arrive(&acc_empty[buf]);
            }
            prob.epilogue(t, m0, n0, row, col + 32, r1, stage_w);
          }
        }
      }
    }
    pdl_trigger();
  }
  // teardown: every role arrives here, also after an abandoned wait
  if (*abort) {
    // give copies still in flight time to land before shared memory is released
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

}  // namespace ronn
