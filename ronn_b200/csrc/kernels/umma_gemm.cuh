// Warp-specialised tcgen05 GEMM mainloop shared by the dense, fused-collective and
// BitNet kernels:  D[128 x BN] (TMEM, fp32/int32) = A[128 x K] * B[BN x K]^T.
//
//   warp 0      : TMA producer (one elected lane) - A and B tiles of 64 (or 128 int8) K-elements per
//                 stage, 128-byte swizzle, ring of STAGES stages guarded by full/empty mbarriers
//   warp 1      : TMEM allocator + UMMA issuer (one elected lane), tcgen05.commit releases stages
//   warps 2..5  : epilogue - each warp owns the TMEM lane quarter (warp_id % 4), reads the
//                 accumulator with tcgen05.ld in 32-column chunks and hands them to the functor
//
// The epilogue functor is called as  epi(row_in_tile, col_in_tile, acc[32])  for every 32-column
// chunk of every row.  A-tile loading can be replaced (policy ALoader) so that peers' shards
// or gathered activations feed the same mainloop.
#pragma once
#include "common.cuh"
#include "ptx_sm100.cuh"

namespace ronn {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK_BYTES = 128;          // one swizzle row: 64 bf16/fp16 or 128 int8
constexpr int GEMM_THREADS = 192;

template <int BN, int STAGES>
struct GemmSmemLayout {
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK_BYTES;
  static constexpr int B_BYTES = BN * GEMM_BK_BYTES;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int TILE_BYTES = STAGES * STAGE_BYTES;
  static constexpr int BAR_OFFSET = TILE_BYTES;
  // full[STAGES], empty[STAGES], accum, then tmem_base + abort words
  static constexpr int TOTAL = TILE_BYTES + (2 * STAGES + 1) * 8 + 16;
  static constexpr int DYN_SMEM = TOTAL + 1024;   // slack for manual 1024-byte alignment
};

struct GemmCtx {
  uint8_t* tiles;
  uint64_t* full;
  uint64_t* empty;
  uint64_t* accum;
  uint32_t* tmem_base_slot;
  volatile uint32_t* abort;
};

template <int BN, int STAGES>
__device__ __forceinline__ GemmCtx gemm_ctx(uint8_t* dyn_smem) {
  using L = GemmSmemLayout<BN, STAGES>;
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dyn_smem) + 1023) & ~uintptr_t(1023));
  GemmCtx c;
  c.tiles = base;
  c.full = reinterpret_cast<uint64_t*>(base + L::BAR_OFFSET);
  c.empty = c.full + STAGES;
  c.accum = c.empty + STAGES;
  c.tmem_base_slot = reinterpret_cast<uint32_t*>(c.accum + 1);
  c.abort = c.tmem_base_slot + 1;
  return c;
}

__host__ __device__ constexpr uint32_t tmem_cols_for(int bn) { return bn <= 32 ? 32u : (bn <= 64 ? 64u : (bn <= 128 ? 128u : 256u)); }

// Default A loader: one TMA box of 128 rows per stage.
struct TmaALoader {
  const CUtensorMap* map;
  int row0;
  __device__ __forceinline__ void load(uint8_t* smem_a, uint64_t* bar, int k_elem) const {
    tma_load_2d(smem_a, map, bar, k_elem, row0);
  }
};

// kind: 0 = f16/bf16 (UMMA_K = 16 elements = 32 bytes), 1 = int8 (UMMA_K = 32 elements = 32 bytes)
template <int BN, int STAGES, int KIND, class ALoader, class Epilogue>
__device__ __forceinline__ void gemm_tile(uint8_t* dyn_smem, const ALoader& aload, const CUtensorMap* map_b, int n0,
                                          int num_kb, int k_elems_per_block, uint32_t idesc, uint32_t* status,
                                          Epilogue& epi, int kb0 = 0) {
  using L = GemmSmemLayout<BN, STAGES>;
  GemmCtx c = gemm_ctx<BN, STAGES>(dyn_smem);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = tmem_cols_for(BN);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&c.full[s], 1);
      mbar_init(&c.empty[s], 1);
    }
    mbar_init(c.accum, 1);
    *c.abort = 0;
    mbar_fence_init();
    fence_proxy_async_smem();
  }
  __syncwarp();
  if (warp == 1) {
    tmem_alloc(c.tmem_base_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *c.tmem_base_slot;

  if (warp == 0) {
    if (lane == 0) {
      // Weights (B) never depend on the previous kernel in the stream: their first stages are requested
      // before the programmatic-dependency wait, the activations (A) after it.
      const int pre = num_kb < STAGES ? num_kb : STAGES;
      for (int kb = 0; kb < pre; ++kb) {
        uint8_t* sa = c.tiles + kb * L::STAGE_BYTES;
        mbar_expect_tx(&c.full[kb], L::STAGE_BYTES);
        tma_load_2d(sa + L::A_BYTES, map_b, &c.full[kb], (kb0 + kb) * k_elems_per_block, n0);
      }
      pdl_wait();
      for (int kb = 0; kb < pre; ++kb)
        aload.load(c.tiles + kb * L::STAGE_BYTES, &c.full[kb], (kb0 + kb) * k_elems_per_block);
      for (int kb = pre; kb < num_kb; ++kb) {
        const int s = kb % STAGES;
        const uint32_t parity = ((kb / STAGES) & 1) ^ 1;
        if (!mbar_wait(&c.empty[s], parity, c.abort, status, STATUS_WAIT_SLOT)) break;
        uint8_t* sa = c.tiles + s * L::STAGE_BYTES;
        uint8_t* sb = sa + L::A_BYTES;
        mbar_expect_tx(&c.full[s], L::STAGE_BYTES);
        aload.load(sa, &c.full[s], (kb0 + kb) * k_elems_per_block);
        tma_load_2d(sb, map_b, &c.full[s], (kb0 + kb) * k_elems_per_block, n0);
      }
    }
    __syncwarp();
    pdl_trigger();
  } else if (warp == 1) {
    if (lane == 0) {
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % STAGES;
        const uint32_t parity = (kb / STAGES) & 1;
        if (!mbar_wait(&c.full[s], parity, c.abort, status, STATUS_WAIT_TMA)) break;
        tc_fence_after_sync();
        const uint32_t sa = smem_u32(c.tiles + s * L::STAGE_BYTES);
        const uint64_t adesc = umma_desc_k128(sa);
        const uint64_t bdesc = umma_desc_k128(sa + L::A_BYTES);
#pragma unroll
        for (int k = 0; k < 4; ++k) {          // 4 x 32 bytes of K per 128-byte row
          const uint32_t acc = (kb | k) != 0;
          if (KIND == 0) umma_f16(tmem_base, adesc + 2 * k, bdesc + 2 * k, idesc, acc);
          else umma_i8(tmem_base, adesc + 2 * k, bdesc + 2 * k, idesc, acc);
        }
        umma_commit(&c.empty[s]);              // frees the stage once these MMAs have read it
      }
      umma_commit(c.accum);
    }
    __syncwarp();
    pdl_trigger();
  } else {
    const int q = warp & 3;                    // TMEM lane quarter this warp may read
    pdl_wait();                                // the epilogue reads residuals and writes buffers the predecessor may use
    bool ok = mbar_wait(c.accum, 0, c.abort, status, STATUS_WAIT_ACCUM);
    ok = __all_sync(0xffffffffu, ok);
    pdl_trigger();
    tc_fence_after_sync();
    if (ok) {
      const int row = q * 32 + lane;
#pragma unroll 1
      for (int col = 0; col < BN; col += 32) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + (uint32_t(q * 32) << 16) + uint32_t(col), r);
        tmem_ld_wait();
        epi(row, col, r);
      }
    }
  }
  // teardown: every role arrives here, also after an abandoned wait
  if (*c.abort) {
    // give copies still in flight time to land before shared memory is released
    unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) { __nanosleep(1000); }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace ronn
