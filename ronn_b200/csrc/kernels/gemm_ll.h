// C interface of the low-latency tensor-parallel projection (gemm_ll.cu): row-parallel GEMM + two-phase all-reduce
// over NVLink with {data, sequence} words + bias, residual and LayerNorm / RMSNorm in one launch.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define RONN_LL_MAX_RANKS 8

#ifdef __cplusplus
extern "C" {
#endif

// scatter_area[r] / result_area[r]: address of rank r's copy of the two symmetric areas as mapped into this process;
// result_mc: multicast address of the result area (nvls = 1) or null.  Both areas start zeroed.  A value takes
// 4 bytes in an area (two 16-bit values share an 8-byte word with the call's sequence number).
typedef struct RonnGemmLLParams {
  const void* A;                 // [M, K] activations of this rank's K shard, row stride lda (elements)
  const void* W;                 // [N, K] weights of this rank's K shard, row stride ldw
  int M, N, K, lda, ldw;         // N % 32 == 0
  int bn;                        // 0 = auto, else 32 | 64 | 128
  int splitk;                    // K slices per rank (clamped so that slices x world <= 8 and no slice is empty)
  int dtype;                     // 0 bf16, 1 fp16
  void* scatter_area[RONN_LL_MAX_RANKS];
  long scatter_parity_stride;    // bytes per parity: >= world * slices * ceil(M / world) * N * 4
  void* result_area[RONN_LL_MAX_RANKS];
  void* result_mc;
  long result_parity_stride;     // bytes per parity: >= M * N * 4
  void* state;                   // 32 zero-initialised bytes in local memory, 8-byte aligned
  int rank, world, nvls;
  void* out;                     // X [M, ld_out], local memory
  void* norm_out;                // H (norm_mode != 0), same row stride
  long ld_out;
  const void* bias;              // [N] or null
  const void* residual;          // [M, ld_res] or null (the same values on every rank)
  long ld_res;
  const void* gamma;
  const void* beta;
  float eps;
  int norm_mode;                 // 0 none, 1 LayerNorm, 2 RMSNorm (N <= 8192), 3 RMSNorm * gamma then per-row int8
                                 // quantisation into quant_out / quant_scale (what a BitLinear layer reads next)
  double wait_seconds;           // limit of every poll
  void* trace;                   // optional: 8 x uint64 %globaltimer stamps per CTA (entry, partials sent, -, owned rows
                                 // reduced and broadcast, all rows unpacked and normalised, -, -, exit)
  int phases;                    // 0 = the whole call.  Otherwise a mask (1 GEMM + scatter, 2 owner reduce + broadcast,
                                 // 4 unpack + norm + epoch advance) of the parts this launch runs: with every rank's
                                 // areas in ONE device's memory, the ranks of a call can then be run one after the
                                 // other (all ranks' part 1, then all part 2, then all part 4) and no launch waits
                                 // for a later one.  That is how W = 4 and 8 are checked on a single GPU.
  void* quant_out;               // norm_mode 3: int8 [M, N] (row stride N bytes)
  float* quant_scale;            // norm_mode 3: [M] scales (max |normalised row| / 127)
} RonnGemmLLParams;

int ronn_gemm_ll(const RonnGemmLLParams* p, uint32_t* status, cudaStream_t stream);

// The same protocol behind the ternary x int8 BitLinear GEMM (bitnet.cu).  `ll` carries M, N, K (this rank's K shard,
// K % 64 == 0), dtype of the output, the areas, state, rank / world / nvls, out, residual, norm and wait fields; its
// A, W, lda, ldw, bn and splitk fields are not used.
typedef struct RonnBitLinearLLParams {
  const void* xq;                // int8 activations [M, K], row stride ldx bytes (ldx % 16 == 0)
  const void* w_packed;          // [N, K / 4] two-bit codes, 16-byte aligned
  const float* x_scale;          // [M] per-token scales of this rank's activation shard
  float w_scale;
  int ldx;
  RonnGemmLLParams ll;
} RonnBitLinearLLParams;

int ronn_bitlinear_ll(const RonnBitLinearLLParams* p, uint32_t* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
