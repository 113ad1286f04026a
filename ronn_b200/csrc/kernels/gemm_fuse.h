// C interface of the fused skinny GEMM (gemm_fuse.cu): split-K GEMM + cross-slice / cross-rank row reduction + bias,
// activation, residual and LayerNorm / RMSNorm in one launch.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define RONN_FUSE_MAX_RANKS 8
#define RONN_FUSE_MAX_ROW_TILES 64     /* M <= 8192 */

#ifdef __cplusplus
extern "C" {
#endif

// Pointer arrays hold one entry per rank (entry 0 only when world == 1).  With world > 1 every entry is the address of
// the same symmetric allocation on that rank as mapped into this process, and the *_mc members are the multicast
// addresses of those allocations (NVLS mode, nvls = 1) or null.
typedef struct RonnGemmFuseParams {
  const void* A;                 // [M, K] activations, row stride lda (elements)
  const void* W;                 // [N, K] weights, row stride ldw
  int M, N, K, lda, ldw;
  int splitk;                    // K slices wanted (clamped so that every slice is non-empty)
  int bn;                        // 0 = auto, else 32 | 64 | 128 (| 0x1000 deep ring, | 0x2000 shallow ring)
  int dtype;                     // 0 bf16, 1 fp16
  void* part[RONN_FUSE_MAX_RANKS];      // fp32 scratch: two parity slots of parity_stride floats each
  void* part_mc;
  long parity_stride;            // floats per parity slot (>= slices * M * N)
  void* flags[RONN_FUSE_MAX_RANKS];     // ronn_gemm_fuse_flag_ints() zero-initialised uint32 counters
  void* flags_mc;
  void* state;                   // ronn_gemm_fuse_state_ints() zero-initialised uint32 in local memory
  int rank, world;
  int nvls;                      // 1: multimem instructions over the multicast addresses, 0: peer loads / stores
  int scatter;                   // 1: reduce-scatter (rank r keeps rows [r ceil(M / world), ...) as rows 0.. of out[rank])
  void* out[RONN_FUSE_MAX_RANKS];       // X, row stride ld_out
  void* out_mc;
  void* norm_out[RONN_FUSE_MAX_RANKS];  // H (norm_mode != 0), same row stride
  void* norm_mc;
  long ld_out;
  const void* bias;              // [N] or null
  const void* residual;          // [rows of out, ld_res] or null; read by the row's owner only
  long ld_res;
  const void* gamma;
  const void* beta;
  float eps;
  int norm_mode;                 // 0 none, 1 LayerNorm, 2 RMSNorm (N <= 8192)
  int act;                       // 0 none, 1 relu, 2 gelu (tanh form); applied before the residual
  double wait_seconds;           // limit of every cross-CTA / cross-rank wait
  void* trace;                   // optional: 8 x uint64 %globaltimer stamps per CTA (entry, GEMM done, published,
                                 // first wait over, rows done, delivered sent, delivered seen, exit)
} RonnGemmFuseParams;

// Returns 0 on success, a negative code for a configuration the kernel does not take.
int ronn_gemm_fuse(const RonnGemmFuseParams* p, uint32_t* status, cudaStream_t stream);
int ronn_gemm_fuse_state_ints(void);
int ronn_gemm_fuse_flag_ints(void);

#ifdef __cplusplus
}
#endif
