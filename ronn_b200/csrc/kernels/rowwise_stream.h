// Streaming row-wise kernels (rowwise_stream.cu): the many-rows path of LayerNorm / RMSNorm, softmax and the int8
// activation quantisers.
#pragma once
#include <cuda_runtime.h>

namespace ronn {

// mode: 0 LayerNorm, 1 RMSNorm, 2 softmax, 3 per-row absmax int8 quantisation, 4 RMSNorm * gamma then quantisation.
// For modes 3 and 4 `y` is the int8 output (row stride ld_y bytes) and `scale_out` receives one fp32 scale per row.
// Returns 1 when the kernel was launched, 0 when the shape does not qualify (few rows, odd strides or alignment, a
// row too long for the shared-memory ring) and the caller should use its own kernel, < 0 on a launch error.
int rowwise_stream_try(int mode, const void* x, const void* res, const void* gamma, const void* beta, void* y,
                       void* sum_out, float* scale_out, long rows, int H, long ld_x, long ld_res, long ld_y, float eps,
                       int dtype, cudaStream_t stream);

}  // namespace ronn
