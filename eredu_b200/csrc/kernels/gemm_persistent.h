// Launcher of the persistent large-M tcgen05 GEMM (gemm_persistent.cu), called by eredu_gemm_bf16 for prefill-
// sized problems. Returns a cudaError_t, a negative tensor-map error, or kPersistentUnsupported when the problem
// does not meet the kernel's layout requirements (the caller then uses the one-tile-per-CTA kernel).
#pragma once
#include <cuda_runtime.h>

namespace eredu {

constexpr int kPersistentUnsupported = -7777;

int launch_gemm_persistent(const void* X, const void* W, void* Y, const void* residual, const void* bias, int M, int N,
                           int K, int ldx, int ldw, int ldy, int ldr, int w_rows, int dual, int dual_row_offset,
                           int sm_count, int* status, const float* ssq_in, int ssq_parts, float norm_eps, int norm_dim,
                           float* ssq_out, cudaStream_t stream);

}  // namespace eredu
