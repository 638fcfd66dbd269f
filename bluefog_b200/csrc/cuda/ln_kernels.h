// LayerNorm forward/backward over the last dimension of a bf16 [R, C] matrix (see ln_kernels.cu).
#pragma once
#include <cuda_runtime.h>

namespace bfb {

// C % 8 == 0 and C <= 2048 (a warp keeps one row in registers).
bool LnShapeSupported(long long R, int C);

// gamma/beta: C values, fp32 or bf16 (param_bf16).  mean/rstd: R fp32 values each (written).
cudaError_t LaunchLnForward(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd,
                            long long R, int C, float eps, int param_bf16, cudaStream_t stream);

// dgamma_zeroed/dbeta_zeroed: C fp32 values each that hold zeros on entry; the kernel adds into them.
// addend / colsum_zeroed (both or neither): dx = LN'(dy) + addend (bf16 [R, C]) and colsum_zeroed[c] += sum_r dx[r, c];
// cudaErrorNotSupported when the kernel that takes them cannot run this shape (the caller then adds and sums itself).
cudaError_t LaunchLnBackward(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd,
                             void* dx, float* dgamma_zeroed, float* dbeta_zeroed, long long R, int C, int param_bf16,
                             cudaStream_t stream, const void* addend = nullptr, float* colsum_zeroed = nullptr);

// out_zeroed[c] += sum_r x[r, c] for a bf16 [R, C] row-major matrix (C % 8 == 0); fp32 sums that hold zeros on entry.
cudaError_t LaunchColumnSum(const void* x, float* out_zeroed, long long R, int C, cudaStream_t stream);

}  // namespace bfb
