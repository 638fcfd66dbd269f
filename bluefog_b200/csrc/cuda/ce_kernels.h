// Mean cross-entropy over the rows of a bf16 logits matrix (see ce_kernels.cu).
#pragma once
#include <cuda_runtime.h>

namespace bfb {

// x: bf16 [R, C] row-major, C % 8 == 0; target: int64 [R] with 0 <= target < C.
// lse: fp32 [R] (written); loss_sum_zeroed: fp32 scalar holding 0 on entry, receives the mean loss.
cudaError_t LaunchCrossEntropyForward(const void* x, const long long* target, float* lse, float* loss_sum_zeroed,
                                      long long R, int C, cudaStream_t stream);

// dx (bf16 [R, C]) = (softmax(x) - onehot(target)) * grad_out[0] / R; grad_out: one fp32 value on the device.
cudaError_t LaunchCrossEntropyBackward(const void* x, const long long* target, const float* lse, const float* grad_out,
                                       void* dx, long long R, int C, cudaStream_t stream);

}  // namespace bfb
