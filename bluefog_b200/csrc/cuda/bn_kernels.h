// Fused training-mode BatchNorm (+ReLU, +residual) for NHWC bf16 activations (see bn_kernels.cu).
#pragma once
#include <cuda_runtime.h>

namespace bfb {

// C must be a multiple of 8, at most 2048, and C/8 must divide 256.
bool BnShapeSupported(long long R, int C);

// sums: 2*C floats, zeroed by the caller. gamma/beta: C values, bf16 when param_bf16 else fp32.
// mask: R*C/8 bytes, bit i of byte (r*C/8 + g) = (y[r, 8g+i] > 0); required when relu != 0.
//
// sum_copies >= 1: `sums` holds sum_copies * 2*C zeroed floats followed by one zeroed 32-bit word (all zeroed by the
// caller, used once).  Then, when the activation is small enough for the SMs to keep their share of the rows in
// shared memory, the pass is ONE cooperative launch (statistics, grid-wide barrier on that word, apply) instead of
// two kernels; blocks spread their additions over the copies.  The bounded barrier wait reports to `status` (set
// to 1).  BnSumCopies(C) is the recommended count.  BLUEFOG_B200_BN_FUSED=0 keeps the two-kernel form.
int BnSumCopies(int C);
cudaError_t LaunchBnForward(const void* x, const void* residual, void* y, void* mask, float* sums, const void* gamma, const void* beta,
                            float* running_mean, float* running_var, float* save_mean, float* save_rstd, long long R,
                            int C, float eps, float momentum, int relu, int param_bf16, cudaStream_t stream,
                            int stats_ready = 0,    // 1: sums already hold sum(x), sum(x^2); no statistics pass
                            int sum_copies = 0, unsigned int* status = nullptr);

// dy2: optional second addend of the incoming gradient (same shape as dy): the kernels use dy + dy2.
cudaError_t LaunchBnBackward(const void* dy, const void* dy2, const void* mask, const void* x, void* dx, void* dres, float* sums,
                             const float* save_mean, const float* save_rstd, const void* gamma, void* dgamma,
                             void* dbeta, long long R, int C, int relu, int param_bf16, cudaStream_t stream,
                             int sum_copies = 0, unsigned int* status = nullptr);

}  // namespace bfb
