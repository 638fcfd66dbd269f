// 3x3 / stride 2 / pad 1 max pooling and global average pooling for NHWC bf16 (see pool_kernels.cu).
#pragma once
#include <cuda_runtime.h>

namespace bfb {

// x: [N,H,W,C] bf16, y: [N,Ho,Wo,C] bf16, idx: [N,Ho,Wo,C] uint8 (window position of the maximum).
cudaError_t LaunchMaxPool3x3s2Forward(const void* x, void* y, void* idx, int N, int H, int W, int C, cudaStream_t stream);
cudaError_t LaunchMaxPool3x3s2Backward(const void* dy, const void* idx, void* dx, int N, int H, int W, int C,
                                       cudaStream_t stream);

// Global average pooling over the P positions of each image: x [N,P,C] bf16 -> y [N,C] bf16 (fp32 sums), and its
// gradient dx[n,p,c] = dy[n,c] / P.  C % 8 == 0.
cudaError_t LaunchAvgPoolForward(const void* x, void* y, int N, int P, int C, cudaStream_t stream);
cudaError_t LaunchAvgPoolBackward(const void* dy, void* dx, int N, int P, int C, cudaStream_t stream);

}  // namespace bfb
