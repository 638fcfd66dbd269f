// 3x3 / stride 1 / pad 1 convolution of NHWC bf16 tensors as an implicit GEMM on tcgen05 (see conv_tcgen05.cu).
#pragma once
#include <cuda_runtime.h>

namespace bfb {

// Patch of output pixels one CTA owns: bn images x bh rows x bw columns, at most 128 pixels. False when W > 128.
bool Conv3x3Patch(int N, int H, int W, int* bw, int* bh, int* bn);

// Cin a multiple of 64, Cout a multiple of 8 and at least 64, W <= 128, TMA descriptors available.
bool Conv3x3Supported(int N, int H, int W, int Cin, int Cout);

// y[N,H,W,Cout] = conv3x3(x[N,H,W,Cin], w[Cout,3,3,Cin]), all bf16, dense, 16-byte aligned bases.
// flip_taps: use filter tap (2 - r, 2 - s) for input tap (r, s) (the 180-degree rotation of the input-gradient form).
// filter_mode 0: w is [Cout,3,3,Cin].  1: w is [Cin,3,3,Cout] (the filter of the forward pass when this call
// computes an input gradient; Cin, Cout are this call's reduction and output channels), read as an MN-major operand.
// status: device word set to 1 when a bounded wait inside the kernel expired (may be null).
cudaError_t LaunchConv3x3Nhwc(const void* x, const void* w, void* y, int N, int H, int W, int Cin, int Cout,
                              int flip_taps, int filter_mode, unsigned int* status, cudaStream_t stream);

}  // namespace bfb
