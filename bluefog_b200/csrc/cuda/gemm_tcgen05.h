// bf16 GEMM on tcgen05 tensor cores (see gemm_tcgen05.cu).
#pragma once
#include <cuda_runtime.h>

namespace bfb {

enum GemmAct : int { kActNone = 0, kActRelu = 1, kActGeluTanh = 2 };
// Extra work of the epilogue: store the pre-activation value (accumulator + bias) to a second matrix besides
// act(...) of it; or multiply the result by GELU'(aux[m, n]) (the input gradient through a GELU whose
// pre-activation was kept).
enum GemmEpi : int { kEpiNone = 0, kEpiStorePreact = 1, kEpiMulGeluGrad = 2, kEpiColumnStats = 3, kEpiAddAux = 4 };

// True when the driver exposes cuTensorMapEncodeTiled (needed to build TMA descriptors).
bool GemmSupported();

// out[M,N] (bf16, row-major) = act(a[M,K] * b[N,K]^T + bias[N]); a, b bf16 row-major, K % 8 == 0,
// all base pointers 16-byte aligned. bias may be null. status: device word set to 1 when a
// bounded wait inside the kernel expired (may be null).
// preact_out (optional, [M,N] bf16, needs N % 8 == 0): receives a*b^T + bias before the activation.
// col_stats (optional, 2*N floats, needs N % 8 == 0, no bias, no activation): col_stats[n] += sum_m out[m,n] and
// col_stats[N + n] += sum_m out[m,n]^2 over the rounded bf16 output (the batch statistics of a following
// normalisation layer, taken while the tile is still on chip).
cudaError_t LaunchGemmBf16NT(const void* a, const void* b, void* out, const void* bias, int M, int N, int K, int act,
                             unsigned int* status, cudaStream_t stream, void* preact_out = nullptr,
                             float* col_stats = nullptr, const void* addend = nullptr);
// addend: bf16 [M, N] added to the product (and the bias) in the epilogue, e.g. the residual stream a layer's output
// joins; needs act == 0, N % 8 == 0, no preact_out and no col_stats.

// out[M,N] = a[M,K] * b[K,N] with b row-major (consumed as an MN-major operand); K % 8 == 0, N % 8 == 0.
// gelu_preact (optional, [M,N] bf16): the result is multiplied elementwise by GELU'(gelu_preact).
// addend (optional, [M,N] bf16, not together with gelu_preact): added to the product in fp32 before rounding (the
// gradient that reaches a block's input through its shortcut, so that no separate addition pass is needed).
cudaError_t LaunchGemmBf16NN(const void* a, const void* b, void* out, int M, int N, int K, unsigned int* status,
                             cudaStream_t stream, const void* gelu_preact = nullptr, const void* addend = nullptr);

// out[M,N] = a[K,M]^T * b[K,N], a and b row-major (both consumed MN-major); M % 8 == 0, N % 8 == 0.
cudaError_t LaunchGemmBf16TN(const void* a, const void* b, void* out, int M, int N, int K, unsigned int* status,
                             cudaStream_t stream);

}  // namespace bfb
