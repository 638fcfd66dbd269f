// bf16 GEMM on tcgen05 tensor cores (see gemm_tcgen05.cu).
#pragma once
#include <cuda_runtime.h>

namespace bfb {

enum GemmAct : int { kActNone = 0, kActRelu = 1, kActGeluTanh = 2 };

// True when the driver exposes cuTensorMapEncodeTiled (needed to build TMA descriptors).
bool GemmSupported();

// out[M,N] (bf16, row-major) = act(a[M,K] * b[N,K]^T + bias[N]); a, b bf16 row-major, K % 8 == 0,
// all base pointers 16-byte aligned. bias may be null. status: device word set to 1 when a
// bounded wait inside the kernel expired (may be null).
cudaError_t LaunchGemmBf16NT(const void* a, const void* b, void* out, const void* bias, int M, int N, int K, int act,
                             unsigned int* status, cudaStream_t stream);

// out[M,N] = a[M,K] * b[K,N] with b row-major (consumed as an MN-major operand); K % 8 == 0, N % 8 == 0.
cudaError_t LaunchGemmBf16NN(const void* a, const void* b, void* out, int M, int N, int K, unsigned int* status,
                             cudaStream_t stream);

// out[M,N] = a[K,M]^T * b[K,N], a and b row-major (both consumed MN-major); M % 8 == 0, N % 8 == 0.
cudaError_t LaunchGemmBf16TN(const void* a, const void* b, void* out, int M, int N, int K, unsigned int* status,
                             cudaStream_t stream);

}  // namespace bfb
