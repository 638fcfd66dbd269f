// Token + position embedding of a GPT-style model, forward and backward (see embed_kernels.cu).
#pragma once
#include <cuda_runtime.h>

namespace bfb {

// out[i, :] = wte[idx[i], :] + wpe[i % T, :] for i < N = B * T; bf16 rows of C values, C % 8 == 0; idx: int64 [N].
// An index outside [0, V) gives a row of wpe alone and sets *bad_index_flag (a device int, may be null) to 1.
cudaError_t LaunchEmbedForward(const long long* idx, const void* wte, const void* wpe, void* out, long long N, int T,
                               int C, long long V, int* bad_index_flag, cudaStream_t stream);

// d_wte (bf16 [V, C], every row written: zeros where no token points) and d_wpe (bf16 [T, C]) from dx (bf16 [N, C]).
// Rows of the same token are added up in fp32: slot (int32 [V], all INT_MAX on entry and on exit) picks the first
// position of every token as its representative, acc (fp32 [N, C], zeros on entry and on exit) collects the sums there.
cudaError_t LaunchEmbedBackward(const long long* idx, const void* dx, void* d_wte, void* d_wpe, int* slot, float* acc,
                                long long N, int T, int C, long long V, cudaStream_t stream);

}  // namespace bfb
