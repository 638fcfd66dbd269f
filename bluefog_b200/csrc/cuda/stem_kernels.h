// Input transform of the space-to-depth ResNet stem (see stem_kernels.cu).
#pragma once
#include <cuda_runtime.h>

namespace bfb {

// x: [N, 3, H, W] fp32 or bf16 with element strides (sn, sc, sh, sw), H and W even.
// out: dense NHWC bf16 [N, (H+6)/2, (W+6)/2, 16].
cudaError_t LaunchS2dStemInput(const void* x, int x_is_bf16, void* out, int N, int H, int W, long long sn, long long sc,
                               long long sh, long long sw, cudaStream_t stream);

}  // namespace bfb
