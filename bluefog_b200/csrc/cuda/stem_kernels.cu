// Input transform of the space-to-depth stem: pad a 3-channel image by 3 pixels, fold every 2x2 pixel block
// into channels (3 x 2 x 2 = 12, ordered c*4 + dy*2 + dx) and pad to 16 channels, NHWC bf16:
//
//   out[n, hb, wb, c*4 + dy*2 + dx] = x[n, c, 2*hb + dy - 3, 2*wb + dx - 3]   (0 outside the image, 0 for channels 12..15)
//
// so that the 7x7 / stride 2 convolution becomes a 4x4 / stride 1 convolution with 16 input channels.  The
// input may be fp32 or bf16 in any dense layout (strides are arguments), which also absorbs the dtype cast
// and the NCHW -> NHWC change of the first layer.  One thread writes one output pixel (two 16-byte stores).
// The reference has no such code (its benchmark feeds torchvision's ResNet, examples/pytorch_benchmark.py:100).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "comm_kernels.h"
#include "stem_kernels.h"

namespace bfb {
namespace {

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__global__ void __launch_bounds__(256) s2d_stem_input_kernel(const T* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                                             int N, int H, int W, long long sn, long long sc,
                                                             long long sh, long long sw, int HB, int WB) {
  const long long total = (long long)N * HB * WB;
  for (long long p = (long long)blockIdx.x * blockDim.x + threadIdx.x; p < total; p += (long long)gridDim.x * blockDim.x) {
    const int wb = (int)(p % WB);
    const int hb = (int)((p / WB) % HB);
    const int n = (int)(p / ((long long)WB * HB));
    float v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = 0.f;
#pragma unroll
    for (int dy = 0; dy < 2; ++dy) {
      const int h = 2 * hb + dy - 3;
      if (h < 0 || h >= H) continue;
#pragma unroll
      for (int dx = 0; dx < 2; ++dx) {
        const int w = 2 * wb + dx - 3;
        if (w < 0 || w >= W) continue;
        const T* px = x + n * sn + h * sh + w * sw;
#pragma unroll
        for (int c = 0; c < 3; ++c) v[c * 4 + dy * 2 + dx] = to_float<T>(px[c * sc]);
      }
    }
    uint4 pk[2];
    __nv_bfloat162* hp = reinterpret_cast<__nv_bfloat162*>(pk);
#pragma unroll
    for (int i = 0; i < 8; ++i) hp[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    uint4* dst = reinterpret_cast<uint4*>(out + p * 16);
    dst[0] = pk[0];
    dst[1] = pk[1];
  }
}

}  // namespace

cudaError_t LaunchS2dStemInput(const void* x, int x_is_bf16, void* out, int N, int H, int W, long long sn, long long sc,
                               long long sh, long long sw, cudaStream_t stream) {
  if (N <= 0 || H <= 0 || W <= 0 || (H % 2) != 0 || (W % 2) != 0) return cudaErrorInvalidValue;
  const int HB = (H + 6) / 2, WB = (W + 6) / 2;
  const long long total = (long long)N * HB * WB;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (x_is_bf16)
    s2d_stem_input_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(out), N, H, W, sn, sc, sh, sw, HB, WB);
  else
    s2d_stem_input_kernel<float><<<(unsigned)blocks, 256, 0, stream>>>(
        static_cast<const float*>(x), static_cast<__nv_bfloat16*>(out), N, H, W, sn, sc, sh, sw, HB, WB);
  CountKernelLaunch();
  return cudaGetLastError();
}

}  // namespace bfb
