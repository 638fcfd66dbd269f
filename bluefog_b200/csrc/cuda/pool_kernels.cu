// 3x3 / stride 2 / pad 1 max pooling for NHWC bf16 activations, forward and backward.
// Forward stores, next to the maximum, the position (0..8) of the first maximum inside the
// window; backward gathers: every input pixel looks at the (at most four) windows that
// contain it and adds the gradients of those that chose it, so no atomics are needed and the
// result is deterministic.  Eight channels per thread, 16-byte accesses.
// Global average pooling (the layer before a ResNet classifier) forward and backward as two more streaming kernels.
// The reference leaves pooling to PyTorch (examples/pytorch_benchmark.py:100).
#include "pool_kernels.h"

#include <cuda_bf16.h>

#include "comm_kernels.h"

namespace bfb {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  const unsigned* u = reinterpret_cast<const unsigned*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(u[i] << 16);
    f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 v;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return v;
}

__global__ void __launch_bounds__(kThreads) maxpool_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                               __nv_bfloat16* __restrict__ y,
                                                               unsigned char* __restrict__ idx, int N, int H, int W,
                                                               int C, int Ho, int Wo) {
  const int CG = C >> 3;
  const long long total = (long long)N * Ho * Wo * CG;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
    const int g = (int)(t % CG);
    long long pix = t / CG;
    const int wo = (int)(pix % Wo);
    pix /= Wo;
    const int ho = (int)(pix % Ho);
    const int n = (int)(pix / Ho);
    float best[8];
    unsigned char where[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      best[i] = -INFINITY;
      where[i] = 0;
    }
#pragma unroll
    for (int dh = 0; dh < 3; ++dh) {
      const int h = 2 * ho - 1 + dh;
      if (h < 0 || h >= H) continue;
#pragma unroll
      for (int dw = 0; dw < 3; ++dw) {
        const int w = 2 * wo - 1 + dw;
        if (w < 0 || w >= W) continue;
        float f[8];
        unpack8(*reinterpret_cast<const uint4*>(x + (((long long)n * H + h) * W + w) * C + g * 8), f);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (f[i] > best[i] || (f[i] != f[i] && !(best[i] != best[i]))) {   // strict: first maximum wins; NaN propagates
            best[i] = f[i];
            where[i] = (unsigned char)(dh * 3 + dw);
          }
        }
      }
    }
    *reinterpret_cast<uint4*>(y + t * 8) = pack8(best);
    uint2 packed;
    unsigned char* pb = reinterpret_cast<unsigned char*>(&packed);
#pragma unroll
    for (int i = 0; i < 8; ++i) pb[i] = where[i];
    *reinterpret_cast<uint2*>(idx + t * 8) = packed;
  }
}

__global__ void __launch_bounds__(kThreads) maxpool_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                                               const unsigned char* __restrict__ idx,
                                                               __nv_bfloat16* __restrict__ dx, int N, int H, int W, int C,
                                                               int Ho, int Wo) {
  const int CG = C >> 3;
  const long long total = (long long)N * H * W * CG;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
    const int g = (int)(t % CG);
    long long pix = t / CG;
    const int w = (int)(pix % W);
    pix /= W;
    const int h = (int)(pix % H);
    const int n = (int)(pix / H);
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    // windows (ho, wo) with 2*ho-1 <= h <= 2*ho+1
    const int ho_lo = h > 0 ? (h - 1 + 1) / 2 : 0;     // ceil((h-1)/2)
    const int ho_hi = (h + 1) / 2;
    const int wo_lo = w > 0 ? (w - 1 + 1) / 2 : 0;
    const int wo_hi = (w + 1) / 2;
    for (int ho = ho_lo; ho <= ho_hi && ho < Ho; ++ho) {
      const int dh = h - (2 * ho - 1);
      for (int wo = wo_lo; wo <= wo_hi && wo < Wo; ++wo) {
        const int dw = w - (2 * wo - 1);
        const unsigned char code = (unsigned char)(dh * 3 + dw);
        const long long o = (((long long)n * Ho + ho) * Wo + wo) * CG + g;
        const uint2 packed = *reinterpret_cast<const uint2*>(idx + o * 8);
        const unsigned char* pb = reinterpret_cast<const unsigned char*>(&packed);
        float f[8];
        unpack8(*reinterpret_cast<const uint4*>(dy + o * 8), f);
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (pb[i] == code) acc[i] += f[i];
      }
    }
    *reinterpret_cast<uint4*>(dx + t * 8) = pack8(acc);
  }
}

// Global average pooling: y[n, c] = mean_p x[n, p, c]; one thread owns eight channels of one image.
__global__ void __launch_bounds__(kThreads) avgpool_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                               __nv_bfloat16* __restrict__ y, int N, int P, int C) {
  const int CG = C >> 3;
  const int total = N * CG;
  for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < total; t += gridDim.x * blockDim.x) {
    const int g = t % CG, n = t / CG;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    const __nv_bfloat16* src = x + (long long)n * P * C + g * 8;
    for (int p = 0; p < P; ++p) {
      float f[8];
      unpack8(*reinterpret_cast<const uint4*>(src + (long long)p * C), f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += f[i];
    }
    const float inv = 1.f / float(P);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] *= inv;
    *reinterpret_cast<uint4*>(y + (long long)n * C + g * 8) = pack8(acc);
  }
}

// dx[n, p, c] = dy[n, c] / P
__global__ void __launch_bounds__(kThreads) avgpool_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                                               __nv_bfloat16* __restrict__ dx, int N, int P, int C) {
  const int CG = C >> 3;
  const long long total = (long long)N * P * CG;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const float inv = 1.f / float(P);
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
    const int g = (int)(t % CG);
    const int n = (int)(t / ((long long)CG * P));
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(dy + (long long)n * C + g * 8), f);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] *= inv;
    *reinterpret_cast<uint4*>(dx + t * 8) = pack8(f);
  }
}

int Grid(long long items) {
  long long b = (items + kThreads - 1) / kThreads;
  if (b < 1) b = 1;
  if (b > 148 * 8) b = 148 * 8;
  return (int)b;
}

}  // namespace

cudaError_t LaunchMaxPool3x3s2Forward(const void* x, void* y, void* idx, int N, int H, int W, int C, cudaStream_t stream) {
  if (C % 8 != 0 || N <= 0 || H <= 0 || W <= 0) return cudaErrorInvalidValue;
  const int Ho = (H + 2 - 3) / 2 + 1, Wo = (W + 2 - 3) / 2 + 1;
  maxpool_fwd_kernel<<<Grid((long long)N * Ho * Wo * (C / 8)), kThreads, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), static_cast<unsigned char*>(idx), N, H, W, C, Ho, Wo);
  CountKernelLaunch();
  return cudaGetLastError();
}

cudaError_t LaunchMaxPool3x3s2Backward(const void* dy, const void* idx, void* dx, int N, int H, int W, int C,
                                       cudaStream_t stream) {
  if (C % 8 != 0 || N <= 0 || H <= 0 || W <= 0) return cudaErrorInvalidValue;
  const int Ho = (H + 2 - 3) / 2 + 1, Wo = (W + 2 - 3) / 2 + 1;
  maxpool_bwd_kernel<<<Grid((long long)N * H * W * (C / 8)), kThreads, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const unsigned char*>(idx), static_cast<__nv_bfloat16*>(dx), N, H, W, C, Ho, Wo);
  CountKernelLaunch();
  return cudaGetLastError();
}

cudaError_t LaunchAvgPoolForward(const void* x, void* y, int N, int P, int C, cudaStream_t stream) {
  if (C % 8 != 0 || N <= 0 || P <= 0) return cudaErrorInvalidValue;
  avgpool_fwd_kernel<<<Grid((long long)N * (C / 8)), kThreads, 0, stream>>>(static_cast<const __nv_bfloat16*>(x),
                                                                          static_cast<__nv_bfloat16*>(y), N, P, C);
  CountKernelLaunch();
  return cudaGetLastError();
}

cudaError_t LaunchAvgPoolBackward(const void* dy, void* dx, int N, int P, int C, cudaStream_t stream) {
  if (C % 8 != 0 || N <= 0 || P <= 0) return cudaErrorInvalidValue;
  avgpool_bwd_kernel<<<Grid((long long)N * P * (C / 8)), kThreads, 0, stream>>>(static_cast<const __nv_bfloat16*>(dy),
                                                                              static_cast<__nv_bfloat16*>(dx), N, P, C);
  CountKernelLaunch();
  return cudaGetLastError();
}

}  // namespace bfb
