// Mean cross-entropy over the rows of a bf16 logits matrix [R, C], forward and backward, with fp32 arithmetic and
// no fp32 copy of the logits:
//
//   forward:  lse_r = log sum_c exp(x[r, c]);  loss = (1/R) sum_r (lse_r - x[r, target_r])      (one read of x)
//   backward: dx[r, c] = (exp(x[r, c] - lse_r) - [c == target_r]) * g / R                         (read x, write dx)
//
// One block owns one row; every thread runs an online (max, sum-of-exponentials) recurrence over its 16-byte
// vectors, the block folds the pairs, and the row's loss is added to the scalar sum with one atomic.  Columns
// holding -inf (the padding of a classifier whose vocabulary was rounded up) contribute exp(-inf) = 0 and get a
// zero gradient.  The reference has no loss kernels; GPT-2's 8192 x 50304 logits are the case this is for.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "ce_kernels.h"
#include "comm_kernels.h"

namespace bfb {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

// (m, s) represents s * exp(m); combining keeps the larger maximum
__device__ __forceinline__ void combine(float& m, float& s, float m2, float s2) {
  if (m2 > m) {
    s = s * __expf(m - m2) + s2;
    m = m2;
  } else if (m2 > -CUDART_INF_F) {
    s += s2 * __expf(m2 - m);
  }
}

__global__ void __launch_bounds__(kThreads) ce_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                          const long long* __restrict__ target, float* __restrict__ lse,
                                                          float* __restrict__ loss_sum, int C, float inv_rows) {
  __shared__ float sm[kThreads / 32], ss[kThreads / 32];
  const long long r = blockIdx.x;
  const __nv_bfloat16* xr = x + r * C;
  const int CG = C >> 3;
  float m = -CUDART_INF_F, s = 0.f;
  for (int g = threadIdx.x; g < CG; g += kThreads) {
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(xr + g * 8), f);
    float vm = f[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) vm = fmaxf(vm, f[i]);
    if (vm > -CUDART_INF_F) {
      float vs = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) vs += __expf(f[i] - vm);
      combine(m, s, vm, vs);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
    combine(m, s, m2, s2);
  }
  if ((threadIdx.x & 31) == 0) {
    sm[threadIdx.x >> 5] = m;
    ss[threadIdx.x >> 5] = s;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < kThreads / 32; ++w) combine(m, s, sm[w], ss[w]);
    const float l = m + logf(s);
    lse[r] = l;
    const float xt = __bfloat162float(xr[target[r]]);
    atomicAdd(loss_sum, (l - xt) * inv_rows);
  }
}

__global__ void __launch_bounds__(kThreads) ce_bwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                          const long long* __restrict__ target,
                                                          const float* __restrict__ lse, const float* __restrict__ grad_out,
                                                          __nv_bfloat16* __restrict__ dx, int C, float inv_rows) {
  const long long r = blockIdx.x;
  const __nv_bfloat16* xr = x + r * C;
  __nv_bfloat16* dr = dx + r * C;
  const float l = lse[r];
  const float scale = grad_out[0] * inv_rows;
  const int t = (int)target[r];
  const int CG = C >> 3;
  for (int g = threadIdx.x; g < CG; g += kThreads) {
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(xr + g * 8), f);
    uint4 out;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float p = __expf(f[i] - l);
      f[i] = (p - ((g * 8 + i) == t ? 1.f : 0.f)) * scale;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    *reinterpret_cast<uint4*>(dr + g * 8) = out;
  }
}

}  // namespace

cudaError_t LaunchCrossEntropyForward(const void* x, const long long* target, float* lse, float* loss_sum_zeroed,
                                      long long R, int C, cudaStream_t stream) {
  if (R <= 0 || R > 0x7fffffffLL || C < 8 || (C % 8) != 0) return cudaErrorInvalidValue;
  ce_fwd_kernel<<<static_cast<unsigned>(R), kThreads, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), target, lse,
                                                                    loss_sum_zeroed, C, 1.f / (float)R);
  CountKernelLaunch();
  return cudaGetLastError();
}

cudaError_t LaunchCrossEntropyBackward(const void* x, const long long* target, const float* lse, const float* grad_out,
                                       void* dx, long long R, int C, cudaStream_t stream) {
  if (R <= 0 || R > 0x7fffffffLL || C < 8 || (C % 8) != 0) return cudaErrorInvalidValue;
  ce_bwd_kernel<<<static_cast<unsigned>(R), kThreads, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), target, lse, grad_out,
                                                                    static_cast<__nv_bfloat16*>(dx), C, 1.f / (float)R);
  CountKernelLaunch();
  return cudaGetLastError();
}

}  // namespace bfb
