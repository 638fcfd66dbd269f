// Fused training-mode BatchNorm for NHWC bf16 activations:
//   forward : y = relu( gamma * (x - mean) * rstd + beta  [+ residual] )
//   backward: dz = dy * (y > 0)   (the forward pass leaves one bit per element for this);  dx = gamma*rstd * (dz - mean(dz) - xhat * mean(dz*xhat));
//             dresidual = dz;  dgamma = sum(dz*xhat);  dbeta = sum(dz)
// The activation is viewed as a [R, C] matrix (R = N*H*W rows, C contiguous).  Each pass is one
// streaming kernel with 16-byte loads: a statistics pass (per-channel sums in fp32, shifted by
// the first row to avoid cancellation) and an apply pass, for forward and for backward.  Fusing
// normalisation, ReLU and the residual add saves the separate elementwise passes, and the
// statistics kernels keep all SMs busy for every channel count of a ResNet (64..2048).
// The reference delegates these ops to PyTorch (examples/pytorch_benchmark.py:100).
#include "bn_kernels.h"

#include <cuda_bf16.h>

#include "comm_kernels.h"

namespace bfb {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxC = 2048;

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
__device__ __forceinline__ float load_param(const void* p, int i, int is_bf16) {
  return is_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]) : static_cast<const float*>(p)[i];
}
__device__ __forceinline__ void store_param(void* p, int i, int is_bf16, float v) {
  if (is_bf16) static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  else static_cast<float*>(p)[i] = v;
}

// Work decomposition of the two reduction kernels.  A block covers `cgb` groups of 8 channels
// (at most 32 groups = 512 contiguous bytes per row) times `rlb` = 256 / cgb rows per step;
// blockIdx.x selects the channel chunk, blockIdx.y the chunk of rows.  Every block adds its
// partial sums into the global accumulators once, so the number of global atomics is
// (#blocks x 2 x 8 x cgb) - small even for 2048 channels.
struct ReduceGeom {
  int cgb;      // channel groups per block
  int rlb;      // row lanes per block
};
__device__ __forceinline__ ReduceGeom reduce_geom(int C) {
  const int CG = C >> 3;
  ReduceGeom g;
  g.cgb = CG < 32 ? CG : 32;
  g.rlb = kThreads / g.cgb;
  return g;
}

// Adds the per-thread partials of one block into sums[c] and sums[C + c] (c = channels of this block).
__device__ __forceinline__ void flush_partials(const float* s1, const float* s2, int lg, int cgb, int c0, int C,
                                               float* sums) {
  __shared__ float sh[2 * 256];           // 32 groups x 8 channels, two statistics
  const int nch = cgb * 8;
  for (int c = threadIdx.x; c < 2 * nch; c += blockDim.x) sh[c] = 0.f;
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    atomicAdd(&sh[lg * 8 + i], s1[i]);
    atomicAdd(&sh[nch + lg * 8 + i], s2[i]);
  }
  __syncthreads();
  for (int c = threadIdx.x; c < nch; c += blockDim.x) {
    atomicAdd(&sums[c0 + c], sh[c]);
    atomicAdd(&sums[C + c0 + c], sh[nch + c]);
  }
}

// sums[c] = sum_r (x[r,c] - x[0,c]);  sums[C+c] = sum_r (x[r,c] - x[0,c])^2
__global__ void __launch_bounds__(kThreads) bn_stats_kernel(const __nv_bfloat16* __restrict__ x, long long R, int C,
                                                            float* __restrict__ sums) {
  const ReduceGeom geo = reduce_geom(C);
  const int lg = threadIdx.x % geo.cgb;                 // group inside the block
  const int rl = threadIdx.x / geo.cgb;
  const int g = blockIdx.x * geo.cgb + lg;              // global channel group
  const int RL = geo.rlb;
  float p[8], s1[8], s2[8];
  unpack8(*reinterpret_cast<const uint4*>(x + g * 8), p);
#pragma unroll
  for (int i = 0; i < 8; ++i) s1[i] = s2[i] = 0.f;
  const long long chunk = (R + gridDim.y - 1) / gridDim.y;
  const long long r0 = (long long)blockIdx.y * chunk;
  const long long r1 = r0 + chunk < R ? r0 + chunk : R;
  long long r = r0 + rl;
  for (; r + 7LL * RL < r1; r += 8LL * RL) {
    uint4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) v[u] = *reinterpret_cast<const uint4*>(x + (r + (long long)u * RL) * C + g * 8);
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      float f[8];
      unpack8(v[u], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float d = f[i] - p[i];
        s1[i] += d;
        s2[i] += d * d;
      }
    }
  }
  for (; r < r1; r += RL) {
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(x + r * C + g * 8), f);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float d = f[i] - p[i];
      s1[i] += d;
      s2[i] += d * d;
    }
  }
  flush_partials(s1, s2, lg, geo.cgb, blockIdx.x * geo.cgb * 8, C, sums);
}

struct BnApplyParams {
  const __nv_bfloat16* x;
  const __nv_bfloat16* residual;   // may be null
  __nv_bfloat16* y;
  unsigned char* mask;             // one bit per element (y > 0), 8 channels per byte; null without ReLU
  const float* sums;               // from bn_stats_kernel
  const void* gamma;
  const void* beta;
  float* running_mean;             // may be null
  float* running_var;
  float* save_mean;
  float* save_rstd;
  long long R;
  int C;
  int relu;
  int param_bf16;
  float eps;
  float momentum;
  int raw_sums;                    // sums are of x itself (a producer's epilogue wrote them), not of x - x[0]
};

__global__ void __launch_bounds__(kThreads) bn_apply_kernel(const BnApplyParams p) {
  const int CG = p.C >> 3;
  const long long gtid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int g = (int)(gtid % CG);
  float pivot[8], scale[8], shift[8];
  unpack8(*reinterpret_cast<const uint4*>(p.x + g * 8), pivot);
  if (p.raw_sums) {
#pragma unroll
    for (int i = 0; i < 8; ++i) pivot[i] = 0.f;
  }
  const float inv_r = 1.f / (float)p.R;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int c = g * 8 + i;
    const float m1 = p.sums[c] * inv_r;
    const float var = fmaxf(p.sums[p.C + c] * inv_r - m1 * m1, 0.f);
    const float mean = pivot[i] + m1;
    const float rstd = rsqrtf(var + p.eps);
    const float ga = load_param(p.gamma, c, p.param_bf16);
    const float be = load_param(p.beta, c, p.param_bf16);
    scale[i] = ga * rstd;
    shift[i] = be - mean * scale[i];
    if (gtid < CG) {
      p.save_mean[c] = mean;
      p.save_rstd[c] = rstd;
      if (p.running_mean != nullptr) {
        const float unbiased = p.R > 1 ? var * (float)p.R / (float)(p.R - 1) : var;
        p.running_mean[c] = (1.f - p.momentum) * p.running_mean[c] + p.momentum * mean;
        p.running_var[c] = (1.f - p.momentum) * p.running_var[c] + p.momentum * unbiased;
      }
    }
  }
  const long long total = p.R * CG;
  const long long stride = (long long)gridDim.x * blockDim.x;   // multiple of CG: g stays fixed
  constexpr int U = 4;
  for (long long base = gtid; base < total; base += stride * U) {
    uint4 vx[U], vr[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long idx = base + (long long)u * stride;
      if (idx < total) {
        vx[u] = *reinterpret_cast<const uint4*>(p.x + idx * 8);
        if (p.residual != nullptr) vr[u] = *reinterpret_cast<const uint4*>(p.residual + idx * 8);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long idx = base + (long long)u * stride;
      if (idx >= total) continue;
      float f[8];
      unpack8(vx[u], f);
      if (p.residual != nullptr) {
        float rr[8];
        unpack8(vr[u], rr);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = f[i] * scale[i] + shift[i] + rr[i];
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = f[i] * scale[i] + shift[i];
      }
      if (p.relu) {
        unsigned bits = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          bits |= (f[i] > 0.f ? 1u : 0u) << i;
          f[i] = fmaxf(f[i], 0.f);
        }
        p.mask[idx] = (unsigned char)bits;
      }
      *reinterpret_cast<uint4*>(p.y + idx * 8) = pack8(f);
    }
  }
}

// sums[c] = sum dz;  sums[C+c] = sum dz * xhat
__global__ void __launch_bounds__(kThreads, 3) bn_bwd_reduce_kernel(const __nv_bfloat16* __restrict__ dy,
                                                                    const unsigned char* __restrict__ mask,
                                                                    const __nv_bfloat16* __restrict__ x,
                                                                    const float* __restrict__ save_mean,
                                                                    const float* __restrict__ save_rstd, long long R,
                                                                    int C, int relu, float* __restrict__ sums) {
  const ReduceGeom geo = reduce_geom(C);
  const int lg = threadIdx.x % geo.cgb;
  const int rl = threadIdx.x / geo.cgb;
  const int g = blockIdx.x * geo.cgb + lg;
  const int RL = geo.rlb;
  float mean[8], rstd[8], s1[8], s2[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    mean[i] = save_mean[g * 8 + i];
    rstd[i] = save_rstd[g * 8 + i];
    s1[i] = s2[i] = 0.f;
  }
  const long long chunk = (R + gridDim.y - 1) / gridDim.y;
  const long long r0 = (long long)blockIdx.y * chunk;
  const long long r1 = r0 + chunk < R ? r0 + chunk : R;
  long long r = r0 + rl;
  constexpr int U = 4;
  const int CG = C >> 3;
  for (; r + (long long)(U - 1) * RL < r1; r += (long long)U * RL) {
    uint4 a[U], b[U];
    unsigned m[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long row = r + (long long)u * RL;
      const long long off = row * C + g * 8;
      a[u] = *reinterpret_cast<const uint4*>(dy + off);
      b[u] = *reinterpret_cast<const uint4*>(x + off);
      m[u] = relu ? mask[row * CG + g] : 0xffu;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float fd[8], fx[8];
      unpack8(a[u], fd);
      unpack8(b[u], fx);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float dz = ((m[u] >> i) & 1u) ? fd[i] : 0.f;
        s1[i] += dz;
        s2[i] += dz * (fx[i] - mean[i]) * rstd[i];
      }
    }
  }
  for (; r < r1; r += RL) {
    const long long off = r * C + g * 8;
    float fd[8], fx[8];
    unpack8(*reinterpret_cast<const uint4*>(dy + off), fd);
    unpack8(*reinterpret_cast<const uint4*>(x + off), fx);
    const unsigned m = relu ? mask[r * CG + g] : 0xffu;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float dz = ((m >> i) & 1u) ? fd[i] : 0.f;
      s1[i] += dz;
      s2[i] += dz * (fx[i] - mean[i]) * rstd[i];
    }
  }
  flush_partials(s1, s2, lg, geo.cgb, blockIdx.x * geo.cgb * 8, C, sums);
}

struct BnBwdApplyParams {
  const __nv_bfloat16* dy;
  const unsigned char* mask;       // bits written by the forward pass (null without ReLU)
  const __nv_bfloat16* x;
  __nv_bfloat16* dx;
  __nv_bfloat16* dres;             // may be null
  const float* sums;               // from bn_bwd_reduce_kernel
  const float* save_mean;
  const float* save_rstd;
  const void* gamma;
  void* dgamma;
  void* dbeta;
  long long R;
  int C;
  int relu;
  int param_bf16;
};

__global__ void __launch_bounds__(kThreads) bn_bwd_apply_kernel(const BnBwdApplyParams p) {
  const int CG = p.C >> 3;
  const long long gtid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int g = (int)(gtid % CG);
  const float inv_r = 1.f / (float)p.R;
  float mean[8], rstd[8], k0[8], k1[8], k2[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int c = g * 8 + i;
    mean[i] = p.save_mean[c];
    rstd[i] = p.save_rstd[c];
    const float ga = load_param(p.gamma, c, p.param_bf16);
    const float s1 = p.sums[c], s2 = p.sums[p.C + c];
    k0[i] = ga * rstd[i];            // dx = k0 * (dz - k1 - xhat * k2)
    k1[i] = s1 * inv_r;
    k2[i] = s2 * inv_r;
    if (gtid < CG) {
      store_param(p.dgamma, c, p.param_bf16, s2);
      store_param(p.dbeta, c, p.param_bf16, s1);
    }
  }
  const long long total = p.R * CG;
  const long long stride = (long long)gridDim.x * blockDim.x;
  constexpr int U = 4;
  for (long long base = gtid; base < total; base += stride * U) {
    uint4 vd[U], vx[U];
    unsigned m[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long idx = base + (long long)u * stride;
      if (idx < total) {
        vd[u] = *reinterpret_cast<const uint4*>(p.dy + idx * 8);
        vx[u] = *reinterpret_cast<const uint4*>(p.x + idx * 8);
        m[u] = p.relu ? p.mask[idx] : 0xffu;
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long idx = base + (long long)u * stride;
      if (idx >= total) continue;
      float fd[8], fx[8], o[8];
      unpack8(vd[u], fd);
      unpack8(vx[u], fx);
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (!((m[u] >> i) & 1u)) fd[i] = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = k0[i] * (fd[i] - k1[i] - (fx[i] - mean[i]) * rstd[i] * k2[i]);
      *reinterpret_cast<uint4*>(p.dx + idx * 8) = pack8(o);
      if (p.dres != nullptr) *reinterpret_cast<uint4*>(p.dres + idx * 8) = pack8(fd);
    }
  }
}

dim3 ReduceGrid(long long R, int C) {
  const int CG = C >> 3;
  const int cgb = CG < 32 ? CG : 32;
  const int rlb = kThreads / cgb;
  const int cchunks = CG / cgb;
  long long rows = (R + (long long)rlb * 16 - 1) / ((long long)rlb * 16);   // >= 16 rows per thread
  long long cap = (148 * 4) / cchunks;
  if (cap < 1) cap = 1;
  if (rows > cap) rows = cap;
  if (rows < 1) rows = 1;
  return dim3(static_cast<unsigned>(cchunks), static_cast<unsigned>(rows));
}
int ApplyGrid(long long R, int C) {
  long long blocks = (R * (C >> 3) + kThreads * 4 - 1) / (kThreads * 4);
  if (blocks < 1) blocks = 1;
  if (blocks > 148 * 6) blocks = 148 * 6;
  return (int)blocks;
}

}  // namespace

bool BnShapeSupported(long long R, int C) {
  const int CG = C >> 3;
  return R > 0 && C >= 8 && C <= kMaxC && (C % 8) == 0 && (kThreads % CG) == 0;
}

cudaError_t LaunchBnForward(const void* x, const void* residual, void* y, void* mask, float* sums, const void* gamma, const void* beta,
                            float* running_mean, float* running_var, float* save_mean, float* save_rstd, long long R,
                            int C, float eps, float momentum, int relu, int param_bf16, cudaStream_t stream,
                            int stats_ready) {
  if (!BnShapeSupported(R, C) || (relu && mask == nullptr)) return cudaErrorInvalidValue;
  if (!stats_ready) {
    bn_stats_kernel<<<ReduceGrid(R, C), kThreads, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), R, C, sums);
    CountKernelLaunch();
  }
  BnApplyParams p{static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(residual),
                  static_cast<__nv_bfloat16*>(y), static_cast<unsigned char*>(mask), sums, gamma, beta, running_mean,
                  running_var, save_mean, save_rstd,
                  R, C, relu, param_bf16, eps, momentum, stats_ready};
  bn_apply_kernel<<<ApplyGrid(R, C), kThreads, 0, stream>>>(p);
  CountKernelLaunch();
  return cudaGetLastError();
}

cudaError_t LaunchBnBackward(const void* dy, const void* mask, const void* x, void* dx, void* dres, float* sums,
                             const float* save_mean, const float* save_rstd, const void* gamma, void* dgamma,
                             void* dbeta, long long R, int C, int relu, int param_bf16, cudaStream_t stream) {
  if (!BnShapeSupported(R, C) || (relu && mask == nullptr)) return cudaErrorInvalidValue;
  bn_bwd_reduce_kernel<<<ReduceGrid(R, C), kThreads, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const unsigned char*>(mask), static_cast<const __nv_bfloat16*>(x),
      save_mean, save_rstd, R, C, relu, sums);
  CountKernelLaunch();
  BnBwdApplyParams p{static_cast<const __nv_bfloat16*>(dy), static_cast<const unsigned char*>(mask),
                     static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(dx),
                     static_cast<__nv_bfloat16*>(dres), sums, save_mean, save_rstd, gamma, dgamma, dbeta, R, C, relu,
                     param_bf16};
  bn_bwd_apply_kernel<<<ApplyGrid(R, C), kThreads, 0, stream>>>(p);
  CountKernelLaunch();
  return cudaGetLastError();
}

}  // namespace bfb
