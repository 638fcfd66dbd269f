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

#include <cstdlib>

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
// dy may arrive as two addends (the gradient through a block's shortcut and the gradient through its first
// convolution): the sum is formed here, in fp32, instead of in a pass of its own.
__device__ __forceinline__ void unpack8_sum(const uint4& a, const __nv_bfloat16* second, long long off, float* f) {
  unpack8(a, f);
  if (second != nullptr) {
    float g[8];
    unpack8(*reinterpret_cast<const uint4*>(second + off), g);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] += g[i];
  }
}
__device__ __forceinline__ void unpack8_add(const uint4& a, const uint4& b, bool second, float* f) {
  unpack8(a, f);
  if (second) {
    float g[8];
    unpack8(b, g);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] += g[i];
  }
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

// Adds the per-thread partials of one block into sums[c] and sums[C + c] (c = channels of this block): every thread
// parks its 16 values in shared memory, thread c adds up column c over the row lanes and issues one global atomic
// (shared-memory fp32 atomics are compare-and-swap loops and crawl when many warps add to the same words).
__device__ __forceinline__ void flush_partials(const float* s1, const float* s2, int lg, int cgb, int c0, int C,
                                               float* sums) {
  __shared__ float sh[kThreads * 16];
  const int nch = cgb * 8;
  const int rl = threadIdx.x / cgb, RL = kThreads / cgb;
  float* row = sh + size_t(rl) * 2 * nch;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    row[lg * 8 + i] = s1[i];
    row[nch + lg * 8 + i] = s2[i];
  }
  __syncthreads();
  for (int c = threadIdx.x; c < 2 * nch; c += blockDim.x) {
    float t = 0.f;
    for (int r = 0; r < RL; ++r) t += sh[size_t(r) * 2 * nch + c];
    atomicAdd(&sums[c < nch ? c0 + c : C + c0 + (c - nch)], t);
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
__global__ void __launch_bounds__(kThreads, 2) bn_bwd_reduce_kernel(const __nv_bfloat16* __restrict__ dy,
                                                                    const __nv_bfloat16* __restrict__ dy2,
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
    uint4 a[U], a2[U], b[U];
    unsigned m[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long row = r + (long long)u * RL;
      const long long off = row * C + g * 8;
      a[u] = *reinterpret_cast<const uint4*>(dy + off);
      if (dy2 != nullptr) a2[u] = *reinterpret_cast<const uint4*>(dy2 + off);
      b[u] = *reinterpret_cast<const uint4*>(x + off);
      m[u] = relu ? mask[row * CG + g] : 0xffu;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float fd[8], fx[8];
      unpack8_add(a[u], a2[u], dy2 != nullptr, fd);
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
    unpack8_sum(*reinterpret_cast<const uint4*>(dy + off), dy2, off, fd);
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
  const __nv_bfloat16* dy2;        // second addend of the incoming gradient, or null
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
    uint4 vd[U], vd2[U], vx[U];
    unsigned m[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long idx = base + (long long)u * stride;
      if (idx < total) {
        vd[u] = *reinterpret_cast<const uint4*>(p.dy + idx * 8);
        if (p.dy2 != nullptr) vd2[u] = *reinterpret_cast<const uint4*>(p.dy2 + idx * 8);
        vx[u] = *reinterpret_cast<const uint4*>(p.x + idx * 8);
        m[u] = p.relu ? p.mask[idx] : 0xffu;
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long idx = base + (long long)u * stride;
      if (idx >= total) continue;
      float fd[8], fx[8], o[8];
      unpack8_add(vd[u], vd2[u], p.dy2 != nullptr, fd);
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

// ------------------------------------------------------------------------------------------------------ //
// One-launch variants for activations that fit on the chip.
//
// Most BatchNorm layers of a ResNet see a few MB: two dependent kernels per pass then cost mostly their launch
// and a handful of dependent memory round trips each (14 us per pass for a 3 MB tensor, against 1.5 us of
// traffic).  These kernels do the whole pass in one cooperative launch with one block per SM: phase 1 reads the
// block's rows once, keeps them in shared memory and adds the block's partial sums to the global accumulators;
// after a grid-wide barrier phase 2 normalises the rows out of shared memory.  The activation is read once
// instead of twice and nothing waits for a second launch.  The barrier is a counter in the zeroed workspace
// (one word after the 2*C sums); its wait is bounded and ends in the caller's status word.
// ------------------------------------------------------------------------------------------------------ //
constexpr int kFusedThreads = 512;
constexpr size_t kFusedStageLimit = 176 * 1024;     // dynamic shared memory for staged rows, per block
constexpr unsigned long long kBarrierLimitNs = 2000000000ull;

__device__ __forceinline__ unsigned long long bn_now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// All blocks of a cooperative grid meet here once.  Returns false (in every thread of the block) when the wait
// ran out; the caller then leaves without touching its outputs.
__device__ __forceinline__ bool grid_barrier_once(unsigned int* counter, unsigned int* status) {
  __shared__ int ok_s;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    atomicAdd(counter, 1u);
    bool ok = true;
    const unsigned long long t0 = bn_now_ns();
    unsigned spins = 0;
    for (;;) {
      unsigned v;
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
      if (v >= gridDim.x) break;
      if ((++spins & 63u) == 0 && bn_now_ns() - t0 > kBarrierLimitNs) { ok = false; break; }
    }
    if (!ok && status != nullptr) atomicExch(status, 1u);
    ok_s = ok ? 1 : 0;
  }
  __syncthreads();
  return ok_s != 0;
}

// Work decomposition of the one-launch kernels: like the reduction kernels, a block covers a chunk of at most 256
// channels (cgb groups of 8) and a chunk of rows; blockIdx.x = row chunk * channel chunks + channel chunk.
struct FusedGeom {
  int cgb, nch, cc, rc, nrc, lg, rl, RL, g;
  long long r0, r1, chunk;
};
__device__ __forceinline__ FusedGeom fused_geom(long long R, int C) {
  FusedGeom f;
  const int CG = C >> 3;
  f.cgb = CG < 32 ? CG : 32;
  f.nch = CG / f.cgb;
  f.cc = blockIdx.x % f.nch;
  f.rc = blockIdx.x / f.nch;
  f.nrc = gridDim.x / f.nch;
  f.lg = threadIdx.x % f.cgb;
  f.rl = threadIdx.x / f.cgb;
  f.RL = kFusedThreads / f.cgb;
  f.g = f.cc * f.cgb + f.lg;
  f.chunk = (R + f.nrc - 1) / f.nrc;
  f.r0 = (long long)f.rc * f.chunk;
  f.r1 = f.r0 + f.chunk < R ? f.r0 + f.chunk : R;
  return f;
}

// Adds the per-thread partials of a block into one copy of the accumulators.  Every thread parks its 16 partial
// sums in shared memory (row lane x channel: kFusedThreads * 16 floats), then thread c adds up column c and issues
// one global atomic: no shared-memory atomics, whose fp32 form is a compare-and-swap loop that crawls when sixteen
// warps add to the same words.  Row chunks spread their additions over `copies` sets of accumulators, because
// same-address atomics serialise in L2.
__device__ __forceinline__ void flush_partials_all(const float* s1, const float* s2, const FusedGeom& f, int C, float* sh,
                                                   float* sums, int copies) {
  const int nchn = f.cgb * 8;
  float* row = sh + size_t(f.rl) * 2 * nchn;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    row[f.lg * 8 + i] = s1[i];
    row[nchn + f.lg * 8 + i] = s2[i];
  }
  __syncthreads();
  float* mine = sums + size_t(f.rc % copies) * 2 * C + f.cc * nchn;
  for (int c = threadIdx.x; c < 2 * nchn; c += blockDim.x) {
    float t = 0.f;
    for (int r = 0; r < f.RL; ++r) t += sh[size_t(r) * 2 * nchn + c];
    atomicAdd(&mine[c < nchn ? c : C + (c - nchn)], t);
  }
}

// After the barrier: totals of the block's channels over all copies into shared memory (sh[c] and sh[nchn + c]),
// once per block, instead of all threads of the grid reading the same few lines of L2.
__device__ __forceinline__ void gather_totals(const float* sums, const FusedGeom& f, int C, int copies, float* sh) {
  __syncthreads();           // the partial sums parked in sh have been consumed by every thread
  const int nchn = f.cgb * 8;
  for (int c = threadIdx.x; c < 2 * nchn; c += blockDim.x) {
    const int at = f.cc * nchn + (c < nchn ? c : C + (c - nchn));
    float t = 0.f;
    for (int k = 0; k < copies; ++k) t += __ldcg(&sums[size_t(k) * 2 * C + at]);
    sh[c] = t;
  }
  __syncthreads();
}

#ifdef BN_TRACE
__device__ unsigned long long g_bn_trace[160][8];
#define BTRACE(i) do { if (threadIdx.x == 0) g_bn_trace[blockIdx.x][i] = bn_now_ns(); } while (0)
#else
#define BTRACE(i) do {} while (0)
#endif

__global__ void __launch_bounds__(kFusedThreads, 1) bn_fwd_fused_kernel(const BnApplyParams p, float* __restrict__ sums,
                                                                       unsigned int* barrier, unsigned int* status,
                                                                       int copies) {
  extern __shared__ uint4 staged[];
  __shared__ float sh[kFusedThreads * 16];       // partial sums of every thread, later the totals (2*C values)
  const int C = p.C, CG = C >> 3;
  const FusedGeom f = fused_geom(p.R, C);
  const int g = f.g, rl = f.rl, RL = f.RL, cgb = f.cgb, lg = f.lg;
  const long long r0 = f.r0, r1 = f.r1;
  float pivot[8], s1[8], s2[8], ga[8], be[8];
  BTRACE(0);
  unpack8(*reinterpret_cast<const uint4*>(p.x + g * 8), pivot);
#pragma unroll
  for (int i = 0; i < 8; ++i) {                  // needed after the barrier only: fetched while the rows stream in
    ga[i] = load_param(p.gamma, g * 8 + i, p.param_bf16);
    be[i] = load_param(p.beta, g * 8 + i, p.param_bf16);
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) s1[i] = s2[i] = 0.f;
  constexpr int U = 4;
  for (long long r = r0 + rl; r < r1; r += (long long)U * RL) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long row = r + (long long)u * RL;
      if (row < r1) v[u] = *reinterpret_cast<const uint4*>(p.x + row * C + g * 8);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long row = r + (long long)u * RL;
      if (row >= r1) continue;
      staged[(row - r0) * cgb + lg] = v[u];
      float f[8];
      unpack8(v[u], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float d = f[i] - pivot[i];
        s1[i] += d;
        s2[i] += d * d;
      }
    }
  }
  BTRACE(1);
  flush_partials_all(s1, s2, f, C, sh, sums, copies);
  BTRACE(2);
  if (!grid_barrier_once(barrier, status)) return;
  BTRACE(3);
  gather_totals(sums, f, C, copies, sh);

  float scale[8], shift[8];
  const float inv_r = 1.f / (float)p.R;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int c = g * 8 + i;
    const float m1 = sh[lg * 8 + i] * inv_r;
    const float var = fmaxf(sh[cgb * 8 + lg * 8 + i] * inv_r - m1 * m1, 0.f);
    const float mean = pivot[i] + m1;
    const float rstd = rsqrtf(var + p.eps);
    scale[i] = ga[i] * rstd;
    shift[i] = be[i] - mean * scale[i];
    if (f.rc == 0 && rl == 0) {
      p.save_mean[c] = mean;
      p.save_rstd[c] = rstd;
      if (p.running_mean != nullptr) {
        const float unbiased = p.R > 1 ? var * (float)p.R / (float)(p.R - 1) : var;
        p.running_mean[c] = (1.f - p.momentum) * p.running_mean[c] + p.momentum * mean;
        p.running_var[c] = (1.f - p.momentum) * p.running_var[c] + p.momentum * unbiased;
      }
    }
  }
  BTRACE(4);
  for (long long r = r0 + rl; r < r1; r += (long long)U * RL) {
    uint4 vr[U];
    if (p.residual != nullptr) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long row = r + (long long)u * RL;
        if (row < r1) vr[u] = *reinterpret_cast<const uint4*>(p.residual + row * C + g * 8);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long row = r + (long long)u * RL;
      if (row >= r1) continue;
      const long long idx = row * CG + g;
      float f[8];
      unpack8(staged[(row - r0) * cgb + lg], f);
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
  BTRACE(5);
}

// Backward in one launch: phase 1 reads dy, x and the ReLU bits once, keeps x (and, when it fits, the masked
// gradient dz) in shared memory and reduces sum(dz), sum(dz * xhat); phase 2 writes dx (and dresidual).
__global__ void __launch_bounds__(kFusedThreads, 1) bn_bwd_fused_kernel(const BnBwdApplyParams p, float* __restrict__ sums,
                                                                       unsigned int* barrier, unsigned int* status,
                                                                       int stage_dz, int copies) {
  extern __shared__ uint4 staged[];
  __shared__ float sh[kFusedThreads * 16];
  const int C = p.C, CG = C >> 3;
  const FusedGeom f = fused_geom(p.R, C);
  const int g = f.g, rl = f.rl, RL = f.RL, cgb = f.cgb, lg = f.lg;
  const long long r0 = f.r0, r1 = f.r1;
  uint4* staged_dz = staged + f.chunk * cgb;
  float mean[8], rstd[8], s1[8], s2[8], ga[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    mean[i] = p.save_mean[g * 8 + i];
    rstd[i] = p.save_rstd[g * 8 + i];
    ga[i] = load_param(p.gamma, g * 8 + i, p.param_bf16);
    s1[i] = s2[i] = 0.f;
  }
  constexpr int U = 4;
  for (long long r = r0 + rl; r < r1; r += (long long)U * RL) {
    uint4 a[U], a2[U], b[U];
    unsigned m[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long row = r + (long long)u * RL;
      if (row < r1) {
        const long long off = row * C + g * 8;
        a[u] = *reinterpret_cast<const uint4*>(p.dy + off);
        if (p.dy2 != nullptr) a2[u] = *reinterpret_cast<const uint4*>(p.dy2 + off);
        b[u] = *reinterpret_cast<const uint4*>(p.x + off);
        m[u] = p.relu ? p.mask[row * CG + g] : 0xffu;
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long row = r + (long long)u * RL;
      if (row >= r1) continue;
      float fd[8], fx[8];
      unpack8_add(a[u], a2[u], p.dy2 != nullptr, fd);
      unpack8(b[u], fx);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (!((m[u] >> i) & 1u)) fd[i] = 0.f;
        s1[i] += fd[i];
        s2[i] += fd[i] * (fx[i] - mean[i]) * rstd[i];
      }
      staged[(row - r0) * cgb + lg] = b[u];
      if (stage_dz) staged_dz[(row - r0) * cgb + lg] = pack8(fd);
    }
  }
  flush_partials_all(s1, s2, f, C, sh, sums, copies);
  if (!grid_barrier_once(barrier, status)) return;
  gather_totals(sums, f, C, copies, sh);

  const float inv_r = 1.f / (float)p.R;
  float k0[8], k1[8], k2[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int c = g * 8 + i;
    const float t1 = sh[lg * 8 + i], t2 = sh[cgb * 8 + lg * 8 + i];
    k0[i] = ga[i] * rstd[i];         // dx = k0 * (dz - k1 - xhat * k2)
    k1[i] = t1 * inv_r;
    k2[i] = t2 * inv_r;
    if (f.rc == 0 && rl == 0) {
      store_param(p.dgamma, c, p.param_bf16, t2);
      store_param(p.dbeta, c, p.param_bf16, t1);
    }
  }
  for (long long r = r0 + rl; r < r1; r += (long long)U * RL) {
    uint4 a[U], a2[U];
    unsigned m[U];
    if (!stage_dz) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long row = r + (long long)u * RL;
        if (row < r1) {
          a[u] = *reinterpret_cast<const uint4*>(p.dy + row * C + g * 8);
          if (p.dy2 != nullptr) a2[u] = *reinterpret_cast<const uint4*>(p.dy2 + row * C + g * 8);
          m[u] = p.relu ? p.mask[row * CG + g] : 0xffu;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long row = r + (long long)u * RL;
      if (row >= r1) continue;
      const long long idx = row * CG + g;
      float fd[8], fx[8], o[8];
      unpack8(staged[(row - r0) * cgb + lg], fx);
      if (stage_dz) {
        unpack8(staged_dz[(row - r0) * cgb + lg], fd);
      } else {
        unpack8_add(a[u], a2[u], p.dy2 != nullptr, fd);
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (!((m[u] >> i) & 1u)) fd[i] = 0.f;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = k0[i] * (fd[i] - k1[i] - (fx[i] - mean[i]) * rstd[i] * k2[i]);
      *reinterpret_cast<uint4*>(p.dx + idx * 8) = pack8(o);
      if (p.dres != nullptr) *reinterpret_cast<uint4*>(p.dres + idx * 8) = pack8(fd);
    }
  }
}

int FusedGrid() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0, coop = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (!coop || sms <= 0) sms = -1;
    static const bool off = [] { const char* e = std::getenv("BLUEFOG_B200_BN_FUSED"); return e != nullptr && e[0] == '0'; }();
    if (off) sms = -1;
  }
  return sms;
}

// Blocks of the one-launch form: every SM for activations of 7 MB and more, fewer for smaller ones (about 48 KB
// of rows per block), because what a small pass costs is the barrier and the contention on the accumulators.  The
// count is a multiple of the number of channel chunks (256 channels each).
int FusedBlocks(long long R, int C, int sms) {
  if (sms <= 0) return 0;
  const int CG = C >> 3;
  const int nch = CG <= 32 ? 1 : CG / 32;
  long long blocks = (R * C * 2 + 48 * 1024 - 1) / (48 * 1024);
  if (blocks < 8) blocks = 8;
  if (blocks > sms) blocks = sms;
  long long nrc = blocks / nch;
  if (nrc < 1) nrc = 1;
  return nrc * nch <= sms ? static_cast<int>(nrc * nch) : 0;
}

// Shared memory one block needs to keep `tensors` copies of its rows; 0 when the one-launch form does not apply.
size_t FusedStageBytes(long long R, int C, int tensors, int grid) {
  const int CG = C >> 3;
  if (grid <= 0 || CG < 1 || (CG < 32 ? (kFusedThreads % CG) != 0 : (CG % 32) != 0)) return 0;
  const int cgb = CG < 32 ? CG : 32;
  const int nrc = grid / (CG / cgb);
  if (nrc < 1) return 0;
  const long long chunk = (R + nrc - 1) / nrc;
  const size_t bytes = size_t(chunk) * cgb * 16 * tensors;
  return bytes <= kFusedStageLimit ? bytes : 0;
}

template <typename K>
cudaError_t LaunchCooperative(K kernel, int grid, size_t smem, void** args, cudaStream_t stream, size_t* attr_bytes) {
  if (smem > *attr_bytes) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kFusedStageLimit));
    if (e != cudaSuccess) return e;
    *attr_bytes = kFusedStageLimit;
  }
  return cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kernel), dim3(grid), dim3(kFusedThreads), args, smem, stream);
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

int BnSumCopies(int C) {
  // row chunks per channel chunk of a full grid: about 148 * 256 / C; eight copies bring the contention per word
  // below twenty for up to 256 channels, wider layers need fewer
  int k = 2048 / C;
  return k < 1 ? 1 : (k > 8 ? 8 : k);
}

bool BnShapeSupported(long long R, int C) {
  const int CG = C >> 3;
  return R > 0 && C >= 8 && C <= kMaxC && (C % 8) == 0 && (kThreads % CG) == 0;
}

cudaError_t LaunchBnForward(const void* x, const void* residual, void* y, void* mask, float* sums, const void* gamma, const void* beta,
                            float* running_mean, float* running_var, float* save_mean, float* save_rstd, long long R,
                            int C, float eps, float momentum, int relu, int param_bf16, cudaStream_t stream,
                            int stats_ready, int sum_copies, unsigned int* status) {
  if (!BnShapeSupported(R, C) || (relu && mask == nullptr)) return cudaErrorInvalidValue;
  BnApplyParams p{static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(residual),
                  static_cast<__nv_bfloat16*>(y), static_cast<unsigned char*>(mask), sums, gamma, beta, running_mean,
                  running_var, save_mean, save_rstd,
                  R, C, relu, param_bf16, eps, momentum, stats_ready};
  if (!stats_ready && sum_copies >= 1) {
    const int grid = FusedBlocks(R, C, FusedGrid());
    const size_t smem = FusedStageBytes(R, C, 1, grid);
    if (smem != 0) {
      static size_t attr_bytes = 0;
      unsigned int* barrier = reinterpret_cast<unsigned int*>(sums + size_t(sum_copies) * 2 * C);
      void* args[] = {&p, &sums, &barrier, &status, &sum_copies};
      cudaError_t e = LaunchCooperative(bn_fwd_fused_kernel, grid, smem, args, stream, &attr_bytes);
      CountKernelLaunch();
      return e != cudaSuccess ? e : cudaGetLastError();
    }
  }
  if (!stats_ready) {
    bn_stats_kernel<<<ReduceGrid(R, C), kThreads, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), R, C, sums);
    CountKernelLaunch();
  }
  bn_apply_kernel<<<ApplyGrid(R, C), kThreads, 0, stream>>>(p);
  CountKernelLaunch();
  return cudaGetLastError();
}

cudaError_t LaunchBnBackward(const void* dy, const void* dy2, const void* mask, const void* x, void* dx, void* dres, float* sums,
                             const float* save_mean, const float* save_rstd, const void* gamma, void* dgamma,
                             void* dbeta, long long R, int C, int relu, int param_bf16, cudaStream_t stream,
                             int sum_copies, unsigned int* status) {
  if (!BnShapeSupported(R, C) || (relu && mask == nullptr)) return cudaErrorInvalidValue;
  BnBwdApplyParams p{static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(dy2),
                     static_cast<const unsigned char*>(mask),
                     static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(dx),
                     static_cast<__nv_bfloat16*>(dres), sums, save_mean, save_rstd, gamma, dgamma, dbeta, R, C, relu,
                     param_bf16};
  if (sum_copies >= 1) {
    const int grid = FusedBlocks(R, C, FusedGrid());
    unsigned int* barrier = reinterpret_cast<unsigned int*>(sums + size_t(sum_copies) * 2 * C);
    int stage_dz = 1;
    size_t smem = FusedStageBytes(R, C, 2, grid);
    if (smem == 0) {
      stage_dz = 0;                      // x stays on the chip, dy and the bits are read again (out of L2)
      smem = FusedStageBytes(R, C, 1, grid);
    }
    if (smem != 0) {
      static size_t attr_bytes = 0;
      void* args[] = {&p, &sums, &barrier, &status, &stage_dz, &sum_copies};
      cudaError_t e = LaunchCooperative(bn_bwd_fused_kernel, grid, smem, args, stream, &attr_bytes);
      CountKernelLaunch();
      return e != cudaSuccess ? e : cudaGetLastError();
    }
  }
  bn_bwd_reduce_kernel<<<ReduceGrid(R, C), kThreads, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(dy2), static_cast<const unsigned char*>(mask),
      static_cast<const __nv_bfloat16*>(x),
      save_mean, save_rstd, R, C, relu, sums);
  CountKernelLaunch();
  bn_bwd_apply_kernel<<<ApplyGrid(R, C), kThreads, 0, stream>>>(p);
  CountKernelLaunch();
  return cudaGetLastError();
}

}  // namespace bfb
