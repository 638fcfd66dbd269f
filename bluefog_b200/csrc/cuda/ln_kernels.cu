// LayerNorm over the last dimension of a bf16 [R, C] matrix, forward and backward.
//
//   forward:  y = (x - mean_r) * rstd_r * gamma + beta          (statistics in fp32, saved per row)
//   backward: g = dy * gamma;  dx = rstd_r * (g - mean_c(g) - xhat * mean_c(g * xhat))
//             dgamma = sum_r dy * xhat;  dbeta = sum_r dy
//
// One warp owns one row at a time and keeps the whole row in registers (C <= 2048: at most eight
// 16-byte vectors per lane), so x is read once in the forward pass and x, dy once in the backward
// pass.  The column sums of the backward pass stay in registers while a warp walks over its rows
// and are folded through shared memory into fp32 atomics once per block.
//
// The reference ships no normalisation kernels (its examples call torch.nn layers); this is the
// LayerNorm of the GPT-2 model of this library.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "comm_kernels.h"
#include "ln_kernels.h"

#include <cstdlib>

namespace bfb {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kMaxC = 2048;

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 v;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ void load_param8(const void* p, int c0, int is_bf16, float* f) {
  if (is_bf16) {
    unpack8(*reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p) + c0), f);
  } else {
    const float4 a = *reinterpret_cast<const float4*>(static_cast<const float*>(p) + c0);
    const float4 b = *reinterpret_cast<const float4*>(static_cast<const float*>(p) + c0 + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
    f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
}

template <int NV>
__global__ void __launch_bounds__(kThreads) ln_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                          const void* __restrict__ gamma,
                                                          const void* __restrict__ beta,
                                                          __nv_bfloat16* __restrict__ y, float* __restrict__ mean_out,
                                                          float* __restrict__ rstd_out, long long R, int C, float eps,
                                                          int param_bf16) {
  const int lane = threadIdx.x & 31;
  const int CG = C >> 3;
  const long long warp0 = (long long)blockIdx.x * kWarps + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * kWarps;
  const float inv_c = 1.f / (float)C;
  for (long long r = warp0; r < R; r += nwarps) {
    const __nv_bfloat16* xr = x + r * C;
    float f[NV][8];
    float s = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int g = lane + 32 * v;
      if (g < CG) {
        unpack8(*reinterpret_cast<const uint4*>(xr + g * 8), f[v]);
#pragma unroll
        for (int i = 0; i < 8; ++i) s += f[v][i];
      }
    }
    const float mean = warp_sum(s) * inv_c;
    float q = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      if (lane + 32 * v < CG) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float d = f[v][i] - mean;
          q += d * d;
        }
      }
    }
    const float rstd = rsqrtf(warp_sum(q) * inv_c + eps);
    if (lane == 0) {
      mean_out[r] = mean;
      rstd_out[r] = rstd;
    }
    __nv_bfloat16* yr = y + r * C;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int g = lane + 32 * v;
      if (g < CG) {
        float ga[8], be[8], o[8];
        load_param8(gamma, g * 8, param_bf16, ga);
        load_param8(beta, g * 8, param_bf16, be);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = (f[v][i] - mean) * rstd * ga[i] + be[i];
        *reinterpret_cast<uint4*>(yr + g * 8) = pack8(o);
      }
    }
  }
}

template <int NV>
__global__ void __launch_bounds__(kThreads) ln_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                                          const __nv_bfloat16* __restrict__ x,
                                                          const void* __restrict__ gamma,
                                                          const float* __restrict__ mean_in,
                                                          const float* __restrict__ rstd_in,
                                                          __nv_bfloat16* __restrict__ dx, float* __restrict__ dgamma,
                                                          float* __restrict__ dbeta, long long R, int C,
                                                          int param_bf16) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int CG = C >> 3;
  const long long warp0 = (long long)blockIdx.x * kWarps + warp;
  const long long nwarps = (long long)gridDim.x * kWarps;
  const float inv_c = 1.f / (float)C;
  float ga[NV][8], sg[NV][8], sb[NV][8];
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int g = lane + 32 * v;
#pragma unroll
    for (int i = 0; i < 8; ++i) ga[v][i] = sg[v][i] = sb[v][i] = 0.f;
    if (g < CG) load_param8(gamma, g * 8, param_bf16, ga[v]);
  }
  for (long long r = warp0; r < R; r += nwarps) {
    const float mean = mean_in[r], rstd = rstd_in[r];
    float fd[NV][8], xh[NV][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int g = lane + 32 * v;
      if (g < CG) {
        unpack8(*reinterpret_cast<const uint4*>(dy + r * C + g * 8), fd[v]);
        unpack8(*reinterpret_cast<const uint4*>(x + r * C + g * 8), xh[v]);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          xh[v][i] = (xh[v][i] - mean) * rstd;
          sg[v][i] += fd[v][i] * xh[v][i];
          sb[v][i] += fd[v][i];
          fd[v][i] *= ga[v][i];
          s1 += fd[v][i];
          s2 += fd[v][i] * xh[v][i];
        }
      }
    }
    s1 = warp_sum(s1) * inv_c;
    s2 = warp_sum(s2) * inv_c;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int g = lane + 32 * v;
      if (g < CG) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = rstd * (fd[v][i] - s1 - xh[v][i] * s2);
        *reinterpret_cast<uint4*>(dx + r * C + g * 8) = pack8(o);
      }
    }
  }
  // column sums: the warps of a block fold one vector slot (256 columns) at a time through shared
  // memory, then the block adds each column once to the global fp32 sums
  __shared__ float fold_g[32 * 8];
  __shared__ float fold_b[32 * 8];
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    __syncthreads();
    for (int i = threadIdx.x; i < 256; i += kThreads) fold_g[i] = fold_b[i] = 0.f;
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      atomicAdd(&fold_g[lane * 8 + i], sg[v][i]);
      atomicAdd(&fold_b[lane * 8 + i], sb[v][i]);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 256; i += kThreads) {
      const int c = (32 * v) * 8 + i;
      if (c < C) {
        atomicAdd(&dgamma[c], fold_g[i]);
        atomicAdd(&dbeta[c], fold_b[i]);
      }
    }
  }
}

// Backward with several warps per row.  The one-warp-per-row kernel above keeps a whole row of dy and x-hat in the
// registers of 32 threads (212 registers at 1024 columns), which leaves one block of eight warps per SM and eight
// rows in flight: the pass is then bound by the latency of one row after the other (34 us for 8192 x 1024, where the
// traffic takes 8).  Here a row belongs to `tpr` threads (the columns / 8, rounded up to warps; one 16-byte vector
// per thread), a block holds 256 / tpr rows side by side and every thread walks two rows per step, so that an SM has
// a dozen rows in flight; the two row sums cross the warps of a row through shared memory (double-buffered, one
// named barrier per step).  Column sums stay in registers per thread and leave through shared memory with one
// vector reduction per four columns and block (no shared-memory atomics: their fp32 form is a CAS loop).
__device__ __forceinline__ void row_bar(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

//
// EXTRA: the row's gradient has a second term that skips the normalisation (the residual stream of a transformer
// block: x feeds the LayerNorm and the addition behind the sub-layer), dx = LN'(dy) + addend, and the column sums of
// that total leave with it (the bias gradient of the linear layer whose output, plus residual, was x).
template <bool EXTRA>
__global__ void __launch_bounds__(kThreads, EXTRA ? 2 : 3) ln_bwd_rows_kernel(
    const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x, const void* __restrict__ gamma,
    const float* __restrict__ mean_in, const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dx,
    float* __restrict__ dgamma, float* __restrict__ dbeta, const __nv_bfloat16* __restrict__ addend,
    float* __restrict__ colsum, long long R, int C, int param_bf16, int tpr) {
  constexpr int kPark = EXTRA ? 24 : 16;
  __shared__ float red[2][8][8][4];              // [buffer][row group][warp of the group][s1, s2 of two rows]
  __shared__ float park[kThreads * kPark];       // column sums of every thread on their way out
  const int CG = C >> 3;
  const int G = kThreads / tpr;                  // row groups per block
  const int grp = threadIdx.x / tpr, t = threadIdx.x % tpr;
  const int lane = threadIdx.x & 31, wig = t >> 5, nw = tpr >> 5;
  const bool active = grp < G && t < CG;         // threads past the last column group only take part in barriers
  const float inv_c = 1.f / (float)C;
  float ga[8], sg[8], sb[8], sc[EXTRA ? 8 : 1];
#pragma unroll
  for (int i = 0; i < 8; ++i) ga[i] = sg[i] = sb[i] = 0.f;
#pragma unroll
  for (int i = 0; i < (EXTRA ? 8 : 1); ++i) sc[i] = 0.f;
  if (active) load_param8(gamma, t * 8, param_bf16, ga);
  const long long step = (long long)gridDim.x * G * 2;
  int buf = 0;
  if (grp < G) {
    for (long long r0 = ((long long)blockIdx.x * G + grp) * 2; r0 < R; r0 += step) {
      const bool two = r0 + 1 < R;
      float fd[2][8], xh[2][8];
      float s[4] = {0.f, 0.f, 0.f, 0.f};
      uint4 ad[2] = {make_uint4(0u, 0u, 0u, 0u), make_uint4(0u, 0u, 0u, 0u)};
      if (EXTRA && active) {
        ad[0] = *reinterpret_cast<const uint4*>(addend + r0 * C + t * 8);
        if (two) ad[1] = *reinterpret_cast<const uint4*>(addend + (r0 + 1) * C + t * 8);
      }
      if (active) {
        const uint4 d0 = *reinterpret_cast<const uint4*>(dy + r0 * C + t * 8);
        const uint4 x0 = *reinterpret_cast<const uint4*>(x + r0 * C + t * 8);
        uint4 d1 = make_uint4(0u, 0u, 0u, 0u), x1 = make_uint4(0u, 0u, 0u, 0u);
        if (two) {
          d1 = *reinterpret_cast<const uint4*>(dy + (r0 + 1) * C + t * 8);
          x1 = *reinterpret_cast<const uint4*>(x + (r0 + 1) * C + t * 8);
        }
        unpack8(d0, fd[0]); unpack8(x0, xh[0]); unpack8(d1, fd[1]); unpack8(x1, xh[1]);
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          if (k == 1 && !two) break;
          const float mean = mean_in[r0 + k], rstd = rstd_in[r0 + k];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            xh[k][i] = (xh[k][i] - mean) * rstd;
            sg[i] += fd[k][i] * xh[k][i];
            sb[i] += fd[k][i];
            fd[k][i] *= ga[i];
            s[2 * k] += fd[k][i];
            s[2 * k + 1] += fd[k][i] * xh[k][i];
          }
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) s[j] = warp_sum(s[j]);
      if (nw > 1) {
        if (lane == 0) {
#pragma unroll
          for (int j = 0; j < 4; ++j) red[buf][grp][wig][j] = s[j];
        }
        row_bar(1 + grp, tpr);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float tsum = 0.f;
          for (int w = 0; w < nw; ++w) tsum += red[buf][grp][w][j];
          s[j] = tsum;
        }
        buf ^= 1;
      }
      if (active) {
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          if (k == 1 && !two) break;
          const float rstd = rstd_in[r0 + k];
          const float m1 = s[2 * k] * inv_c, m2 = s[2 * k + 1] * inv_c;
          float o[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = rstd * (fd[k][i] - m1 - xh[k][i] * m2);
          if (EXTRA) {
            float a[8];
            unpack8(ad[k], a);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              o[i] += a[i];
              sc[i] += o[i];
            }
          }
          *reinterpret_cast<uint4*>(dx + (r0 + k) * C + t * 8) = pack8(o);
        }
      }
    }
  }
  // column sums: every thread parks its values, one thread per column quad adds up the row groups and issues one
  // vector reduction per four columns
  {
    float* mine = park + size_t(threadIdx.x) * kPark;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      mine[i] = (grp < G) ? sg[i] : 0.f;
      mine[8 + i] = (grp < G) ? sb[i] : 0.f;
      if (EXTRA) mine[16 + i] = (grp < G) ? sc[i] : 0.f;
    }
  }
  __syncthreads();
  constexpr int kSums = EXTRA ? 3 : 2;           // dgamma, dbeta(, column sums of dx)
  for (int qd = threadIdx.x; qd < CG * 2 * kSums; qd += kThreads) {
    const int g8 = qd / (2 * kSums), rem = qd % (2 * kSums), which = rem >> 1, half = rem & 1;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int gg = 0; gg < G; ++gg) {
      const float* src = park + size_t(gg * tpr + g8) * kPark + which * 8 + half * 4;
      acc.x += src[0]; acc.y += src[1]; acc.z += src[2]; acc.w += src[3];
    }
    float* dst = (which == 0 ? dgamma : which == 1 ? dbeta : colsum) + g8 * 8 + half * 4;
    asm volatile("red.relaxed.gpu.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(acc.x), "f"(acc.y), "f"(acc.z), "f"(acc.w) : "memory");
  }
}

// out[c] += sum over rows of x[r, c]  (bf16 [R, C] row-major, fp32 sums; out holds zeros on entry).
// The bias gradient of a linear layer.  A block owns 256 consecutive columns (one 16-byte vector per lane
// and row) and a slice of the rows; its warps stride over the rows, park their partial sums in shared memory and
// one thread per column adds them to the global sums.
__global__ void __launch_bounds__(kThreads) column_sum_kernel(const __nv_bfloat16* __restrict__ x,
                                                              float* __restrict__ out, long long R, int C) {
  __shared__ float fold[kWarps][256];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int c0 = blockIdx.x * 256 + lane * 8;
  const long long chunk = (R + gridDim.y - 1) / gridDim.y;
  const long long r0 = (long long)blockIdx.y * chunk;
  const long long r1 = r0 + chunk < R ? r0 + chunk : R;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  if (c0 < C) {
    constexpr int U = 4;
    long long r = r0 + warp;
    for (; r + (long long)(U - 1) * kWarps < r1; r += (long long)U * kWarps) {
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) v[u] = *reinterpret_cast<const uint4*>(x + (r + (long long)u * kWarps) * C + c0);
#pragma unroll
      for (int u = 0; u < U; ++u) {
        float f[8];
        unpack8(v[u], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += f[i];
      }
    }
    for (; r < r1; r += kWarps) {
      float f[8];
      unpack8(*reinterpret_cast<const uint4*>(x + r * C + c0), f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += f[i];
    }
  }
  // every warp parks its 256 partial sums; one thread per column adds the eight warps up (fp32 atomics on shared
  // memory are a CAS loop, eight-way contended here)
#pragma unroll
  for (int i = 0; i < 8; ++i) fold[warp][lane * 8 + i] = acc[i];
  __syncthreads();
  for (int i = threadIdx.x; i < 256; i += kThreads) {
    const int c = blockIdx.x * 256 + i;
    if (c < C) {
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) t += fold[w][i];
      atomicAdd(&out[c], t);
    }
  }
}

int SmCount() {
  static int sms = [] {
    int dev = 0, n = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    return n > 0 ? n : 148;
  }();
  return sms;
}

int GridFor(long long R) {
  long long blocks = (R + kWarps - 1) / kWarps;
  if (blocks < 1) blocks = 1;
  if (blocks > SmCount() * 4) blocks = SmCount() * 4;
  return (int)blocks;
}

// The backward kernel ends with one global atomic per column and block: few, long-lived blocks (one per SM)
// keep the contention on the 2*C sums low.
int GridForBackward(long long R) {
  long long blocks = (R + kWarps - 1) / kWarps;
  if (blocks < 1) blocks = 1;
  if (blocks > SmCount()) blocks = SmCount();
  return (int)blocks;
}

}  // namespace

bool LnShapeSupported(long long R, int C) { return R > 0 && C >= 8 && C <= kMaxC && (C % 8) == 0; }

#define BFB_LN_DISPATCH(NVV, CALL)                 \
  switch (NVV) {                                   \
    case 1: { constexpr int NV = 1; CALL; } break; \
    case 2: { constexpr int NV = 2; CALL; } break; \
    case 3: { constexpr int NV = 3; CALL; } break; \
    case 4: { constexpr int NV = 4; CALL; } break; \
    case 5: { constexpr int NV = 5; CALL; } break; \
    case 6: { constexpr int NV = 6; CALL; } break; \
    case 7: { constexpr int NV = 7; CALL; } break; \
    default: { constexpr int NV = 8; CALL; } break; \
  }

cudaError_t LaunchLnForward(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd,
                            long long R, int C, float eps, int param_bf16, cudaStream_t stream) {
  if (!LnShapeSupported(R, C)) return cudaErrorInvalidValue;
  const int nv = ((C >> 3) + 31) / 32;
  BFB_LN_DISPATCH(nv, (ln_fwd_kernel<NV><<<GridFor(R), kThreads, 0, stream>>>(
                          static_cast<const __nv_bfloat16*>(x), gamma, beta, static_cast<__nv_bfloat16*>(y), mean,
                          rstd, R, C, eps, param_bf16)));
  CountKernelLaunch();
  return cudaGetLastError();
}

cudaError_t LaunchLnBackward(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd,
                             void* dx, float* dgamma_zeroed, float* dbeta_zeroed, long long R, int C, int param_bf16,
                             cudaStream_t stream, const void* addend, float* colsum_zeroed) {
  if (!LnShapeSupported(R, C)) return cudaErrorInvalidValue;
  if ((addend == nullptr) != (colsum_zeroed == nullptr)) return cudaErrorInvalidValue;
  const int CG = C >> 3;
  static const bool rows_off = [] { const char* e = std::getenv("BLUEFOG_B200_LN_ROWS"); return e != nullptr && e[0] == '0'; }();
  // the sums are reduced as 16-byte vectors: dgamma and dbeta have to be 16-byte aligned for the row-group kernel
  if (!rows_off && CG <= kThreads && (reinterpret_cast<uintptr_t>(dgamma_zeroed) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(dbeta_zeroed) & 15) == 0 && (reinterpret_cast<uintptr_t>(colsum_zeroed) & 15) == 0) {
    const int tpr = ((CG + 31) / 32) * 32;                     // threads per row, whole warps
    const int G = kThreads / tpr;
    long long blocks = (R + 2 * G - 1) / (2 * G);
    const long long cap = (long long)SmCount() * (addend != nullptr ? 2 : 3);
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    if (addend != nullptr)
      ln_bwd_rows_kernel<true><<<static_cast<unsigned>(blocks), kThreads, 0, stream>>>(
          static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x), gamma, mean, rstd,
          static_cast<__nv_bfloat16*>(dx), dgamma_zeroed, dbeta_zeroed, static_cast<const __nv_bfloat16*>(addend),
          colsum_zeroed, R, C, param_bf16, tpr);
    else
      ln_bwd_rows_kernel<false><<<static_cast<unsigned>(blocks), kThreads, 0, stream>>>(
          static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x), gamma, mean, rstd,
          static_cast<__nv_bfloat16*>(dx), dgamma_zeroed, dbeta_zeroed, nullptr, nullptr, R, C, param_bf16, tpr);
    CountKernelLaunch();
    return cudaGetLastError();
  }
  if (addend != nullptr) return cudaErrorNotSupported;       // only the row-group kernel takes the second term
  const int nv = ((C >> 3) + 31) / 32;
  BFB_LN_DISPATCH(nv, (ln_bwd_kernel<NV><<<GridForBackward(R), kThreads, 0, stream>>>(
                          static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x), gamma, mean,
                          rstd, static_cast<__nv_bfloat16*>(dx), dgamma_zeroed, dbeta_zeroed, R, C, param_bf16)));
  CountKernelLaunch();
  return cudaGetLastError();
}

cudaError_t LaunchColumnSum(const void* x, float* out_zeroed, long long R, int C, cudaStream_t stream) {
  if (R <= 0 || C < 8 || (C % 8) != 0) return cudaErrorInvalidValue;
  const int col_blocks = (C + 255) / 256;
  long long row_blocks = (SmCount() * 4 + col_blocks - 1) / col_blocks;
  const long long max_rows = (R + kWarps * 4 - 1) / (kWarps * 4);      // at least four rows per warp
  if (row_blocks > max_rows) row_blocks = max_rows;
  if (row_blocks < 1) row_blocks = 1;
  column_sum_kernel<<<dim3(static_cast<unsigned>(col_blocks), static_cast<unsigned>(row_blocks)), kThreads, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), out_zeroed, R, C);
  CountKernelLaunch();
  return cudaGetLastError();
}

}  // namespace bfb
