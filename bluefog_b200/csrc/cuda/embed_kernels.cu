// Token + position embedding, forward and backward, bf16 rows with fp32 sums.
//
// The reference has no model code of its own (its examples take torchvision models, examples/pytorch_benchmark.py:100);
// these kernels serve this library's GPT-2 (models/gpt2.py).  PyTorch's path is two gathers and an addition forward,
// and a sort by token, a segmented reduction, a dense scatter and a separate position sum backward (about 0.33 ms
// for 8192 tokens of 1024 values into a 50257-row table).  Here:
//   forward   one pass: out = wte[idx] + wpe[pos], 16-byte vectors;
//   backward  (1) the first position of every token becomes its representative (atomicMin into a slot table),
//             (2) every row of dx is added (fp32 vector reductions) into the representative's row of a [N, C]
//                 accumulator, and the position gradient is the plain sum over the batch,
//             (3) the dense table gradient is zero-filled and the representatives' rows are converted into it; the
//                 slot table and the accumulator are handed back clean.
// Sums over repeated tokens are taken in fp32 in an order that varies from run to run (atomics).
#include "embed_kernels.h"

#include <cuda_bf16.h>
#include <stdint.h>

#include <climits>

#include "comm_kernels.h"

namespace bfb {
void CountKernelLaunch();

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 v;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return v;
}

// one thread per 16-byte vector of the output
__global__ void __launch_bounds__(kThreads) embed_fwd_kernel(const long long* __restrict__ idx,
                                                             const __nv_bfloat16* __restrict__ wte,
                                                             const __nv_bfloat16* __restrict__ wpe,
                                                             __nv_bfloat16* __restrict__ out, long long N, int T, int CG,
                                                             long long V, int* __restrict__ bad) {
  const long long total = N * CG;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
    const long long row = e / CG;
    const int g = (int)(e - row * CG);
    const long long tok = idx[row];
    const int C = CG * 8;
    float a[8], b[8];
    unpack8(*reinterpret_cast<const uint4*>(wpe + (row % T) * C + g * 8), b);
    if (tok >= 0 && tok < V) {
      unpack8(*reinterpret_cast<const uint4*>(wte + tok * C + g * 8), a);
#pragma unroll
      for (int i = 0; i < 8; ++i) b[i] += a[i];
    } else if (bad != nullptr && g == 0) {
      *bad = 1;
    }
    *reinterpret_cast<uint4*>(out + row * C + g * 8) = pack8(b);
  }
}

__global__ void __launch_bounds__(kThreads) embed_slot_kernel(const long long* __restrict__ idx, int* __restrict__ slot,
                                                              long long N, long long V) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < N) {
    const long long tok = idx[i];
    if (tok >= 0 && tok < V) atomicMin(&slot[tok], (int)i);
  }
}

// blocks [0, rows_blocks): token rows into the accumulator; the rest: the position gradient
__global__ void __launch_bounds__(kThreads) embed_accumulate_kernel(const long long* __restrict__ idx,
                                                                    const __nv_bfloat16* __restrict__ dx,
                                                                    const int* __restrict__ slot, float* __restrict__ acc,
                                                                    __nv_bfloat16* __restrict__ d_wpe, long long N, int T,
                                                                    int CG, long long V, long long token_vecs) {
  const int C = CG * 8;
  const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e < token_vecs) {                              // token_vecs is padded to whole blocks
    const long long row = e / CG;
    if (row >= N) return;
    const int g = (int)(e - row * CG);
    const long long tok = idx[row];
    if (tok < 0 || tok >= V) return;
    const int rep = slot[tok];
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(dx + row * C + g * 8), f);
    float* dst = acc + (long long)rep * C + g * 8;
    asm volatile("red.relaxed.gpu.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(f[0]), "f"(f[1]), "f"(f[2]), "f"(f[3]) : "memory");
    asm volatile("red.relaxed.gpu.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + 4), "f"(f[4]), "f"(f[5]), "f"(f[6]), "f"(f[7]) : "memory");
  } else {
    const long long p = e - token_vecs;
    if (p >= (long long)T * CG) return;
    const long long t = p / CG;
    const int g = (int)(p - t * CG);
    float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (long long row = t; row < N; row += T) {
      float f[8];
      unpack8(*reinterpret_cast<const uint4*>(dx + row * C + g * 8), f);
#pragma unroll
      for (int i = 0; i < 8; ++i) s[i] += f[i];
    }
    *reinterpret_cast<uint4*>(d_wpe + t * C + g * 8) = pack8(s);
  }
}

// zero fill of the dense gradient (grid-stride, 16 bytes per thread and step)
__global__ void __launch_bounds__(kThreads) embed_zero_kernel(uint4* __restrict__ p, long long n_vec) {
  const uint4 z = make_uint4(0u, 0u, 0u, 0u);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += (long long)gridDim.x * blockDim.x) p[i] = z;
}

// representatives write their token's row; every position resets what it touched
__global__ void __launch_bounds__(kThreads) embed_finalize_kernel(const long long* __restrict__ idx, int* __restrict__ slot,
                                                                  float* __restrict__ acc, __nv_bfloat16* __restrict__ d_wte,
                                                                  long long N, int CG, long long V) {
  const int C = CG * 8;
  const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= N * CG) return;
  const long long row = e / CG;
  const int g = (int)(e - row * CG);
  const long long tok = idx[row];
  if (tok < 0 || tok >= V) return;
  if (slot[tok] != (int)row) return;           // not the representative: its accumulator row was never written
  float* src = acc + row * C + g * 8;
  const float4 lo = *reinterpret_cast<const float4*>(src), hi = *reinterpret_cast<const float4*>(src + 4);
  const float f[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
  *reinterpret_cast<uint4*>(d_wte + tok * C + g * 8) = pack8(f);
  *reinterpret_cast<float4*>(src) = make_float4(0.f, 0.f, 0.f, 0.f);
  *reinterpret_cast<float4*>(src + 4) = make_float4(0.f, 0.f, 0.f, 0.f);
}

// after every thread of the finalize pass has compared against the slot table
__global__ void __launch_bounds__(kThreads) embed_reset_slot_kernel(const long long* __restrict__ idx, int* __restrict__ slot,
                                                                    long long N, long long V) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < N) {
    const long long tok = idx[i];
    if (tok >= 0 && tok < V) slot[tok] = INT_MAX;
  }
}

unsigned Blocks(long long n) { return static_cast<unsigned>((n + kThreads - 1) / kThreads); }

}  // namespace

cudaError_t LaunchEmbedForward(const long long* idx, const void* wte, const void* wpe, void* out, long long N, int T,
                               int C, long long V, int* bad_index_flag, cudaStream_t stream) {
  if (N <= 0 || T <= 0 || C < 8 || (C % 8) != 0 || V <= 0) return cudaErrorInvalidValue;
  const int CG = C / 8;
  long long blocks = (N * CG + kThreads - 1) / kThreads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  embed_fwd_kernel<<<static_cast<unsigned>(blocks), kThreads, 0, stream>>>(
      idx, static_cast<const __nv_bfloat16*>(wte), static_cast<const __nv_bfloat16*>(wpe), static_cast<__nv_bfloat16*>(out), N,
      T, CG, V, bad_index_flag);
  CountKernelLaunch();
  return cudaGetLastError();
}

cudaError_t LaunchEmbedBackward(const long long* idx, const void* dx, void* d_wte, void* d_wpe, int* slot, float* acc,
                                long long N, int T, int C, long long V, cudaStream_t stream) {
  if (N <= 0 || T <= 0 || C < 8 || (C % 8) != 0 || V <= 0 || N > INT_MAX || (N % T) != 0) return cudaErrorInvalidValue;
  const int CG = C / 8;
  const long long token_vecs = N * CG;
  embed_slot_kernel<<<Blocks(N), kThreads, 0, stream>>>(idx, slot, N, V);
  // the token part is padded to whole blocks so that a block is either all token rows or all position rows
  const long long token_padded = (token_vecs + kThreads - 1) / kThreads * kThreads;
  embed_accumulate_kernel<<<Blocks(token_padded + (long long)T * CG), kThreads, 0, stream>>>(
      idx, static_cast<const __nv_bfloat16*>(dx), slot, acc, static_cast<__nv_bfloat16*>(d_wpe), N, T, CG, V, token_padded);
  const long long n_vec = V * CG;
  long long zb = (n_vec + kThreads - 1) / kThreads;
  if (zb > 148 * 32) zb = 148 * 32;
  embed_zero_kernel<<<static_cast<unsigned>(zb), kThreads, 0, stream>>>(static_cast<uint4*>(d_wte), n_vec);
  embed_finalize_kernel<<<Blocks(token_vecs), kThreads, 0, stream>>>(idx, slot, acc, static_cast<__nv_bfloat16*>(d_wte), N, CG, V);
  embed_reset_slot_kernel<<<Blocks(N), kThreads, 0, stream>>>(idx, slot, N, V);
  for (int i = 0; i < 5; ++i) CountKernelLaunch();
  return cudaGetLastError();
}

}  // namespace bfb
