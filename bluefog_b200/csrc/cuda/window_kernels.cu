// Window kernels for sm_100a: plain and vector stores/reductions into peer memory.
#include "window_kernels.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace bfb {
namespace {

constexpr int kThreads = 512;

__device__ __forceinline__ void red_add_release_sys_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void red_add_sys_f64(double* p, double v) {
  asm volatile("red.relaxed.sys.global.add.f64 [%0], %1;" ::"l"(p), "d"(v) : "memory");
}
__device__ __forceinline__ void red_add_v4_f32(float* p, float a, float b, float c, float d) {
  asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}

__device__ bool last_block(unsigned int* counter) {
  __shared__ bool is_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned int prev = atomicAdd(counter, 1u);
    is_last = (prev == gridDim.x - 1);
    if (is_last) *counter = 0;
    __threadfence_system();
  }
  __syncthreads();
  return is_last;
}

template <typename T> struct WT;  // scalar traits
template <> struct WT<float> { using A = float; static __device__ A ld(const float* p) { return *p; } static __device__ void st(float* p, A a) { *p = a; }
  static __device__ void add(float* p, A a) { asm volatile("red.relaxed.sys.global.add.f32 [%0], %1;" ::"l"(p), "f"(a) : "memory"); } };
template <> struct WT<double> { using A = double; static __device__ A ld(const double* p) { return *p; } static __device__ void st(double* p, A a) { *p = a; }
  static __device__ void add(double* p, A a) { red_add_sys_f64(p, a); } };
template <> struct WT<int> { using A = double; static __device__ A ld(const int* p) { return (double)*p; } static __device__ void st(int* p, A a) { *p = (int)a; }
  static __device__ void add(int* p, A a) { int v = (int)a; asm volatile("red.relaxed.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); } };
template <> struct WT<long long> { using A = double; static __device__ A ld(const long long* p) { return (double)*p; } static __device__ void st(long long* p, A a) { *p = (long long)a; }
  static __device__ void add(long long* p, A a) { unsigned long long v = (unsigned long long)(long long)a; asm volatile("red.relaxed.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory"); } };
template <> struct WT<__nv_bfloat16> { using A = float; static __device__ A ld(const __nv_bfloat16* p) { return __bfloat162float(*p); } static __device__ void st(__nv_bfloat16* p, A a) { *p = __float2bfloat16_rn(a); }
  static __device__ void add(__nv_bfloat16* p, A a) { atomicAdd(p, __float2bfloat16_rn(a)); } };
template <> struct WT<__half> { using A = float; static __device__ A ld(const __half* p) { return __half2float(*p); } static __device__ void st(__half* p, A a) { *p = __float2half_rn(a); }
  static __device__ void add(__half* p, A a) { atomicAdd(p, __float2half_rn(a)); } };

template <typename T>
__global__ void __launch_bounds__(kThreads) win_put_kernel(const __grid_constant__ WinPutParams p) {
  using A = typename WT<T>::A;
  const T* src = static_cast<const T*>(p.src);
  T* self_t = static_cast<T*>(p.self_scale_target);
  const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
  const unsigned long long tid = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
  const bool scale_self = self_t != nullptr && p.self_weight != 1.0;
  constexpr bool kIsF32 = sizeof(T) == 4 && sizeof(A) == 4;
  bool vec_ok = kIsF32 && ((reinterpret_cast<uintptr_t>(src) & 15) == 0) &&
                (self_t == nullptr || (reinterpret_cast<uintptr_t>(self_t) & 15) == 0);
  unsigned long long vec_elems = 0;
  if (vec_ok) {
    vec_elems = p.numel & ~3ull;
    for (unsigned long long i = tid * 4; i < vec_elems; i += stride * 4) {
      float4 x = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(src) + i);
      for (int d = 0; d < p.n_dst; ++d) {
        const float w = (float)p.weight[d];
        float* dst = static_cast<float*>(p.dst_slot[d]) + i;
        if (p.accumulate) red_add_v4_f32(dst, w * x.x, w * x.y, w * x.z, w * x.w);
        else *reinterpret_cast<float4*>(dst) = make_float4(w * x.x, w * x.y, w * x.z, w * x.w);
      }
      if (scale_self) {
        const float s = (float)p.self_weight;
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(self_t) + i) = make_float4(s * x.x, s * x.y, s * x.z, s * x.w);
      }
    }
  }
  for (unsigned long long i = vec_elems + tid; i < p.numel; i += stride) {
    const A x = WT<T>::ld(src + i);
    for (int d = 0; d < p.n_dst; ++d) {
      T* dst = static_cast<T*>(p.dst_slot[d]) + i;
      const A v = (A)(x * (A)p.weight[d]);
      if (p.accumulate) WT<T>::add(dst, v); else WT<T>::st(dst, v);
    }
    if (scale_self) WT<T>::st(self_t + i, (A)(x * (A)p.self_weight));
  }
  if (last_block(p.block_counter)) {
    // The data is visible system-wide (fences in last_block); now publish versions and p.
    if (threadIdx.x < p.n_dst) {
      const int d = threadIdx.x;
      if (p.with_p) {
        const double mine = p.my_header->p[p.my_rank];
        double* slot = &p.dst_header[d]->p[p.my_rank];
        if (p.accumulate) red_add_sys_f64(slot, mine * p.weight[d]);
        else *reinterpret_cast<volatile double*>(slot) = mine * p.weight[d];
        __threadfence_system();
      }
      red_add_release_sys_u64(&p.dst_header[d]->version[p.my_rank], 1ull);
    }
    __syncthreads();
    if (threadIdx.x == 0 && p.with_p && p.self_weight != 1.0) p.my_header->p[p.my_rank] *= p.self_weight;
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) win_get_kernel(const __grid_constant__ WinGetParams p) {
  using A = typename WT<T>::A;
  const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
  const unsigned long long tid = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
  for (int s = 0; s < p.n_src; ++s) {
    const T* src = static_cast<const T*>(p.src_self[s]);
    T* dst = static_cast<T*>(p.local_slot[s]);
    const A w = (A)p.weight[s];
    for (unsigned long long i = tid; i < p.numel; i += stride) {
      T raw;
      if (sizeof(T) == 4) { unsigned v; asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(src + i) : "memory"); raw = *reinterpret_cast<T*>(&v); }
      else if (sizeof(T) == 8) { unsigned long long v; asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(src + i) : "memory"); raw = *reinterpret_cast<T*>(&v); }
      else { unsigned short v; asm volatile("ld.relaxed.sys.global.u16 %0, [%1];" : "=h"(v) : "l"(src + i) : "memory"); raw = *reinterpret_cast<T*>(&v); }
      WT<T>::st(dst + i, (A)(WT<T>::ld(&raw) * w));
    }
  }
  if (last_block(p.block_counter)) {
    if (threadIdx.x < p.n_src) atomicAdd(&p.my_header->version[p.src_rank[threadIdx.x]], 1ull);
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) win_update_kernel(const __grid_constant__ WinUpdateParams p) {
  using A = typename WT<T>::A;
  T* self_t = static_cast<T*>(p.self);
  T* out = static_cast<T*>(p.out);
  const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
  const unsigned long long tid = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
  for (unsigned long long i = tid; i < p.numel; i += stride) {
    A acc = (A)(WT<T>::ld(self_t + i) * (A)p.self_weight);
    for (int s = 0; s < p.n_src; ++s) {
      T* slot = static_cast<T*>(p.slot[s]) + i;
      acc += (A)(WT<T>::ld(slot) * (A)p.weight[s]);
      if (p.reset) WT<T>::st(slot, (A)0);
    }
    WT<T>::st(out + i, acc);
  }
  if (last_block(p.block_counter)) {
    if (threadIdx.x == 0) {
      if (p.with_p) {
        double v = p.my_header->p[p.my_rank] * p.self_weight;
        for (int s = 0; s < p.n_src; ++s) {
          v += p.my_header->p[p.src_rank[s]] * p.weight[s];
          if (p.reset) p.my_header->p[p.src_rank[s]] = 0.0;
        }
        p.my_header->p[p.my_rank] = v;
      }
    }
    // Versions of every source are cleared by an update.
    for (int r = threadIdx.x; r < kMaxWorld; r += blockDim.x) p.my_header->version[r] = 0ull;
    __threadfence_system();
  }
}

int Grid(unsigned long long items) {
  unsigned long long b = (items + kThreads - 1) / kThreads;
  if (b < 1) b = 1;
  return (int)(b < 296 ? b : 296);
}

#define BFB_DISPATCH_WIN(kernel, grid, stream, p)                                      \
  switch ((p).elem_type) {                                                             \
    case kF32: kernel<float><<<grid, kThreads, 0, stream>>>(p); break;                 \
    case kF64: kernel<double><<<grid, kThreads, 0, stream>>>(p); break;                \
    case kI32: kernel<int><<<grid, kThreads, 0, stream>>>(p); break;                   \
    case kI64: kernel<long long><<<grid, kThreads, 0, stream>>>(p); break;             \
    case kBF16: kernel<__nv_bfloat16><<<grid, kThreads, 0, stream>>>(p); break;        \
    case kF16: kernel<__half><<<grid, kThreads, 0, stream>>>(p); break;                \
    default: return cudaErrorInvalidValue;                                             \
  }

}  // namespace

cudaError_t LaunchWinPut(const WinPutParams& p, cudaStream_t stream) {
  const int grid = Grid(p.numel / 4 + 1);
  BFB_DISPATCH_WIN(win_put_kernel, grid, stream, p);
  CountKernelLaunch();
  return cudaGetLastError();
}

cudaError_t LaunchWinGet(const WinGetParams& p, cudaStream_t stream) {
  const int grid = Grid(p.numel);
  BFB_DISPATCH_WIN(win_get_kernel, grid, stream, p);
  CountKernelLaunch();
  return cudaGetLastError();
}

cudaError_t LaunchWinUpdate(const WinUpdateParams& p, cudaStream_t stream) {
  const int grid = Grid(p.numel);
  BFB_DISPATCH_WIN(win_update_kernel, grid, stream, p);
  CountKernelLaunch();
  return cudaGetLastError();
}

}  // namespace bfb
