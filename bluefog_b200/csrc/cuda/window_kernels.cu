// Window kernels for sm_100a: 16-byte stores, vector reductions and 16-byte loads into / out of peer memory for
// every element type, an atomic read-and-clear for win_update(reset), and the device-side window mutex.
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
__device__ __forceinline__ uint4 ld_sys_v4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
// Atomic read-and-clear of 16 bytes: what a concurrent reduction adds lands either before the exchange (and is
// returned) or after it (and stays for the next update); nothing is lost.
__device__ __forceinline__ uint4 exch_zero_v4(void* p) {
  uint4 v;
  asm volatile(
      "{\n\t.reg .b128 old, zero;\n\t"
      "mov.b128 zero, {%5, %5};\n\t"
      "atom.relaxed.sys.global.exch.b128 old, [%4], zero;\n\t"
      "mov.b128 {%0, %1, %2, %3}, old;\n\t}"
      : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
      : "l"(p), "l"(0ull)
      : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
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

// Element traits: A = arithmetic type, N = elements per 16 bytes, unpack/pack of a 16-byte vector, scalar access,
// scalar and 16-byte reductions into (peer) global memory.
template <typename T> struct WT;
template <> struct WT<float> {
  using A = float; static constexpr int N = 4;
  static __device__ A ld(const float* p) { return *p; }
  static __device__ void st(float* p, A a) { *p = a; }
  static __device__ void add(float* p, A a) { asm volatile("red.relaxed.sys.global.add.f32 [%0], %1;" ::"l"(p), "f"(a) : "memory"); }
  static __device__ void unpack(const uint4& v, A* a) { a[0] = __uint_as_float(v.x); a[1] = __uint_as_float(v.y); a[2] = __uint_as_float(v.z); a[3] = __uint_as_float(v.w); }
  static __device__ uint4 pack(const A* a) { return make_uint4(__float_as_uint(a[0]), __float_as_uint(a[1]), __float_as_uint(a[2]), __float_as_uint(a[3])); }
  static __device__ void add16(void* p, const A* a) {
    asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(a[0]), "f"(a[1]), "f"(a[2]), "f"(a[3]) : "memory");
  }
};
template <> struct WT<double> {
  using A = double; static constexpr int N = 2;
  static __device__ A ld(const double* p) { return *p; }
  static __device__ void st(double* p, A a) { *p = a; }
  static __device__ void add(double* p, A a) { red_add_sys_f64(p, a); }
  static __device__ void unpack(const uint4& v, A* a) {
    a[0] = __longlong_as_double((long long)(((unsigned long long)v.y << 32) | v.x));
    a[1] = __longlong_as_double((long long)(((unsigned long long)v.w << 32) | v.z));
  }
  static __device__ uint4 pack(const A* a) {
    const unsigned long long x = (unsigned long long)__double_as_longlong(a[0]), y = (unsigned long long)__double_as_longlong(a[1]);
    return make_uint4((unsigned)x, (unsigned)(x >> 32), (unsigned)y, (unsigned)(y >> 32));
  }
  static __device__ void add16(void* p, const A* a) { red_add_sys_f64(static_cast<double*>(p), a[0]); red_add_sys_f64(static_cast<double*>(p) + 1, a[1]); }
};
template <> struct WT<int> {
  using A = double; static constexpr int N = 4;
  static __device__ A ld(const int* p) { return (double)*p; }
  static __device__ void st(int* p, A a) { *p = (int)a; }
  static __device__ void add(int* p, A a) { int v = (int)a; asm volatile("red.relaxed.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
  static __device__ void unpack(const uint4& v, A* a) { a[0] = (int)v.x; a[1] = (int)v.y; a[2] = (int)v.z; a[3] = (int)v.w; }
  static __device__ uint4 pack(const A* a) { return make_uint4((unsigned)(int)a[0], (unsigned)(int)a[1], (unsigned)(int)a[2], (unsigned)(int)a[3]); }
  static __device__ void add16(void* p, const A* a) { for (int i = 0; i < 4; ++i) add(static_cast<int*>(p) + i, a[i]); }
};
template <> struct WT<long long> {
  using A = double; static constexpr int N = 2;
  static __device__ A ld(const long long* p) { return (double)*p; }
  static __device__ void st(long long* p, A a) { *p = (long long)a; }
  static __device__ void add(long long* p, A a) { unsigned long long v = (unsigned long long)(long long)a; asm volatile("red.relaxed.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory"); }
  static __device__ void unpack(const uint4& v, A* a) {
    a[0] = (double)(long long)(((unsigned long long)v.y << 32) | v.x);
    a[1] = (double)(long long)(((unsigned long long)v.w << 32) | v.z);
  }
  static __device__ uint4 pack(const A* a) {
    const unsigned long long x = (unsigned long long)(long long)a[0], y = (unsigned long long)(long long)a[1];
    return make_uint4((unsigned)x, (unsigned)(x >> 32), (unsigned)y, (unsigned)(y >> 32));
  }
  static __device__ void add16(void* p, const A* a) { add(static_cast<long long*>(p), a[0]); add(static_cast<long long*>(p) + 1, a[1]); }
};
template <> struct WT<__nv_bfloat16> {
  using A = float; static constexpr int N = 8;
  static __device__ A ld(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  static __device__ void st(__nv_bfloat16* p, A a) { *p = __float2bfloat16_rn(a); }
  static __device__ void add(__nv_bfloat16* p, A a) { atomicAdd(p, __float2bfloat16_rn(a)); }
  static __device__ void unpack(const uint4& v, A* a) {
    const unsigned u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { a[2 * i] = __uint_as_float(u[i] << 16); a[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u); }
  }
  static __device__ uint4 pack(const A* a) {
    uint4 v;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(a[2 * i], a[2 * i + 1]);
    return v;
  }
  // eight bf16 values in one reduction: four packed pairs
  static __device__ void add16(void* p, const A* a) {
    const uint4 v = pack(a);
    asm volatile("red.relaxed.sys.global.add.noftz.v4.bf16x2 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
  }
};
template <> struct WT<__half> {
  using A = float; static constexpr int N = 8;
  static __device__ A ld(const __half* p) { return __half2float(*p); }
  static __device__ void st(__half* p, A a) { *p = __float2half_rn(a); }
  static __device__ void add(__half* p, A a) { atomicAdd(p, __float2half_rn(a)); }
  static __device__ void unpack(const uint4& v, A* a) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); a[2 * i] = f.x; a[2 * i + 1] = f.y; }
  }
  static __device__ uint4 pack(const A* a) {
    uint4 v;
    __half2* h = reinterpret_cast<__half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(a[2 * i], a[2 * i + 1]);
    return v;
  }
  static __device__ void add16(void* p, const A* a) {
    const uint4 v = pack(a);
    asm volatile("red.relaxed.sys.global.add.noftz.v4.f16x2 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
  }
};

__device__ __forceinline__ bool guard_failed(const WinLockState* s) {
  return s != nullptr && *reinterpret_cast<const volatile unsigned int*>(&s->failed) != 0u;
}
__device__ __forceinline__ bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <typename T>
__global__ void __launch_bounds__(kThreads) win_put_kernel(const __grid_constant__ WinPutParams p) {
  using A = typename WT<T>::A;
  constexpr int N = WT<T>::N;
  if (guard_failed(p.lock_state)) return;
  const T* src = static_cast<const T*>(p.src);
  T* self_t = static_cast<T*>(p.self_scale_target);
  const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
  const unsigned long long tid = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
  const bool scale_self = self_t != nullptr && p.self_weight != 1.0;
  // 16-byte path: the slots are 256-byte aligned by construction, the source and the scaled tensor may not be
  bool vec_ok = aligned16(src) && (self_t == nullptr || aligned16(self_t));
  for (int d = 0; d < p.n_dst; ++d) vec_ok = vec_ok && aligned16(p.dst_slot[d]);
  unsigned long long vec_elems = 0;
  if (vec_ok) {
    vec_elems = p.numel - p.numel % N;
    for (unsigned long long i = tid * N; i < vec_elems; i += stride * N) {
      A x[N];
      WT<T>::unpack(*reinterpret_cast<const uint4*>(src + i), x);
      for (int d = 0; d < p.n_dst; ++d) {
        const A w = (A)p.weight[d];
        A y[N];
#pragma unroll
        for (int k = 0; k < N; ++k) y[k] = (A)(x[k] * w);
        T* dst = static_cast<T*>(p.dst_slot[d]) + i;
        if (p.accumulate) WT<T>::add16(dst, y);
        else *reinterpret_cast<uint4*>(dst) = WT<T>::pack(y);
      }
      if (scale_self) {
        A y[N];
#pragma unroll
        for (int k = 0; k < N; ++k) y[k] = (A)(x[k] * (A)p.self_weight);
        *reinterpret_cast<uint4*>(self_t + i) = WT<T>::pack(y);
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
  constexpr int N = WT<T>::N;
  if (guard_failed(p.lock_state)) return;
  const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
  const unsigned long long tid = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
  for (int s = 0; s < p.n_src; ++s) {
    const T* src = static_cast<const T*>(p.src_self[s]);
    T* dst = static_cast<T*>(p.local_slot[s]);
    const A w = (A)p.weight[s];
    unsigned long long vec_elems = 0;
    if (aligned16(src) && aligned16(dst)) {
      vec_elems = p.numel - p.numel % N;
      for (unsigned long long i = tid * N; i < vec_elems; i += stride * N) {
        A x[N];
        WT<T>::unpack(ld_sys_v4(src + i), x);                 // 16 bytes per load over NVLink
#pragma unroll
        for (int k = 0; k < N; ++k) x[k] = (A)(x[k] * w);
        *reinterpret_cast<uint4*>(dst + i) = WT<T>::pack(x);
      }
    }
    for (unsigned long long i = vec_elems + tid; i < p.numel; i += stride) {
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
  constexpr int N = WT<T>::N;
  if (guard_failed(p.lock_state)) return;
  T* self_t = static_cast<T*>(p.self);
  T* out = static_cast<T*>(p.out);
  const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
  const unsigned long long tid = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
  bool vec_ok = aligned16(self_t) && aligned16(out);
  for (int s = 0; s < p.n_src; ++s) vec_ok = vec_ok && aligned16(p.slot[s]);
  unsigned long long vec_elems = 0;
  if (vec_ok) {
    vec_elems = p.numel - p.numel % N;
    for (unsigned long long i = tid * N; i < vec_elems; i += stride * N) {
      A acc[N];
      WT<T>::unpack(*reinterpret_cast<const uint4*>(self_t + i), acc);
#pragma unroll
      for (int k = 0; k < N; ++k) acc[k] = (A)(acc[k] * (A)p.self_weight);
      for (int s = 0; s < p.n_src; ++s) {
        T* slot = static_cast<T*>(p.slot[s]) + i;
        // reset: read and clear in one atomic, so that an accumulate arriving meanwhile is kept for the next update
        const uint4 raw = p.reset ? exch_zero_v4(slot) : ld_sys_v4(slot);
        A v[N];
        WT<T>::unpack(raw, v);
#pragma unroll
        for (int k = 0; k < N; ++k) acc[k] += (A)(v[k] * (A)p.weight[s]);
      }
      *reinterpret_cast<uint4*>(out + i) = WT<T>::pack(acc);
    }
  }
  for (unsigned long long i = vec_elems + tid; i < p.numel; i += stride) {
    A acc = (A)(WT<T>::ld(self_t + i) * (A)p.self_weight);
    for (int s = 0; s < p.n_src; ++s) {
      T* slot = static_cast<T*>(p.slot[s]) + i;
      acc += (A)(WT<T>::ld(slot) * (A)p.weight[s]);
      if (p.reset) WT<T>::st(slot, (A)0);      // the ragged tail (fewer than 16 bytes) is cleared with a plain store
    }
    WT<T>::st(out + i, acc);
  }
  if (last_block(p.block_counter)) {
    if (threadIdx.x == 0) {
      if (p.with_p) {
        double v = p.my_header->p[p.my_rank] * p.self_weight;
        for (int s = 0; s < p.n_src; ++s) {
          double* ps = &p.my_header->p[p.src_rank[s]];
          double got;
          if (p.reset) {
            const unsigned long long old = atomicExch(reinterpret_cast<unsigned long long*>(ps), 0ull);
            got = __longlong_as_double((long long)old);
          } else {
            got = *reinterpret_cast<volatile double*>(ps);
          }
          v += got * p.weight[s];
        }
        p.my_header->p[p.my_rank] = v;
      }
    }
    // Versions of every source are cleared by an update.
    for (int r = threadIdx.x; r < kMaxWorld; r += blockDim.x) p.my_header->version[r] = 0ull;
    __threadfence_system();
  }
}

// One thread takes or frees the words in order.  A word that stays taken for longer than the limit makes the
// launch give back what it already holds, raise `failed` (the guarded kernels that follow on the stream then do
// nothing) and report kCommTimeoutLock; the context stays usable.
__global__ void win_lock_kernel(const __grid_constant__ WinLockParams p) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  WinLockState* st = p.state;
  if (!p.acquire) {
    if (st->failed == 0u) {
      __threadfence_system();
      for (int i = 0; i < p.n; ++i) {
        unsigned int* w = &p.header[i]->lock[p.index[i]];
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(w), "r"(0u) : "memory");
      }
    }
    st->failed = 0u;          // the next lock launch starts clean
    st->held = 0u;
    return;
  }
  st->failed = 0u;
  const unsigned int mine = 1u + (unsigned)p.my_rank;
  int got = 0;
  for (; got < p.n; ++got) {
    unsigned int* w = &p.header[got]->lock[p.index[got]];
    const unsigned long long t0 = globaltimer_ns();
    unsigned backoff = 64;
    bool ok = false;
    for (unsigned long long it = 0; it < (1ull << 32); ++it) {
      unsigned int old;
      asm volatile("atom.acquire.sys.global.cas.b32 %0, [%1], %2, %3;" : "=r"(old) : "l"(w), "r"(0u), "r"(mine) : "memory");
      if (old == 0u) { ok = true; break; }
      if ((it & 7ull) == 7ull && globaltimer_ns() - t0 > p.timeout_ns) break;
      __nanosleep(backoff);
      if (backoff < 4096) backoff <<= 1;
    }
    if (!ok) break;
  }
  if (got < p.n) {
    for (int i = 0; i < got; ++i) {
      unsigned int* w = &p.header[i]->lock[p.index[i]];
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(w), "r"(0u) : "memory");
    }
    st->failed = 1u;
    st->failed_rank = (unsigned)p.owner[got];
    st->held = 0u;
    if (p.status != nullptr) {
      volatile CommStatus* v = p.status;
      if (v->error == 0u) {
        v->peer = (unsigned)p.owner[got];
        v->want = 0ull;
        v->seen = 1ull;
        v->error = kCommTimeoutLock;
        __threadfence_system();
      }
    }
  } else {
    st->held = (unsigned)p.n;
  }
  __threadfence_system();
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

int VecElems(int elem_type) { return 16 / ElemSize(elem_type); }

}  // namespace

cudaError_t LaunchWinPut(const WinPutParams& p, cudaStream_t stream) {
  const int grid = Grid(p.numel / VecElems(p.elem_type) + 1);
  BFB_DISPATCH_WIN(win_put_kernel, grid, stream, p);
  CountKernelLaunch();
  return cudaGetLastError();
}

cudaError_t LaunchWinGet(const WinGetParams& p, cudaStream_t stream) {
  const int grid = Grid(p.numel / VecElems(p.elem_type) + 1);
  BFB_DISPATCH_WIN(win_get_kernel, grid, stream, p);
  CountKernelLaunch();
  return cudaGetLastError();
}

cudaError_t LaunchWinUpdate(const WinUpdateParams& p, cudaStream_t stream) {
  const int grid = Grid(p.numel / VecElems(p.elem_type) + 1);
  BFB_DISPATCH_WIN(win_update_kernel, grid, stream, p);
  CountKernelLaunch();
  return cudaGetLastError();
}

cudaError_t LaunchWinLock(const WinLockParams& p, cudaStream_t stream) {
  if (p.n < 0 || p.n > kMaxWinPeers || p.state == nullptr) return cudaErrorInvalidValue;
  win_lock_kernel<<<1, 32, 0, stream>>>(p);
  CountKernelLaunch();
  return cudaGetLastError();
}

}  // namespace bfb
