// Peer-memory communication kernels for sm_100a (see comm_kernels.h for the protocol).
//
// Remote payloads are read with 16-byte `ld.relaxed.sys` loads that go straight over
// NVLink to the owner's HBM; flags use `ld.acquire.sys` / `st.release.sys` /
// `red.release.sys`.  No TMA and no cluster multicast is used anywhere in this file.
#include "comm_kernels.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <atomic>

namespace bfb {

namespace {

std::atomic<unsigned long long> g_launches{0};

constexpr int kThreads = 512;
constexpr int kUnroll = 4;
constexpr unsigned long long kMaxSpinIters = 1ull << 28;

// ------------------------------------------------------------------------------------ //
// memory-model primitives
// ------------------------------------------------------------------------------------ //
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void red_add_release_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ double ld_relaxed_sys_f64(const double* p) {
  double v;
  asm volatile("ld.relaxed.sys.global.f64 %0, [%1];" : "=d"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_peer_v4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Bounded wait until *flag >= target. Returns false on timeout (time or iteration limit).
__device__ bool wait_ge(const unsigned long long* flag, unsigned long long target,
                        unsigned long long timeout_ns, unsigned long long* seen) {
  unsigned long long v = ld_acquire_sys(flag);
  if (v >= target) return true;
  const unsigned long long t0 = globaltimer_ns();
  unsigned backoff = 32;
  for (unsigned long long it = 0; it < kMaxSpinIters; ++it) {
    v = ld_acquire_sys(flag);
    if (v >= target) return true;
    // the timer is a slow read next to a poll: look at it once per eight polls
    if ((it & 7ull) == 7ull && globaltimer_ns() - t0 > timeout_ns) break;
    __nanosleep(backoff);
    if (backoff < 2048) backoff <<= 1;
  }
  *seen = v;
  return false;
}

__device__ void report_error(CommStatus* st, unsigned code, unsigned peer, unsigned long long want,
                             unsigned long long seen) {
  if (st == nullptr) return;
  // Plain stores into pinned host memory: several blocks may report the same failure, the
  // fields they write agree up to the observed value, so no atomic is needed.
  volatile CommStatus* v = st;
  if (v->error == 0u) {
    v->peer = peer;
    v->want = want;
    v->seen = seen;
    v->error = code;
    __threadfence_system();
  }
}

// Returns true for exactly one block: the last one of the grid to arrive.  All threads
// must call it after their global writes; it contains the fences that make those writes
// visible before the caller publishes a flag.
__device__ bool grid_last_block(unsigned int* counter) {
  __shared__ bool is_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned int prev = atomicAdd(counter, 1u);
    is_last = (prev == gridDim.x - 1);
    if (is_last) *counter = 0;  // re-arm for the next launch (stream ordered)
    __threadfence_system();
  }
  __syncthreads();
  return is_last;
}

// Every block waits for the sources' epochs; weights (including the owners' per-destination
// weights) are left in shared memory. Returns false if any wait timed out.
template <typename W>
__device__ bool pull_prologue(const PullSync& s, const W* host_w, int n_w, W* smem_w) {
  __shared__ int ok;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  for (int j = threadIdx.x; j < s.n_src; j += blockDim.x) {
    unsigned long long seen = 0;
    if (!wait_ge(&s.src_ctrl[j]->epoch, s.wait_epoch, s.timeout_ns, &seen)) {
      report_error(s.status, kCommTimeoutEpoch, (unsigned)s.src_rank[j], s.wait_epoch, seen);
      ok = 0;
    } else if (ld_acquire_sys(&s.src_ctrl[j]->failed_epoch) == s.wait_epoch) {
      // the owner gave up while producing this version: its payload is not to be combined
      report_error(s.status, kCommPeerFailed, (unsigned)s.src_rank[j], s.wait_epoch, s.wait_epoch);
      ok = 0;
    }
    if (ok && s.use_dst_weight == 2 && !wait_ge(&s.src_ctrl[j]->weight_epoch, s.wait_epoch, s.timeout_ns, &seen)) {
      report_error(s.status, kCommTimeoutEpoch, (unsigned)s.src_rank[j], s.wait_epoch, seen);
      ok = 0;
    }
    W w = (j < n_w) ? host_w[j] : W(1);
    if (s.use_dst_weight)
      w = w * (W)ld_relaxed_sys_f64(&s.src_ctrl[j]->dst_weight[s.half][s.my_rank]);
    smem_w[j] = w;
  }
  __syncthreads();
  return ok != 0;
}

__device__ void pull_epilogue(const PullSync& s) {
  if (!s.signal_done) {
    // still contributes nothing to the counter: other launches of the round do not count
    return;
  }
  if (grid_last_block(&s.my_ctrl->block_counter[s.counter_slot])) {
    for (int j = threadIdx.x; j < s.n_src; j += blockDim.x)
      red_add_release_sys(&s.src_ctrl[j]->done[s.half], 1ull);
  }
}

__device__ __forceinline__ int find_segment(const unsigned long long* starts, int n, unsigned long long c) {
  int lo = 0, hi = n - 1;
  while (lo < hi) {
    int mid = (lo + hi + 1) >> 1;
    if (starts[mid] <= c) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// ------------------------------------------------------------------------------------ //
// element traits: 16-byte vectors <-> accumulator arrays
// ------------------------------------------------------------------------------------ //
template <typename T> struct Elem;
template <> struct Elem<float> {
  using Acc = float; static constexpr int N = 4;
  static __device__ void unpack(const uint4& v, Acc* a) { a[0] = __uint_as_float(v.x); a[1] = __uint_as_float(v.y); a[2] = __uint_as_float(v.z); a[3] = __uint_as_float(v.w); }
  static __device__ uint4 pack(const Acc* a) { return make_uint4(__float_as_uint(a[0]), __float_as_uint(a[1]), __float_as_uint(a[2]), __float_as_uint(a[3])); }
  static __device__ Acc load(const float* p) { return *p; }
  static __device__ void store(float* p, Acc a) { *p = a; }
};
template <> struct Elem<double> {
  using Acc = double; static constexpr int N = 2;
  static __device__ void unpack(const uint4& v, Acc* a) { a[0] = __hiloint2double(v.y, v.x); a[1] = __hiloint2double(v.w, v.z); }
  static __device__ uint4 pack(const Acc* a) { return make_uint4(__double2loint(a[0]), __double2hiint(a[0]), __double2loint(a[1]), __double2hiint(a[1])); }
  static __device__ Acc load(const double* p) { return *p; }
  static __device__ void store(double* p, Acc a) { *p = a; }
};
template <> struct Elem<__half> {
  using Acc = float; static constexpr int N = 8;
  static __device__ void unpack(const uint4& v, Acc* a) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 f = __half22float2(h[i]); a[2 * i] = f.x; a[2 * i + 1] = f.y; }
  }
  static __device__ uint4 pack(const Acc* a) {
    uint4 v; __half2* h = reinterpret_cast<__half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(a[2 * i], a[2 * i + 1]);
    return v;
  }
  static __device__ Acc load(const __half* p) { return __half2float(*p); }
  static __device__ void store(__half* p, Acc a) { *p = __float2half_rn(a); }
};
template <> struct Elem<__nv_bfloat16> {
  using Acc = float; static constexpr int N = 8;
  static __device__ void unpack(const uint4& v, Acc* a) {
    const unsigned* u = reinterpret_cast<const unsigned*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) { a[2 * i] = __uint_as_float(u[i] << 16); a[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u); }
  }
  static __device__ uint4 pack(const Acc* a) {
    uint4 v; __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(a[2 * i], a[2 * i + 1]);
    return v;
  }
  static __device__ Acc load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  static __device__ void store(__nv_bfloat16* p, Acc a) { *p = __float2bfloat16_rn(a); }
};
template <> struct Elem<int> {
  using Acc = long long; static constexpr int N = 4;
  static __device__ void unpack(const uint4& v, Acc* a) { a[0] = (int)v.x; a[1] = (int)v.y; a[2] = (int)v.z; a[3] = (int)v.w; }
  static __device__ uint4 pack(const Acc* a) { return make_uint4((unsigned)(int)a[0], (unsigned)(int)a[1], (unsigned)(int)a[2], (unsigned)(int)a[3]); }
  static __device__ Acc load(const int* p) { return *p; }
  static __device__ void store(int* p, Acc a) { *p = (int)a; }
};
template <> struct Elem<long long> {
  using Acc = long long; static constexpr int N = 2;
  static __device__ void unpack(const uint4& v, Acc* a) {
    a[0] = (long long)(((unsigned long long)v.y << 32) | v.x); a[1] = (long long)(((unsigned long long)v.w << 32) | v.z);
  }
  static __device__ uint4 pack(const Acc* a) {
    return make_uint4((unsigned)a[0], (unsigned)((unsigned long long)a[0] >> 32), (unsigned)a[1], (unsigned)((unsigned long long)a[1] >> 32));
  }
  static __device__ Acc load(const long long* p) { return *p; }
  static __device__ void store(long long* p, Acc a) { *p = a; }
};

// Weight type used for the multiply-accumulate: double for fp64 payloads and for
// integers (so that an exact integer sum with weight 1 stays exact), float otherwise.
template <typename T> struct WeightOf { using type = float; };
template <> struct WeightOf<double> { using type = double; };
template <> struct WeightOf<int> { using type = double; };
template <> struct WeightOf<long long> { using type = double; };

template <typename Acc, typename W>
__device__ __forceinline__ Acc mul_w(Acc a, W w) { return (Acc)(a * w); }
template <>
__device__ __forceinline__ long long mul_w<long long, double>(long long a, double w) {
  return w == 1.0 ? a : (long long)((double)a * w);
}

// ------------------------------------------------------------------------------------ //
// pack + publish
// ------------------------------------------------------------------------------------ //
__global__ void __launch_bounds__(kThreads) pack_publish_kernel(const __grid_constant__ PackParams p) {
  __shared__ int ok;
  __shared__ unsigned long long starts[kMaxSeg + 1];
  if (threadIdx.x == 0) {
    ok = 1;
    if (p.wait_done) {
      unsigned long long seen = 0;
      if (!wait_ge(&p.ctrl->done[p.half], p.need_done, p.timeout_ns, &seen)) {
        report_error(p.status, kCommTimeoutDone, (unsigned)p.my_rank, p.need_done, seen);
        ok = 0;
        atomicExch(&p.ctrl->launch_failed, 1u);     // later launches of this version skip their copies too
      }
    } else if (*reinterpret_cast<volatile unsigned int*>(&p.ctrl->launch_failed) != 0u) {
      ok = 0;
    }
  }
  for (int i = threadIdx.x; i <= p.n_seg; i += blockDim.x) starts[i] = p.chunk_start[i];
  __syncthreads();
  if (ok) {
    const unsigned long long total = starts[p.n_seg];
    const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
    for (unsigned long long c = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; c < total; c += stride) {
      const int s = find_segment(starts, p.n_seg, c);
      const unsigned long long l = c - starts[s];
      const unsigned char* src = static_cast<const unsigned char*>(p.src[s]) + l * 16;
      unsigned char* dst = p.arena_half + p.dst_off[s] + l * 16;
      const unsigned long long left = p.nbytes[s] - l * 16;
      if (left >= 16 && ((reinterpret_cast<uintptr_t>(src) & 15) == 0)) {
        *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
      } else {
        const int n = left < 16 ? (int)left : 16;
        for (int b = 0; b < n; ++b) dst[b] = src[b];
      }
    }
  }
  if (p.publish) {
    if (grid_last_block(&p.ctrl->block_counter[0])) {
      if (p.has_dst_weight)
        for (int r = threadIdx.x; r < p.world; r += blockDim.x) p.ctrl->dst_weight[p.half][r] = p.dst_weight[r];
      if (threadIdx.x == 0) {
        p.ctrl->payload_bytes[p.half] = p.payload_bytes;
        p.ctrl->payload_loc[p.half] = p.loc;
        // a version that was not written completely is still announced (nobody may hang on it), but marked
        if (*reinterpret_cast<volatile unsigned int*>(&p.ctrl->launch_failed) != 0u) {
          p.ctrl->failed_epoch = p.publish_epoch;
          p.ctrl->launch_failed = 0u;
        }
      }
      __threadfence_system();
      __syncthreads();
      if (threadIdx.x == 0) st_release_sys(&p.ctrl->epoch, p.publish_epoch);
    }
  }
}

// ------------------------------------------------------------------------------------ //
// pull + weighted combine
// ------------------------------------------------------------------------------------ //
template <typename T>
__global__ void __launch_bounds__(kThreads) combine_kernel(const __grid_constant__ CombineParams p) {
  using E = Elem<T>;
  using Acc = typename E::Acc;
  using W = typename WeightOf<T>::type;
  constexpr int N = E::N;
  __shared__ W w_s[kMaxSrc];
  __shared__ W w_host[kMaxSrc];
  __shared__ unsigned long long starts[kMaxSeg + 1];
  for (int j = threadIdx.x; j < p.sync.n_src; j += blockDim.x) w_host[j] = (W)p.src_w[j];
  for (int i = threadIdx.x; i <= p.n_seg; i += blockDim.x) starts[i] = p.chunk_start[i];
  __syncthreads();
  bool ok = pull_prologue<W>(p.sync, w_host, p.sync.n_src, w_s);
  // where each source keeps this version: in its arena, or in place in registered memory
  __shared__ const unsigned char* base_s[kMaxSrc];
  __shared__ int layout_ok;
  if (threadIdx.x == 0) layout_ok = 1;
  __syncthreads();
  if (ok) {
    for (int j = threadIdx.x; j < p.sync.n_src; j += blockDim.x) {
      const unsigned long long loc = ld_acquire_sys(&p.sync.src_ctrl[j]->payload_loc[p.sync.half]);
      const unsigned long long have = ld_acquire_sys(&p.sync.src_ctrl[j]->payload_bytes[p.sync.half]);
      if (have < p.need_bytes) {
        report_error(p.sync.status, kCommLayoutMismatch, (unsigned)p.sync.src_rank[j], p.need_bytes, have);
        layout_ok = 0;
      } else if (loc == 0ull) {
        base_s[j] = p.sync.src_arena[j];
      } else if (loc == p.my_loc) {
        base_s[j] = p.alt_src[j];
      } else {
        report_error(p.sync.status, kCommLayoutMismatch, (unsigned)p.sync.src_rank[j], p.my_loc, loc);
        layout_ok = 0;
      }
    }
  }
  __syncthreads();
  ok = ok && layout_ok != 0;
  if (ok) {
    const W self_w = (W)p.self_w;
    const W post = (W)p.post_scale;
    const bool has_post = p.post_scale != 1.0;
    const int n_src = p.sync.n_src;
    const unsigned long long total = starts[p.n_seg];
    const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
    for (unsigned long long c0 = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; c0 < total;
         c0 += stride * kUnroll) {
      unsigned long long boff[kUnroll];   // byte offset inside an arena half
      int seg[kUnroll];
      int cnt[kUnroll];                   // valid elements in this chunk (0 = no chunk)
      Acc acc[kUnroll][N];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const unsigned long long c = c0 + (unsigned long long)u * stride;
        cnt[u] = 0;
        seg[u] = 0;
        boff[u] = 0;
        if (c < total) {
          const int s = find_segment(starts, p.n_seg, c);
          const unsigned long long l = c - starts[s];
          const unsigned long long left = p.numel[s] - l * N;
          seg[u] = s;
          cnt[u] = left >= (unsigned long long)N ? N : (int)left;
          boff[u] = p.off[s] + l * 16;
        }
      }
      // self term (local memory). Arena segments start on 16-byte boundaries and are padded,
      // so a full 16-byte read of the last chunk stays inside the arena.
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        if (cnt[u] > 0 && p.self_arena != nullptr) {
          uint4 v = *reinterpret_cast<const uint4*>(p.self_arena + boff[u]);
          E::unpack(v, acc[u]);
#pragma unroll
          for (int i = 0; i < N; ++i) acc[u][i] = mul_w<Acc, W>(acc[u][i], self_w);
        } else {
#pragma unroll
          for (int i = 0; i < N; ++i) acc[u][i] = Acc(0);
        }
      }
      for (int j = 0; j < n_src; ++j) {
        const unsigned char* base = base_s[j];
        const W w = w_s[j];
        uint4 v[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
          if (cnt[u] > 0) v[u] = ld_peer_v4(base + boff[u]);
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          if (cnt[u] > 0) {
            Acc t[N];
            E::unpack(v[u], t);
#pragma unroll
            for (int i = 0; i < N; ++i) acc[u][i] += mul_w<Acc, W>(t[i], w);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        if (cnt[u] == 0) continue;
        if (has_post) {
#pragma unroll
          for (int i = 0; i < N; ++i) acc[u][i] = mul_w<Acc, W>(acc[u][i], post);
        }
        const int s = seg[u];
        const unsigned long long l = (boff[u] - p.off[s]) / 16;
        T* out = static_cast<T*>(p.out[s]) + l * N;
        if (cnt[u] == N && ((reinterpret_cast<uintptr_t>(out) & 15) == 0)) {
          *reinterpret_cast<uint4*>(out) = E::pack(acc[u]);
        } else {
#pragma unroll
          for (int i = 0; i < N; ++i)
            if (i < cnt[u]) E::store(out + i, acc[u][i]);
        }
      }
    }
  }
  pull_epilogue(p.sync);
}

// ------------------------------------------------------------------------------------ //
// pull + plain copy (allgather, neighbor_allgather, broadcast)
// ------------------------------------------------------------------------------------ //
__global__ void __launch_bounds__(kThreads) gather_kernel(const __grid_constant__ GatherParams p) {
  __shared__ float w_s[kMaxSrc];
  __shared__ unsigned long long starts[kMaxSeg + 1];
  for (int i = threadIdx.x; i <= p.n_copy; i += blockDim.x) starts[i] = p.chunk_start[i];
  __syncthreads();
  const bool ok = pull_prologue<float>(p.sync, nullptr, 0, w_s);
  if (ok) {
    const unsigned long long total = starts[p.n_copy];
    const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
    for (unsigned long long c = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; c < total; c += stride) {
      const int s = find_segment(starts, p.n_copy, c);
      const unsigned long long l = c - starts[s];
      const int js = p.copy_src[s];
      const unsigned char* src = (js < 0 ? p.self_arena : p.sync.src_arena[js]) + p.src_off[s] + l * 16;
      unsigned char* dst = static_cast<unsigned char*>(p.out[s]) + l * 16;
      const unsigned long long left = p.nbytes[s] - l * 16;
      // Source chunks are 16-byte aligned and padded inside the arena: always one vector load.
      uint4 v = (js < 0) ? *reinterpret_cast<const uint4*>(src) : ld_peer_v4(src);
      if (left >= 16 && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
        *reinterpret_cast<uint4*>(dst) = v;
      } else {
        const unsigned char* b = reinterpret_cast<const unsigned char*>(&v);
        const int n = left < 16 ? (int)left : 16;
        for (int i = 0; i < n; ++i) dst[i] = b[i];
      }
    }
  }
  pull_epilogue(p.sync);
}

// ------------------------------------------------------------------------------------ //
// fused bucket step: neighbor combine + optimizer update + casts, one pass over the bucket
// ------------------------------------------------------------------------------------ //
struct OptConst {
  int opt, nesterov, adamw, amsgrad, first_step, maximize;
  float lr, momentum, dampening, wd, beta1, beta2, eps, bias1, bias2;
};

// Applies one optimizer update to parameter value c with gradient g. Returns the new value.  The optimizer state of
// the element (s1: momentum buffer or first moment, s2: second moment, s3: running maximum of the second moment)
// lives in registers: the caller moves it as 16-byte vectors.  Through pointers every store of an element's state
// would order the loads of the next element behind it, four dependent memory round trips per 16 bytes.
__device__ __forceinline__ float opt_update(const OptConst& o, float c, float g, float& s1, float& s2, float& s3) {
  if (o.maximize) g = -g;
  if (o.opt == kOptSGD) {
    float d = g + o.wd * c;
    if (o.momentum != 0.f) {
      float buf = o.first_step ? d : o.momentum * s1 + (1.f - o.dampening) * d;
      s1 = buf;
      d = o.nesterov ? d + o.momentum * buf : buf;
    }
    return c - o.lr * d;
  }
  if (o.opt == kOptAdam) {
    if (o.adamw) c = c * (1.f - o.lr * o.wd); else g = g + o.wd * c;
    float m = o.beta1 * s1 + (1.f - o.beta1) * g;
    float v = o.beta2 * s2 + (1.f - o.beta2) * g * g;
    s1 = m;
    s2 = v;
    float vhat = v;
    if (o.amsgrad) { vhat = fmaxf(s3, v); s3 = vhat; }
    // correctly rounded square root and division whatever the build's fast-math setting: v is tiny early in training
    const float denom = __fdiv_rn(__fsqrt_rn(vhat), __fsqrt_rn(o.bias2)) + o.eps;
    return c - __fdiv_rn(o.lr, o.bias1) * __fdiv_rn(m, denom);
  }
  if (o.opt == kOptRMSprop) {                       // torch.optim.RMSprop: beta2 = alpha, amsgrad = centered
    g = g + o.wd * c;
    const float sq = o.beta2 * s1 + (1.f - o.beta2) * g * g;
    s1 = sq;
    float avg;
    if (o.amsgrad) {
      const float ga = o.beta2 * s3 + (1.f - o.beta2) * g;
      s3 = ga;
      avg = __fsqrt_rn(sq - ga * ga);
    } else {
      avg = __fsqrt_rn(sq);
    }
    avg += o.eps;
    if (o.momentum > 0.f) {
      const float buf = o.momentum * s2 + __fdiv_rn(g, avg);
      s2 = buf;
      return c - o.lr * buf;
    }
    return c - o.lr * __fdiv_rn(g, avg);
  }
  if (o.opt == kOptAdagrad) {                       // torch.optim.Adagrad: lr is the decayed rate of this step
    g = g + o.wd * c;
    const float sum = s1 + g * g;
    s1 = sum;
    return c - o.lr * __fdiv_rn(g, __fsqrt_rn(sum) + o.eps);
  }
  if (o.opt == kOptAdadelta) {                      // torch.optim.Adadelta: beta2 = rho
    g = g + o.wd * c;
    const float sq = o.beta2 * s1 + (1.f - o.beta2) * g * g;
    s1 = sq;
    const float delta = __fdiv_rn(__fsqrt_rn(s2 + o.eps), __fsqrt_rn(sq + o.eps)) * g;
    s2 = o.beta2 * s2 + (1.f - o.beta2) * delta * delta;
    return c - o.lr * delta;
  }
  return c;
}

// Four consecutive floats starting at a 16-byte boundary; `cnt` < 4 only in the last step of a buffer.
__device__ __forceinline__ void load4f(const float* __restrict__ p, int cnt, float* v) {
  if (cnt == 4) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = i < cnt ? p[i] : 0.f;
  }
}
__device__ __forceinline__ void store4f(float* __restrict__ p, int cnt, const float* v) {
  if (cnt == 4) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (i < cnt) p[i] = v[i];
  }
}
// Up to four gradient elements, scaled; one vector load when all four exist and the address allows it.
template <typename GradT>
__device__ __forceinline__ void load4g(const GradT* __restrict__ gp, unsigned long long have, float scale, float* g) {
  if (have >= 4 && (reinterpret_cast<uintptr_t>(gp) & (4 * sizeof(GradT) - 1)) == 0) {
    if (sizeof(GradT) == 4) {
      const float4 t = *reinterpret_cast<const float4*>(gp);
      g[0] = t.x * scale; g[1] = t.y * scale; g[2] = t.z * scale; g[3] = t.w * scale;
    } else {
      const uint2 t = *reinterpret_cast<const uint2*>(gp);
      g[0] = __uint_as_float(t.x << 16) * scale; g[1] = __uint_as_float(t.x & 0xffff0000u) * scale;
      g[2] = __uint_as_float(t.y << 16) * scale; g[3] = __uint_as_float(t.y & 0xffff0000u) * scale;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) g[i] = (unsigned long long)i < have ? Elem<GradT>::load(gp + i) * scale : 0.f;
  }
}

template <typename PubT, typename GradT>
__global__ void __launch_bounds__(kThreads) bucket_step_kernel(const __grid_constant__ BucketParams p) {
  using PE = Elem<PubT>;
  using GE = Elem<GradT>;
  __shared__ float w_s[kMaxSrc];
  __shared__ float w_host[kMaxSrc];
  __shared__ int okd;
  const bool reads_peers = (p.mode == kModeAWC || p.mode == kModeCombineOnly || p.mode == kModeGradReduce);
  bool ok = true;
  if (p.dst_weight_mode == 2 && blockIdx.x == 0) {
    // the weights this rank attaches to the version its neighbors pull in this step, announced before any wait
    for (int r = threadIdx.x; r < p.world; r += blockDim.x) p.sync.my_ctrl->dst_weight[p.sync.half][r] = (double)p.dst_weight[r];
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) st_release_sys(&p.sync.my_ctrl->weight_epoch, p.sync.wait_epoch);
  }
  if (p.mode == kModeAnnounceWeights) return;
  if (reads_peers) {
    for (int j = threadIdx.x; j < p.sync.n_src; j += blockDim.x) w_host[j] = p.src_w[j];
    __syncthreads();
    ok = pull_prologue<float>(p.sync, w_host, p.sync.n_src, w_s);
  }
  if (p.pub_write != nullptr && p.wait_done) {
    if (threadIdx.x == 0) {
      okd = 1;
      unsigned long long seen = 0;
      if (!wait_ge(&p.sync.my_ctrl->done[p.write_half], p.need_done, p.sync.timeout_ns, &seen)) {
        report_error(p.sync.status, kCommTimeoutDone, (unsigned)p.sync.my_rank, p.need_done, seen);
        okd = 0;
      }
    }
    __syncthreads();
    ok = ok && (okd != 0);
  }
  if (ok) {
    OptConst o{p.opt, p.nesterov, p.adamw, p.amsgrad, p.first_step, p.maximize, p.lr, p.momentum, p.dampening,
               p.weight_decay, p.beta1, p.beta2, p.eps, p.bias1, p.bias2};
    const int n_src = reads_peers ? p.sync.n_src : 0;
    const unsigned long long n4 = p.numel / 4;
    const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
    const int mode = p.mode;
    const bool any_grad = p.grad != nullptr || p.grad_ptrs != nullptr;
    const bool has_grad = any_grad && p.opt != kOptNone;
    const bool wants_grad = any_grad && (has_grad || mode == kModeGradReduce || mode == kModePublishOnly);
    // which state arrays the optimizer reads (ld) and writes (st)
    const bool st1 = (o.opt == kOptSGD && o.momentum != 0.f) || o.opt >= kOptAdam;
    const bool ld1 = st1 && !(o.opt == kOptSGD && o.first_step);
    const bool st2 = o.opt == kOptAdam || o.opt == kOptAdadelta || (o.opt == kOptRMSprop && o.momentum > 0.f);
    const bool st3 = (o.opt == kOptAdam || o.opt == kOptRMSprop) && o.amsgrad;
    // Main loop: 4 elements per thread per step; published/grad buffers are padded to 16 bytes.
    for (unsigned long long q = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; q * 4 < p.numel; q += stride) {
      const unsigned long long i0 = q * 4;
      const int cnt = (q < n4) ? 4 : (int)(p.numel - i0);
      float x[4], g[4], acc[4];
      // local master
      if (p.master == nullptr) {
        for (int i = 0; i < 4; ++i) x[i] = 0.f;
      } else if (cnt == 4) {
        float4 m = *reinterpret_cast<const float4*>(p.master + i0);
        x[0] = m.x; x[1] = m.y; x[2] = m.z; x[3] = m.w;
      } else {
        for (int i = 0; i < 4; ++i) x[i] = i < cnt ? p.master[i0 + i] : 0.f;
      }
      // gradient.  A parameter of the table without a gradient (frozen, or unused in this step) takes no optimizer
      // update at all - no weight decay, no decay of its moments - as torch.optim skips it.
      bool seg_has_grad = true;
      for (int i = 0; i < 4; ++i) g[i] = 0.f;
      if (wants_grad) {
        if (p.grad != nullptr) {
          load4g<GradT>(static_cast<const GradT*>(p.grad) + i0, (unsigned long long)cnt, p.grad_scale, g);
        } else {
          // per-parameter gradients: parameters start at multiples of 4 elements, so the four
          // elements of this step belong to one parameter (or to the padding behind it)
          int lo = 0, hi = p.n_seg - 1;
          while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (p.seg_start[mid] <= i0) lo = mid; else hi = mid - 1;
          }
          const GradT* gp = static_cast<const GradT*>(p.grad_ptrs[lo]);
          const unsigned long long local = i0 - p.seg_start[lo];
          const unsigned long long n = p.seg_numel[lo];
          if (gp != nullptr)
            load4g<GradT>(gp + local, local < n ? n - local : 0ull, p.grad_scale, g);
          else
            seg_has_grad = false;
        }
      }
      // optimizer state of these four elements, requested before the peers' terms so that all loads of the step
      // are in flight together
      const bool upd = has_grad && seg_has_grad;
      const bool touch = (mode == kModeGradReduce) ? true : (upd && (mode == kModeAWC || mode == kModeAdaptPublish));
      float s1[4] = {0.f, 0.f, 0.f, 0.f}, s2[4] = {0.f, 0.f, 0.f, 0.f}, s3[4] = {0.f, 0.f, 0.f, 0.f};
      if (touch) {
        if (ld1) load4f(p.state1 + i0, cnt, s1);
        if (st2) load4f(p.state2 + i0, cnt, s2);
        if (st3) load4f(p.state3 + i0, cnt, s3);
      }
      // remote terms
      if (mode == kModeAWC || mode == kModeCombineOnly) {
        // the own term comes from the fp32 master in both modes (after the adapt half of adapt-then-combine
        // the master holds the adapted value), so a 16-bit exchange format only rounds the neighbors' terms
        for (int i = 0; i < 4; ++i) acc[i] = p.self_w * x[i];
      } else if (mode == kModeGradReduce) {
        for (int i = 0; i < 4; ++i) acc[i] = g[i];
      } else {
        for (int i = 0; i < 4; ++i) acc[i] = 0.f;
      }
      for (int j = 0; j < n_src; ++j) {
        const PubT* rp = reinterpret_cast<const PubT*>(p.sync.src_arena[j]) + i0;
        const float w = w_s[j];
        if (sizeof(PubT) == 4) {
          uint4 v = ld_peer_v4(rp);
          acc[0] += w * __uint_as_float(v.x); acc[1] += w * __uint_as_float(v.y);
          acc[2] += w * __uint_as_float(v.z); acc[3] += w * __uint_as_float(v.w);
        } else {
          // 4 x 16-bit = 8 bytes
          uint2 v;
          asm volatile("ld.relaxed.sys.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(rp) : "memory");
          acc[0] += w * __uint_as_float(v.x << 16); acc[1] += w * __uint_as_float(v.x & 0xffff0000u);
          acc[2] += w * __uint_as_float(v.y << 16); acc[3] += w * __uint_as_float(v.y & 0xffff0000u);
        }
      }
      float y[4];
      if (mode == kModeAWC) {
        for (int i = 0; i < 4; ++i) y[i] = (upd && i < cnt) ? opt_update(o, acc[i], g[i], s1[i], s2[i], s3[i]) : acc[i];
      } else if (mode == kModeAdaptPublish) {
        for (int i = 0; i < 4; ++i) y[i] = (upd && i < cnt) ? opt_update(o, x[i], g[i], s1[i], s2[i], s3[i]) : x[i];
      } else if (mode == kModeCombineOnly) {
        for (int i = 0; i < 4; ++i) y[i] = acc[i];
      } else if (mode == kModeGradReduce) {
        for (int i = 0; i < 4; ++i) y[i] = i < cnt ? opt_update(o, x[i], acc[i] * p.post_scale, s1[i], s2[i], s3[i]) : 0.f;
      } else {  // publish only: payload is the master (or the gradient when grad != null and opt == none)
        for (int i = 0; i < 4; ++i) y[i] = any_grad ? g[i] : x[i];
      }
      if (touch) {
        if (st1) store4f(p.state1 + i0, cnt, s1);
        if (st2) store4f(p.state2 + i0, cnt, s2);
        if (st3) store4f(p.state3 + i0, cnt, s3);
      }
      const bool writes_master = (mode == kModeAWC || mode == kModeCombineOnly || mode == kModeGradReduce ||
                                  (mode == kModeAdaptPublish && p.master != nullptr));
      if (writes_master) {
        if (cnt == 4) *reinterpret_cast<float4*>(p.master + i0) = make_float4(y[0], y[1], y[2], y[3]);
        else for (int i = 0; i < cnt; ++i) p.master[i0 + i] = y[i];
        // the shadow is what the next forward pass reads: only the final value of the step goes there
        if (p.shadow != nullptr && mode != kModeAdaptPublish) {
          __nv_bfloat16* sh = static_cast<__nv_bfloat16*>(p.shadow) + i0;
          if (cnt == 4) {
            __nv_bfloat162 a = __floats2bfloat162_rn(y[0], y[1]), b = __floats2bfloat162_rn(y[2], y[3]);
            uint2 pk = make_uint2(*reinterpret_cast<unsigned*>(&a), *reinterpret_cast<unsigned*>(&b));
            *reinterpret_cast<uint2*>(sh) = pk;
          } else {
            for (int i = 0; i < cnt; ++i) sh[i] = __float2bfloat16_rn(y[i]);
          }
        }
      }
      if (p.pub_write != nullptr && mode != kModeCombineOnly) {
        PubT* wp = reinterpret_cast<PubT*>(p.pub_write) + i0;
        // padded to a multiple of 4 elements: full-width store is always in bounds
        if (sizeof(PubT) == 4) {
          *reinterpret_cast<float4*>(wp) = make_float4(y[0], y[1], y[2], y[3]);
        } else {
          __nv_bfloat162 a = __floats2bfloat162_rn(y[0], y[1]), b = __floats2bfloat162_rn(y[2], y[3]);
          *reinterpret_cast<uint2*>(wp) = make_uint2(*reinterpret_cast<unsigned*>(&a), *reinterpret_cast<unsigned*>(&b));
        }
      }
    }
  }
  // Tail: publish my new version and release the sources.  A block whose wait ran out has not written its part
  // of the new version: the version is announced all the same (a neighbor must never hang on it) but marked as
  // failed, so that readers report an error instead of combining it.
  const bool need_tail = p.publish || (reads_peers && p.sync.signal_done);
  if (need_tail) {
    if (!ok && threadIdx.x == 0) atomicExch(&p.sync.my_ctrl->launch_failed, 1u);
    if (grid_last_block(&p.sync.my_ctrl->block_counter[p.sync.counter_slot])) {
      if (p.publish) {
        if (p.dst_weight_mode == 1)
          for (int r = threadIdx.x; r < p.world; r += blockDim.x)
            p.sync.my_ctrl->dst_weight[p.write_half][r] = (double)p.dst_weight[r];
        if (threadIdx.x == 0 && *reinterpret_cast<volatile unsigned int*>(&p.sync.my_ctrl->launch_failed) != 0u) {
          p.sync.my_ctrl->failed_epoch = p.publish_epoch;
          p.sync.my_ctrl->launch_failed = 0u;
        }
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x == 0) st_release_sys(&p.sync.my_ctrl->epoch, p.publish_epoch);
      } else if (threadIdx.x == 0) {
        p.sync.my_ctrl->launch_failed = 0u;
      }
      if (reads_peers && p.sync.signal_done)
        for (int j = threadIdx.x; j < p.sync.n_src; j += blockDim.x)
          red_add_release_sys(&p.sync.src_ctrl[j]->done[p.sync.half], 1ull);
    }
  }
}

// ------------------------------------------------------------------------------------ //
// scale
// ------------------------------------------------------------------------------------ //
template <typename T>
__global__ void __launch_bounds__(kThreads) scale_kernel(T* buf, unsigned long long numel, double s) {
  using E = Elem<T>;
  using Acc = typename E::Acc;
  using W = typename WeightOf<T>::type;
  constexpr int N = E::N;
  const W w = (W)s;
  const unsigned long long nvec = numel / N;
  const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
  const unsigned long long tid = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
  if ((reinterpret_cast<uintptr_t>(buf) & 15) == 0) {
    for (unsigned long long q = tid; q < nvec; q += stride) {
      Acc a[N];
      uint4 v = reinterpret_cast<uint4*>(buf)[q];
      E::unpack(v, a);
#pragma unroll
      for (int i = 0; i < N; ++i) a[i] = mul_w<Acc, W>(a[i], w);
      reinterpret_cast<uint4*>(buf)[q] = E::pack(a);
    }
    for (unsigned long long i = nvec * N + tid; i < numel; i += stride) E::store(buf + i, mul_w<Acc, W>(E::load(buf + i), w));
  } else {
    for (unsigned long long i = tid; i < numel; i += stride) E::store(buf + i, mul_w<Acc, W>(E::load(buf + i), w));
  }
}

int GridFor(unsigned long long work_items) {
  static int sms = [] {
    int dev = 0, n = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    return n > 0 ? n : 148;
  }();
  unsigned long long blocks = (work_items + kThreads - 1) / kThreads;
  unsigned long long cap = (unsigned long long)sms * 2;  // two 512-thread CTAs per SM, all co-resident
  if (blocks < 1) blocks = 1;
  return (int)(blocks < cap ? blocks : cap);
}

}  // namespace

int ElemSize(int t) {
  switch (t) {
    case kF32: case kI32: return 4;
    case kF64: case kI64: return 8;
    case kF16: case kBF16: case kI16: return 2;
    default: return 1;
  }
}

unsigned long long KernelLaunchCount() { return g_launches.load(); }
void CountKernelLaunch() { g_launches.fetch_add(1); }

cudaError_t LaunchPack(const PackParams& p, cudaStream_t stream) {
  const unsigned long long total = p.chunk_start[p.n_seg];
  pack_publish_kernel<<<GridFor(total), kThreads, 0, stream>>>(p);
  CountKernelLaunch();
  return cudaGetLastError();
}

__global__ void wait_readers_kernel(ChannelCtrl* ctrl, int half, unsigned long long need, unsigned long long timeout_ns,
                                    CommStatus* status, int my_rank) {
  unsigned long long seen = 0;
  if (!wait_ge(&ctrl->done[half], need, timeout_ns, &seen))
    report_error(status, kCommTimeoutDone, (unsigned)my_rank, need, seen);
}

cudaError_t LaunchWaitReaders(ChannelCtrl* ctrl, int half, unsigned long long need, unsigned long long timeout_ns,
                              CommStatus* status, int my_rank, cudaStream_t stream) {
  wait_readers_kernel<<<1, 1, 0, stream>>>(ctrl, half, need, timeout_ns, status, my_rank);
  CountKernelLaunch();
  return cudaGetLastError();
}

cudaError_t LaunchCombine(const CombineParams& p, cudaStream_t stream) {
  const unsigned long long total = p.chunk_start[p.n_seg];
  const int grid = GridFor((total + kUnroll - 1) / kUnroll);
  switch (p.elem_type) {
    case kF32: combine_kernel<float><<<grid, kThreads, 0, stream>>>(p); break;
    case kF64: combine_kernel<double><<<grid, kThreads, 0, stream>>>(p); break;
    case kF16: combine_kernel<__half><<<grid, kThreads, 0, stream>>>(p); break;
    case kBF16: combine_kernel<__nv_bfloat16><<<grid, kThreads, 0, stream>>>(p); break;
    case kI32: combine_kernel<int><<<grid, kThreads, 0, stream>>>(p); break;
    case kI64: combine_kernel<long long><<<grid, kThreads, 0, stream>>>(p); break;
    default: return cudaErrorInvalidValue;
  }
  CountKernelLaunch();
  return cudaGetLastError();
}

cudaError_t LaunchGather(const GatherParams& p, cudaStream_t stream) {
  const unsigned long long total = p.chunk_start[p.n_copy];
  gather_kernel<<<GridFor(total), kThreads, 0, stream>>>(p);
  CountKernelLaunch();
  return cudaGetLastError();
}

cudaError_t LaunchBucketStep(const BucketParams& p, cudaStream_t stream) {
  const int grid = GridFor((p.numel + 3) / 4);
  const bool pub_bf16 = p.pub_elem == kBF16;
  const bool grad_bf16 = p.grad_elem == kBF16;
  if (!pub_bf16 && !grad_bf16) bucket_step_kernel<float, float><<<grid, kThreads, 0, stream>>>(p);
  else if (!pub_bf16 && grad_bf16) bucket_step_kernel<float, __nv_bfloat16><<<grid, kThreads, 0, stream>>>(p);
  else if (pub_bf16 && !grad_bf16) bucket_step_kernel<__nv_bfloat16, float><<<grid, kThreads, 0, stream>>>(p);
  else bucket_step_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, kThreads, 0, stream>>>(p);
  CountKernelLaunch();
  return cudaGetLastError();
}

cudaError_t LaunchScale(void* buf, unsigned long long numel, double s, int elem_type, cudaStream_t stream) {
  if (numel == 0) return cudaSuccess;
  const int grid = GridFor(numel / 4 + 1);
  switch (elem_type) {
    case kF32: scale_kernel<float><<<grid, kThreads, 0, stream>>>(static_cast<float*>(buf), numel, s); break;
    case kF64: scale_kernel<double><<<grid, kThreads, 0, stream>>>(static_cast<double*>(buf), numel, s); break;
    case kF16: scale_kernel<__half><<<grid, kThreads, 0, stream>>>(static_cast<__half*>(buf), numel, s); break;
    case kBF16: scale_kernel<__nv_bfloat16><<<grid, kThreads, 0, stream>>>(static_cast<__nv_bfloat16*>(buf), numel, s); break;
    case kI32: scale_kernel<int><<<grid, kThreads, 0, stream>>>(static_cast<int*>(buf), numel, s); break;
    case kI64: scale_kernel<long long><<<grid, kThreads, 0, stream>>>(static_cast<long long*>(buf), numel, s); break;
    default: return cudaErrorInvalidValue;
  }
  CountKernelLaunch();
  return cudaGetLastError();
}

}  // namespace bfb
