// Allocation-free variant of the pull-combine kernel (see combine_noalloc.h).
#include "combine_noalloc.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <mutex>

#include "comm_kernels.h"

namespace {

constexpr int kMaxSources = BFB200_NOALLOC_MAX_SOURCES;
constexpr int kScratchBytes = BFB200_NOALLOC_SCRATCH_BYTES;
constexpr int kThreads = 512;
constexpr int kMaxDevices = 64;

// Control words of the kernel. Layout: one 256-byte header, then one 256-byte record per source.
struct alignas(256) ScratchHeader {
  unsigned int block_counter;        // blocks that finished their part of the current call
  unsigned int reserved;
  unsigned long long calls_done;     // incremented by the last block of every call
};
struct alignas(256) SourceRecord {
  unsigned long long done;           // completion counter of this source, as in ChannelCtrl::done
};
static_assert(sizeof(ScratchHeader) == 256 && sizeof(SourceRecord) == 256, "scratch layout");
static_assert(sizeof(ScratchHeader) + kMaxSources * sizeof(SourceRecord) == kScratchBytes, "scratch size");

// The scratch itself. In host code this name is only a handle for cudaGetSymbolAddress; the
// kernel receives the resolved device address as an argument.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

struct NoAllocParams {
  const void* self_in;
  void* out;
  unsigned long long numel;
  double self_w, post_scale;
  int n_src;
  unsigned char* scratch;
  const void* src[kMaxSources];
  double w[kMaxSources];
};

template <typename T> struct V;  // 16-byte vector <-> accumulators
template <> struct V<float> {
  using A = float; static constexpr int N = 4;
  static __device__ void un(const uint4& v, A* a) { a[0] = __uint_as_float(v.x); a[1] = __uint_as_float(v.y); a[2] = __uint_as_float(v.z); a[3] = __uint_as_float(v.w); }
  static __device__ uint4 pk(const A* a) { return make_uint4(__float_as_uint(a[0]), __float_as_uint(a[1]), __float_as_uint(a[2]), __float_as_uint(a[3])); }
};
template <> struct V<double> {
  using A = double; static constexpr int N = 2;
  static __device__ void un(const uint4& v, A* a) { a[0] = __hiloint2double(v.y, v.x); a[1] = __hiloint2double(v.w, v.z); }
  static __device__ uint4 pk(const A* a) { return make_uint4(__double2loint(a[0]), __double2hiint(a[0]), __double2loint(a[1]), __double2hiint(a[1])); }
};
template <> struct V<__half> {
  using A = float; static constexpr int N = 8;
  static __device__ void un(const uint4& v, A* a) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 f = __half22float2(h[i]); a[2 * i] = f.x; a[2 * i + 1] = f.y; }
  }
  static __device__ uint4 pk(const A* a) {
    uint4 v; __half2* h = reinterpret_cast<__half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(a[2 * i], a[2 * i + 1]);
    return v;
  }
};
template <> struct V<__nv_bfloat16> {
  using A = float; static constexpr int N = 8;
  static __device__ void un(const uint4& v, A* a) {
    const unsigned* u = reinterpret_cast<const unsigned*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) { a[2 * i] = __uint_as_float(u[i] << 16); a[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u); }
  }
  static __device__ uint4 pk(const A* a) {
    uint4 v; __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(a[2 * i], a[2 * i + 1]);
    return v;
  }
};

template <typename T>
__global__ void __launch_bounds__(kThreads) combine_noalloc_kernel(const __grid_constant__ NoAllocParams p) {
  using A = typename V<T>::A;
  constexpr int N = V<T>::N;
  __shared__ A w_s[kMaxSources];
  __shared__ bool is_last;
  for (int j = threadIdx.x; j < p.n_src; j += blockDim.x) w_s[j] = (A)p.w[j];
  __syncthreads();
  const A self_w = (A)p.self_w, post = (A)p.post_scale;
  const bool has_post = p.post_scale != 1.0;
  const unsigned long long nvec = p.numel / N;
  const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
  for (unsigned long long q = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; q < nvec; q += stride) {
    A acc[N];
    V<T>::un(reinterpret_cast<const uint4*>(p.self_in)[q], acc);
#pragma unroll
    for (int i = 0; i < N; ++i) acc[i] = acc[i] * self_w;
    for (int j = 0; j < p.n_src; ++j) {
      A t[N];
      V<T>::un(reinterpret_cast<const uint4*>(p.src[j])[q], t);
#pragma unroll
      for (int i = 0; i < N; ++i) acc[i] += t[i] * w_s[j];
    }
    if (has_post) {
#pragma unroll
      for (int i = 0; i < N; ++i) acc[i] = acc[i] * post;
    }
    reinterpret_cast<uint4*>(p.out)[q] = V<T>::pk(acc);
  }
  // Completion bookkeeping in the static scratch: the last block to arrive marks every source
  // as consumed and counts the call, and re-arms the arrival counter.
  ScratchHeader* hdr = reinterpret_cast<ScratchHeader*>(p.scratch);
  SourceRecord* rec = reinterpret_cast<SourceRecord*>(p.scratch + sizeof(ScratchHeader));
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(&hdr->block_counter, 1u);
    is_last = prev == gridDim.x - 1;
  }
  __syncthreads();
  if (is_last) {
    for (int j = threadIdx.x; j < p.n_src; j += blockDim.x) atomicAdd(&rec[j].done, 1ull);
    if (threadIdx.x == 0) {
      hdr->block_counter = 0;
      atomicAdd(&hdr->calls_done, 1ull);
    }
  }
}

std::mutex g_mu;
unsigned char* g_scratch_ptr[kMaxDevices] = {nullptr};

int Fail(char* err, int err_len, int code, const char* msg) {
  if (err != nullptr && err_len > 0) std::snprintf(err, static_cast<size_t>(err_len), "%s", msg);
  return code;
}

}  // namespace

extern "C" int bfb200_combine_noalloc(const void* self_in, const void* const* src_in, const double* src_w, int n_src,
                                      double self_w, double post_scale, void* out, unsigned long long numel,
                                      int elem_type, void* stream, char* err, int err_len) {
  if (n_src < 0 || n_src > kMaxSources)
    return Fail(err, err_len, 1, "bfb200_combine_noalloc: more than 64 sources do not fit the static scratch array");
  if (self_in == nullptr || out == nullptr || (n_src > 0 && (src_in == nullptr || src_w == nullptr)))
    return Fail(err, err_len, 2, "bfb200_combine_noalloc: null pointer argument");
  const int esize = bfb::ElemSize(elem_type);
  if (elem_type != bfb::kF32 && elem_type != bfb::kF64 && elem_type != bfb::kF16 && elem_type != bfb::kBF16)
    return Fail(err, err_len, 3, "bfb200_combine_noalloc: element type must be f32, f64, f16 or bf16");
  if ((numel * static_cast<unsigned long long>(esize)) % 16 != 0)
    return Fail(err, err_len, 4, "bfb200_combine_noalloc: numel * element size must be a multiple of 16 bytes");
  auto misaligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) != 0; };
  if (misaligned(self_in) || misaligned(out)) return Fail(err, err_len, 5, "bfb200_combine_noalloc: pointers must be 16-byte aligned");
  for (int j = 0; j < n_src; ++j)
    if (src_in[j] == nullptr || misaligned(src_in[j]))
      return Fail(err, err_len, 5, "bfb200_combine_noalloc: source pointers must be non-null and 16-byte aligned");
  if (numel == 0) return 0;

  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return Fail(err, err_len, 6, cudaGetErrorString(e));
  if (device < 0 || device >= kMaxDevices) return Fail(err, err_len, 6, "bfb200_combine_noalloc: device index out of range");
  // The kernel runs on the current device with that device's copy of the scratch array: the stream has to be one
  // of its streams, and self_in/out have to be memory the device can address (not plain host memory).
  if (stream != nullptr && stream != cudaStreamLegacy && stream != cudaStreamPerThread) {
    int stream_device = -1;
    e = cudaStreamGetDevice(static_cast<cudaStream_t>(stream), &stream_device);
    if (e != cudaSuccess) return Fail(err, err_len, 10, cudaGetErrorString(e));
    if (stream_device != device)
      return Fail(err, err_len, 10, "bfb200_combine_noalloc: the stream does not belong to the current device");
  }
  for (const void* ptr : {self_in, static_cast<const void*>(out)}) {
    cudaPointerAttributes attr;
    e = cudaPointerGetAttributes(&attr, ptr);
    if (e != cudaSuccess) return Fail(err, err_len, 11, cudaGetErrorString(e));
    if (attr.type == cudaMemoryTypeUnregistered)
      return Fail(err, err_len, 11, "bfb200_combine_noalloc: self_in and out must be device-accessible memory");
  }
  unsigned char* scratch = nullptr;
  {
    // Set-up, once per device, with that device current: resolve the device address of the array.
    std::lock_guard<std::mutex> g(g_mu);
    if (g_scratch_ptr[device] == nullptr) {
      void* ptr = nullptr;
      e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
      if (e != cudaSuccess || ptr == nullptr)
        return Fail(err, err_len, 7, e != cudaSuccess ? cudaGetErrorString(e) : "cudaGetSymbolAddress returned null");
      g_scratch_ptr[device] = static_cast<unsigned char*>(ptr);
    }
    scratch = g_scratch_ptr[device];
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // The array keeps the previous call's contents: everything the kernel counts from zero is cleared.
  e = cudaMemsetAsync(scratch, 0, sizeof(ScratchHeader) + static_cast<size_t>(n_src) * sizeof(SourceRecord), st);
  if (e != cudaSuccess) return Fail(err, err_len, 8, cudaGetErrorString(e));

  NoAllocParams p;
  std::memset(&p, 0, sizeof(p));
  p.self_in = self_in;
  p.out = out;
  p.numel = numel;
  p.self_w = self_w;
  p.post_scale = post_scale;
  p.n_src = n_src;
  p.scratch = scratch;
  for (int j = 0; j < n_src; ++j) {
    p.src[j] = src_in[j];
    p.w[j] = src_w[j];
  }
  const int per_vec = 16 / esize;
  unsigned long long blocks = (numel / per_vec + kThreads - 1) / kThreads;
  if (blocks < 1) blocks = 1;
  if (blocks > 296) blocks = 296;
  const int grid = static_cast<int>(blocks);
  switch (elem_type) {
    case bfb::kF32: combine_noalloc_kernel<float><<<grid, kThreads, 0, st>>>(p); break;
    case bfb::kF64: combine_noalloc_kernel<double><<<grid, kThreads, 0, st>>>(p); break;
    case bfb::kF16: combine_noalloc_kernel<__half><<<grid, kThreads, 0, st>>>(p); break;
    default: combine_noalloc_kernel<__nv_bfloat16><<<grid, kThreads, 0, st>>>(p); break;
  }
  bfb::CountKernelLaunch();
  e = cudaGetLastError();
  if (e != cudaSuccess) return Fail(err, err_len, 9, cudaGetErrorString(e));
  return 0;
}

namespace bfb {

cudaError_t NoAllocScratchRead(int n_src, unsigned int* block_counter, unsigned long long* calls_done,
                               unsigned long long* done) {
  if (n_src < 0 || n_src > kMaxSources) return cudaErrorInvalidValue;
  ScratchHeader hdr;
  cudaError_t e = cudaMemcpyFromSymbol(&hdr, g_noalloc_scratch, sizeof(hdr), 0, cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return e;
  *block_counter = hdr.block_counter;
  *calls_done = hdr.calls_done;
  for (int j = 0; j < n_src; ++j) {
    SourceRecord rec;
    e = cudaMemcpyFromSymbol(&rec, g_noalloc_scratch, sizeof(rec), sizeof(ScratchHeader) + j * sizeof(SourceRecord),
                             cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return e;
    done[j] = rec.done;
  }
  return cudaSuccess;
}

}  // namespace bfb
