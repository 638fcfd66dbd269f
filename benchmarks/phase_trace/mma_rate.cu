// Clocks per tcgen05.mma (128 x N x 16, bf16) issued back to back by one thread out of shared memory that nothing
// else touches: K-major or MN-major operands (A and/or B), N in {64, 128, 256}.  See README.md for the build line.
#include <cstdio>
#include <cuda_runtime.h>
#include "../../bluefog_b200/csrc/cuda/tcgen05_common.cuh"
using namespace bfb::t5;
template <int N>
__global__ void __launch_bounds__(192, 1) rate_kernel(long long* out, int iters, int amn, int bmn) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint32_t tmem_base_s;
  __shared__ uint64_t bar;
  __shared__ int failed_s;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < (160 * 1024) / 4; i += blockDim.x) { uint32_t h = (i + 1) * 2654435761u; h ^= h >> 13; uint32_t lo = 0x3c00u | (h & 0x3ffu) | ((h >> 3) & 0x8000u); uint32_t hi = 0x3c00u | ((h >> 10) & 0x3ffu) | ((h >> 5) & 0x8000u); reinterpret_cast<uint32_t*>(smem)[i] = lo | (hi << 16); }
  if (threadIdx.x == 0) { failed_s = 0; mbar_init(smem_u32(&bar), 1); asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_s;
  if (warp == 1 && lane == 0) {
    const uint32_t a0 = smem_u32(smem), b0 = smem_u32(smem + 64 * 1024);
    const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (amn ? (1u << 15) : 0u) | (bmn ? (1u << 16) : 0u) |
                           (uint32_t(N >> 3) << 17) | (uint32_t(128 >> 4) << 24);
    // K-major: tile of [rows x 64 k] per 128B row, k-step = 32 bytes inside the row (desc + 2).
    // MN-major: boxes of [128 k rows x 64 mn], box stride 16 KB, k-step = 16 rows = 2048 bytes (desc + 128).
    const uint64_t adesc = amn ? make_desc_mn(a0, 16384, 1024) : make_desc(a0);
    const uint64_t bdesc = bmn ? make_desc_mn(b0, 16384, 1024) : make_desc(b0);
    const uint64_t astep = amn ? 128 : 2, bstep = bmn ? 128 : 2;
    const long long t0 = clock64();
    for (int i = 0; i < iters; ++i) {
#pragma unroll
      for (int k = 0; k < 4; ++k) umma_f16(tmem_base, adesc + astep * k, bdesc + bstep * k, idesc, 1u);
    }
    const long long t1 = clock64();
    umma_commit(smem_u32(&bar));
    mbar_wait(smem_u32(&bar), 0, &failed_s);
    const long long t2 = clock64();
    if (blockIdx.x == 0) { out[0] = t1 - t0; out[1] = t2 - t0; }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}
template <int N>
void run(long long* d, int iters, int amn, int bmn) {
  cudaFuncSetAttribute(rate_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, 170 * 1024);
  for (int rep = 0; rep < 2; ++rep) rate_kernel<N><<<148, 192, 170 * 1024>>>(d, iters, amn, bmn);
  cudaError_t e = cudaDeviceSynchronize();
  long long h[2];
  cudaMemcpy(h, d, sizeof(h), cudaMemcpyDeviceToHost);
  printf("N=%d A %s B %s: issue %.1f clk/MMA, complete %.1f clk/MMA %s\n", N, amn ? "MN" : "K ", bmn ? "MN" : "K ",
         double(h[0]) / (4.0 * iters), double(h[1]) / (4.0 * iters), cudaGetErrorString(e));
}
int main() {
  long long* d;
  cudaMalloc(&d, 16);
  const int iters = 1800;
  for (int amn = 0; amn < 2; ++amn) for (int bmn = 0; bmn < 2; ++bmn) { run<64>(d, iters, amn, bmn); run<128>(d, iters, amn, bmn); run<256>(d, iters, amn, bmn); }
  return 0;
}
