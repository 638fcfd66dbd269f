// Phase timeline of bn_fwd_fused_kernel and per-pass times of the one-launch and two-kernel BatchNorm forms
// (see README.md in this folder for the build line).  Usage: bn_trace [rows channels]
#include "../../bluefog_b200/csrc/cuda/bn_kernels.cu"
#include <cstdio>
#include <vector>
#include <algorithm>
namespace bfb { void CountKernelLaunch() {} }
int main(int argc, char** argv) {
  long long R = argc > 1 ? atoll(argv[1]) : 12544; int C = argc > 2 ? atoi(argv[2]) : 256;
  size_t n = size_t(R) * C;
  __nv_bfloat16 *x, *y, *dy, *dx; unsigned char* mask; float *sums, *gamma, *beta, *mean, *rstd, *dg, *db; unsigned int* status;
  cudaMalloc(&x, n * 2); cudaMalloc(&y, n * 2); cudaMalloc(&dy, n * 2); cudaMalloc(&dx, n * 2); cudaMalloc(&mask, n / 8);
  const int iters = 20; const int slot = 8 * 2 * C + 64;
  cudaMalloc(&sums, size_t(slot) * 4 * iters * 4); cudaMalloc(&gamma, C * 4); cudaMalloc(&beta, C * 4); cudaMalloc(&mean, C * 4); cudaMalloc(&rstd, C * 4);
  cudaMalloc(&dg, C * 4); cudaMalloc(&db, C * 4); cudaMalloc(&status, 4); cudaMemset(status, 0, 4);
  std::vector<__nv_bfloat16> h(n); for (size_t i = 0; i < n; ++i) h[i] = __float2bfloat16(float((i * 7919) % 17) * 0.1f - 0.8f);
  cudaMemcpy(x, h.data(), n * 2, cudaMemcpyHostToDevice); cudaMemcpy(dy, h.data(), n * 2, cudaMemcpyHostToDevice);
  std::vector<float> ones(C, 1.f); cudaMemcpy(gamma, ones.data(), C * 4, cudaMemcpyHostToDevice); cudaMemset(beta, 0, C * 4);
  for (int fused = 1; fused >= 0; --fused) {
    for (int pass = 0; pass < 2; ++pass) {
      float ms_best = 1e9;
      for (int rep = 0; rep < 3; ++rep) {
        cudaMemset(sums, 0, size_t(slot) * 4 * iters * 4);
#ifdef BN_TRACE
        { static unsigned long long z[160][8]; cudaMemcpyToSymbol(bfb::g_bn_trace, z, sizeof(z)); }
#endif
        cudaDeviceSynchronize();
        cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
        cudaEventRecord(e0);
        for (int i = 0; i < iters; ++i) {
          float* s = sums + size_t(slot) * (pass * iters + i);
          int bar = fused ? bfb::BnSumCopies(C) : 0;
          cudaError_t e = pass == 0
            ? bfb::LaunchBnForward(x, nullptr, y, mask, s, gamma, beta, nullptr, nullptr, mean, rstd, R, C, 1e-5f, 0.1f, 1, 0, 0, 0, bar, status)
            : bfb::LaunchBnBackward(dy, nullptr, mask, x, dx, nullptr, s, mean, rstd, gamma, dg, db, R, C, 1, 0, 0, bar, status);
          if (e != cudaSuccess) { printf("launch error %s\n", cudaGetErrorString(e)); return 1; }
        }
        cudaEventRecord(e1);
        if (cudaDeviceSynchronize() != cudaSuccess) { printf("sync error\n"); return 1; }
        float ms; cudaEventElapsedTime(&ms, e0, e1); if (ms < ms_best) ms_best = ms;
      }
#ifdef BN_TRACE
      if (fused && pass == 0) {
        static unsigned long long h[160][8];
        cudaMemcpyFromSymbol(h, bfb::g_bn_trace, sizeof(h));
        unsigned long long t0 = ~0ull;
        for (int b = 0; b < 148; ++b) if (h[b][0] && h[b][0] < t0) t0 = h[b][0];
        const char* nm[6] = {"entry", "loads done", "flushed", "barrier passed", "params ready", "exit"};
        for (int i = 0; i < 6; ++i) {
          std::vector<long long> v; for (int b = 0; b < 148; ++b) if (h[b][0]) v.push_back((long long)(h[b][i] - t0));
          std::sort(v.begin(), v.end());
          printf("   %-16s min %6lld med %6lld max %6lld ns (%zu blocks)\n", nm[i], v[0], v[v.size() / 2], v.back(), v.size());
        }
      }
#endif
      unsigned st; cudaMemcpy(&st, status, 4, cudaMemcpyDeviceToHost);
      printf("R=%lld C=%d %s %s: %.1f us per pass (status %u)\n", R, C, fused ? "one launch " : "two kernels", pass ? "bwd" : "fwd", ms_best * 1000 / iters, st);
    }
  }
  return 0;
}
