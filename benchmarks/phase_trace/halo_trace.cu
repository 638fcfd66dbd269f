// Phase timeline of conv_halo_kernel: when the MMA thread has issued each of its first tiles and what it waited for
// (see README.md in this folder for the build line).  Usage: halo_trace [N H W Cin Cout]
#include "../../bluefog_b200/csrc/cuda/conv_tcgen05.cu"
#include <vector>
#include <algorithm>
namespace bfb {
void CountKernelLaunch() {}
void Dump() {
  static unsigned long long h[160][16];
  cudaMemcpyFromSymbol(h, g_halo_trace, sizeof(h));
  unsigned long long t0 = ~0ull;
  for (int b = 0; b < 148; ++b) if (h[b][0] && h[b][0] < t0) t0 = h[b][0];
  const char* nm[8] = {"entry", "first patch in", "tile 0 issued", "tile 1 issued", "tile 2 issued", "tile 3 issued", "mma thread done", "exit"};
  for (int i = 0; i < 8; ++i) {
    std::vector<long long> v; for (int b = 0; b < 148; ++b) if (h[b][i]) v.push_back((long long)(h[b][i] - t0));
    if (v.empty()) continue; std::sort(v.begin(), v.end());
    printf("   %-16s min %6lld med %6lld max %6lld ns\n", nm[i], v[0], v[v.size()/2], v.back());
  }
  const char* wn[3] = {"acc_empty", "full_a (patches)", "full_b (filter)"};
  for (int i = 8; i < 11; ++i) {
    std::vector<long long> v; for (int b = 0; b < 148; ++b) if (h[b][0]) v.push_back((long long)h[b][i]);
    std::sort(v.begin(), v.end());
    printf("   mma thread waited on %-18s med %6lld max %6lld clk\n", wn[i-8], v[v.size()/2], v.back());
  }
}
void Clear() { static unsigned long long z[160][16]; cudaMemcpyToSymbol(g_halo_trace, z, sizeof(z)); }
}
int main(int argc, char** argv) {
  int N = 64, H = 28, W = 28, Cin = 128, Cout = 128;
  if (argc >= 6) { N = atoi(argv[1]); H = atoi(argv[2]); W = atoi(argv[3]); Cin = atoi(argv[4]); Cout = atoi(argv[5]); }
  size_t nx = size_t(N) * H * W * Cin, ny = size_t(N) * H * W * Cout, nw = size_t(Cout) * 9 * Cin;
  __nv_bfloat16 *x, *y, *w; unsigned int* status;
  cudaMalloc(&x, nx * 2); cudaMalloc(&y, ny * 2); cudaMalloc(&w, nw * 2); cudaMalloc(&status, 4); cudaMemset(status, 0, 4);
  cudaMemset(x, 0, nx * 2); cudaMemset(w, 0, nw * 2);
  for (int i = 0; i < 3; ++i) if (bfb::LaunchConv3x3Nhwc(x, w, y, N, H, W, Cin, Cout, 0, 0, status, 0) != cudaSuccess) { printf("launch failed\n"); return 1; }
  cudaDeviceSynchronize();
  cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
  cudaEventRecord(e0);
  for (int i = 0; i < 20; ++i) bfb::LaunchConv3x3Nhwc(x, w, y, N, H, W, Cin, Cout, 0, 0, status, 0);
  cudaEventRecord(e1); cudaDeviceSynchronize();
  float ms; cudaEventElapsedTime(&ms, e0, e1);
  bfb::Clear();
  bfb::LaunchConv3x3Nhwc(x, w, y, N, H, W, Cin, Cout, 0, 0, status, 0);
  if (cudaDeviceSynchronize() != cudaSuccess) { printf("sync failed\n"); return 1; }
  unsigned st; cudaMemcpy(&st, status, 4, cudaMemcpyDeviceToHost);
  printf("N=%d %dx%d %d->%d: %.1f us per launch, status %u\n", N, H, W, Cin, Cout, ms * 1000 / 20, st);
  bfb::Dump();
  return 0;
}
