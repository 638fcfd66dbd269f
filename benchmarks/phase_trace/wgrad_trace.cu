// Phase timeline of conv_wgrad_kernel (see README.md in this folder for the build line).
#include "../../bluefog_b200/csrc/cuda/conv_tcgen05.cu"
#include <vector>
#include <algorithm>
namespace bfb {
void CountKernelLaunch() {}
void Dump(int ctas, const char* label) {
  static unsigned long long h[160][16];
  cudaMemcpyFromSymbol(h, g_wgrad_trace, sizeof(h));
  unsigned long long t0 = ~0ull, tend = 0;
  for (int b = 0; b < ctas; ++b) { if (!h[b][0]) continue; t0 = std::min(t0, h[b][0]); tend = std::max(tend, h[b][9]); }
  printf("%s: kernel span %llu ns over %d CTAs\n", label, tend - t0, ctas);
  const char* names[10] = {"entry", "setup done", "first load issued", "producer done", "first full", "mma issued all", "epi: acc ready", "epi: stored", "epi: finalized", "exit"};
  for (int i = 0; i < 10; ++i) {
    std::vector<long long> v;
    for (int b = 0; b < ctas; ++b) if (h[b][i]) v.push_back((long long)(h[b][i] - t0));
    if (v.empty()) continue;
    std::sort(v.begin(), v.end());
    printf("  %-18s min %6lld med %6lld max %6lld\n", names[i], v.front(), v[v.size() / 2], v.back());
  }
  std::vector<long long> pw, mw;
  for (int b = 0; b < ctas; ++b) { pw.push_back(h[b][10]); mw.push_back(h[b][11]); }
  std::sort(pw.begin(), pw.end()); std::sort(mw.begin(), mw.end());
  printf("  producer waited on empty: med %lld max %lld ns; mma waited on full: med %lld max %lld ns\n", pw[pw.size()/2], pw.back(), mw[mw.size()/2], mw.back());
}
void Clear() { static unsigned long long z[160][16]; cudaMemcpyToSymbol(g_wgrad_trace, z, sizeof(z)); }
}
int main(int argc, char** argv) {
  int N = 64, H = 7, W = 7, Cin = 512, Cout = 2048, k = 1;
  if (argc >= 7) { N = atoi(argv[1]); H = atoi(argv[2]); W = atoi(argv[3]); Cin = atoi(argv[4]); Cout = atoi(argv[5]); k = atoi(argv[6]); }
  size_t nx = size_t(N) * H * W * Cin, ndy = size_t(N) * H * W * Cout, nw = size_t(Cout) * k * k * Cin;
  __nv_bfloat16 *x, *dy, *dw; float* ws; unsigned int* cnt; unsigned int* status;
  cudaMalloc(&x, nx * 2); cudaMalloc(&dy, ndy * 2); cudaMalloc(&dw, nw * 2);
  cudaMalloc(&ws, std::max<size_t>(nw, 8u << 20) * 4); cudaMalloc(&cnt, 4096 * 4); cudaMalloc(&status, 4);
  cudaMemset(ws, 0, std::max<size_t>(nw, 8u << 20) * 4); cudaMemset(cnt, 0, 4096 * 4); cudaMemset(status, 0, 4);
  std::vector<__nv_bfloat16> hx(nx), hdy(ndy);
  for (size_t i = 0; i < nx; ++i) hx[i] = __float2bfloat16(float((i * 7919) % 13) * 0.1f - 0.6f);
  for (size_t i = 0; i < ndy; ++i) hdy[i] = __float2bfloat16(float((i * 104729) % 11) * 0.1f - 0.5f);
  cudaMemcpy(x, hx.data(), nx * 2, cudaMemcpyHostToDevice); cudaMemcpy(dy, hdy.data(), ndy * 2, cudaMemcpyHostToDevice);
  bfb::WgradProblem p{};
  p.dy = bfb::ConvView{dy, N, H, W, Cout, Cout, (long long)W * Cout, (long long)H * W * Cout};
  p.x = bfb::ConvView{x, N, H, W, Cin, Cin, (long long)W * Cin, (long long)H * W * Cin};
  p.in_stride = 1; p.taps.T = k * k; p.w_taps = k * k;
  for (int t = 0; t < k * k; ++t) { p.taps.dh[t] = t / k - k / 2; p.taps.dw[t] = t % k - k / 2; p.taps.wt[t] = t; }
  p.dw = dw; p.workspace = ws; p.workspace_floats = (long long)std::max<size_t>(nw, 8u << 20); p.counters = cnt; p.n_counters = 4096;
  const char* plans[] = {nullptr, "64,1,1,1", "128,1,2,1", "256,1,4,1", "256,1,1,4"};
  for (const char* plan : plans) {
    if (plan) setenv("BLUEFOG_B200_WGRAD_PLAN", plan, 1); else unsetenv("BLUEFOG_B200_WGRAD_PLAN");
    for (int i = 0; i < 3; ++i) if (bfb::LaunchConvWgrad(p, status, 0) != cudaSuccess) { printf("launch failed\n"); return 1; }
    cudaDeviceSynchronize();
    cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
    cudaEventRecord(e0);
    for (int i = 0; i < 20; ++i) bfb::LaunchConvWgrad(p, status, 0);
    cudaEventRecord(e1); cudaDeviceSynchronize();
    float ms; cudaEventElapsedTime(&ms, e0, e1);
    bfb::Clear();
    bfb::LaunchConvWgrad(p, status, 0);
    if (cudaDeviceSynchronize() != cudaSuccess) { printf("sync failed\n"); return 1; }
    unsigned int st; cudaMemcpy(&st, status, 4, cudaMemcpyDeviceToHost);
    printf("plan %s: %.1f us per launch (stream of 20), status %u\n", plan ? plan : "auto", ms * 1000 / 20, st);
    bfb::Dump(148, plan ? plan : "auto");
  }
  return 0;
}
