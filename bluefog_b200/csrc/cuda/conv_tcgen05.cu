// 3x3 / stride 1 / pad 1 convolution of NHWC bf16 activations as an implicit GEMM on tcgen05:
//
//   y[n, h, w, co] = sum_{r, s, ci} x[n, h + r - 1, w + s - 1, ci] * wgt[co, r, s, ci]
//
// (with flip_taps the filter tap is (2 - r, 2 - s): the input gradient of such a convolution is the
// same convolution of the output gradient with the filter rotated by 180 degrees and its channel
// axes exchanged, so only the exchange of axes is left to the caller)
//
// The GEMM view is  M = output pixels, N = Cout, K = 9 * Cin,  and no im2col matrix is ever
// written: one CTA owns a patch of  bn images x bh rows x bw columns  (at most 128 pixels, the M
// extent of one tcgen05.mma), and for every filter tap (r, s) and every 64-channel slice the
// producer warp fetches the *shifted* input patch with one 4-D tiled TMA load — box
// {64 channels, bw, bh, bn} starting at (ci0, w0 + s - 1, h0 + r - 1, n0).  Coordinates outside
// the image read zeros, which is exactly the padding.  The box lands in shared memory as
// [pixels x 128 bytes] in the 128-byte swizzle, i.e. the K-major A tile that the matrix
// descriptor expects.  The weights [Cout, 3, 3, Cin] (channels-last filter memory) are the K-major
// B matrix [Cout, 9 * Cin] and arrive through plain 2-D TMA loads.  No load uses cluster multicast.
//
// As in the persistent GEMM: warp 0 produces, warp 1 issues tcgen05.mma into one of two
// accumulator buffers in tensor memory, warps 2-5 drain the other buffer, convert to bf16,
// stage [pixels x 64 channels] boxes in shared memory and hand them to 4-D TMA stores, which
// clip patches that hang over the image or batch edge.  All mbarrier waits have a time limit;
// on expiry the kernel raises a status word, drains its copies in flight, frees its tensor
// memory and returns.
//
// The reference has no convolution code (its benchmark calls cuDNN through torchvision,
// examples/pytorch_benchmark.py:100).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "comm_kernels.h"
#include "conv_tcgen05.h"
#include "tcgen05_common.cuh"

namespace bfb {
namespace {

using namespace t5;

constexpr int BM = 128, BK = 64;
constexpr int kUmmaK = 16;
constexpr int kThreads = 192;

template <int BN_>
struct ConvCfg {
  static constexpr int kStages = (BN_ == 256) ? 4 : (BN_ == 128 ? 5 : 6);
  static constexpr uint32_t kBytesA = BM * BK * 2;          // room for 128 pixels, the box may be smaller
  static constexpr uint32_t kBytesB = BN_ * BK * 2;
  static constexpr uint32_t kBytesStage = kBytesA + kBytesB;
  static constexpr uint32_t kCols = 2 * BN_ < 32 ? 32 : 2 * BN_;
  static constexpr uint32_t kBytesOutBox = BM * 64 * 2;     // [128 pixels x 64 channels]
  static constexpr uint32_t kBytesOut = 2 * kBytesOutBox;
  static constexpr size_t kSmem = 1024 + size_t(kStages) * kBytesStage + kBytesOut + 256;
  static constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(BN_ >> 3) << 17) | (uint32_t(BM >> 4) << 24);
};

struct ConvGeom {
  int N, H, W, Cin, Cout;
  int bw, bh, bn;            // patch extent (bw * bh * bn <= 128)
  int tiles_w, tiles_h, tiles_img, tiles_co;
  int flip_taps;             // 1: input tap (r, s) meets filter tap (2 - r, 2 - s) (input-gradient form)
};

__device__ __forceinline__ void epilogue_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// BMODE 0: the filter is [Cout, 3, 3, Cin] and supplies K-major B tiles.  BMODE 1 (input-gradient form): the
// filter stays in the layout of the forward pass, [Cred, 3, 3, Cout'] with the reduction channels outermost,
// and supplies MN-major B tiles: BN_/64 boxes of [64 reduction rows x 64 output channels] per stage.
template <int BN_, int BMODE = 0>
__global__ void __launch_bounds__(kThreads, 1)
conv3x3_nhwc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    const __grid_constant__ CUtensorMap map_y, const ConvGeom g, unsigned int* __restrict__ status) {
  using Cfg = ConvCfg<BN_>;
  constexpr int S = Cfg::kStages;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* stage_a = smem;
  unsigned char* stage_b = smem + size_t(S) * Cfg::kBytesA;
  unsigned char* stage_out = smem + size_t(S) * Cfg::kBytesStage;
  uint64_t* bars = reinterpret_cast<uint64_t*>(stage_out + Cfg::kBytesOut);
  // bars[0..S): full, [S..2S): empty, [2S..2S+2): acc_full, [2S+2..2S+4): acc_empty
  __shared__ uint32_t tmem_base_s;
  __shared__ int failed_s;
  __shared__ int go_s;              // the epilogue warps' common decision to process a tile
  volatile int* failed = &failed_s;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int spatial = g.tiles_w * g.tiles_h * g.tiles_img;
  const int num_tiles = spatial * g.tiles_co;
  const int cblocks = g.Cin / BK;
  const int num_kb = 9 * cblocks;
  const uint32_t bytes_a = uint32_t(g.bw * g.bh * g.bn) * 128u;      // what one A box delivers

  if (threadIdx.x == 0) {
    failed_s = 0;
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(&bars[s]), 1);
      mbar_init(smem_u32(&bars[S + s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&bars[2 * S + a]), 1);        // one tcgen05.commit
      mbar_init(smem_u32(&bars[2 * S + 2 + a]), 4);    // one arrive per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(Cfg::kCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_s;

  // tile -> (co0, n0, h0, w0); consecutive tiles share the input patch and differ in co0
  auto tile_coords = [&](int tile, int& co0, int& n0, int& h0, int& w0) {
    const int sp = tile / g.tiles_co;
    co0 = (tile % g.tiles_co) * BN_;
    w0 = (sp % g.tiles_w) * g.bw;
    h0 = ((sp / g.tiles_w) % g.tiles_h) * g.bh;
    n0 = (sp / (g.tiles_w * g.tiles_h)) * g.bn;
  };

  int armed = 0;
  if (warp == 0) {
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int co0, n0, h0, w0;
        tile_coords(tile, co0, n0, h0, w0);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int tap = kb / cblocks;
          const int ci0 = (kb % cblocks) * BK;
          const int r = tap / 3, sx = tap % 3;
          const int s = it % S;
          if (!mbar_wait(smem_u32(&bars[S + s]), ((it / S) & 1) ^ 1, failed)) { ok = false; break; }
          const uint32_t full = smem_u32(&bars[s]);
          mbar_expect_tx(full, bytes_a + Cfg::kBytesB);
          tma_load_4d(smem_u32(stage_a + size_t(s) * Cfg::kBytesA), &map_x, full, ci0, w0 + sx - 1, h0 + r - 1, n0);
          const int wtap = g.flip_taps ? 8 - tap : tap;
          if (BMODE == 0) {
            tma_load_2d(smem_u32(stage_b + size_t(s) * Cfg::kBytesB), &map_w, full, wtap * g.Cin + ci0, co0);
          } else {
#pragma unroll
            for (int j = 0; j < BN_ / 64; ++j)
              tma_load_2d(smem_u32(stage_b + size_t(s) * Cfg::kBytesB + size_t(j) * 8192), &map_w, full,
                          wtap * g.Cout + co0 + j * 64, ci0);
          }
          armed = it + 1;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int it = 0, local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
        const int acc = local & 1;
        if (!mbar_wait(smem_u32(&bars[2 * S + 2 + acc]), ((local >> 1) & 1) ^ 1, failed)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_d = tmem_base + uint32_t(acc * BN_);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % S;
          if (!mbar_wait(smem_u32(&bars[s]), (it / S) & 1, failed)) { ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint64_t adesc = make_desc(smem_u32(stage_a + size_t(s) * Cfg::kBytesA));
          const uint32_t b_addr = smem_u32(stage_b + size_t(s) * Cfg::kBytesB);
          const uint64_t bdesc = BMODE == 0 ? make_desc(b_addr) : make_desc_mn(b_addr, 8192, 1024);
          constexpr uint32_t idesc = Cfg::kIdesc | (BMODE != 0 ? (1u << 16) : 0u);      // bit 16: B is MN-major
          constexpr uint64_t b_step = BMODE == 0 ? 2 : (16 * 128) >> 4;                 // 16 reduction rows per MMA
#pragma unroll
          for (int k = 0; k < BK / kUmmaK; ++k)
            umma_f16(tmem_d, adesc + uint64_t(2 * k), bdesc + b_step * uint64_t(k), idesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit(smem_u32(&bars[S + s]));
        }
        if (ok) umma_commit(smem_u32(&bars[2 * S + acc]));
      }
    }
  } else {
    const int q = warp & 3;                  // accumulator lanes [32q, 32q + 32)
    const bool issuer = (warp == 2 && lane == 0);
    int local = 0;
    int boxes = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
      const int acc = local & 1;
      int co0, n0, h0, w0;
      tile_coords(tile, co0, n0, h0, w0);
      // The four epilogue warps meet at named barriers below, so they must agree on whether this
      // tile is processed: every thread waits (a timeout raises the flag), then one thread reads
      // the flag once and publishes the decision.
      mbar_wait(smem_u32(&bars[2 * S + acc]), (local >> 1) & 1, failed);
      epilogue_bar();
      if (issuer) go_s = (*failed == 0);
      epilogue_bar();
      if (!*reinterpret_cast<volatile int*>(&go_s)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
      for (int c = 0; c < BN_ / 64; ++c) {
        const int cbase = co0 + c * 64;
        if (cbase >= g.Cout) break;                                   // uniform over the CTA
        uint32_t rr[64];
        const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + uint32_t(acc * BN_ + c * 64);
        tmem_ld32(taddr, rr);
        tmem_ld32(taddr + 32, rr + 32);
        // the box staged two stores ago must have left shared memory before it is overwritten
        if (issuer) tma_store_wait_read<1>();
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        epilogue_bar();
        unsigned char* box = stage_out + size_t(boxes & 1) * Cfg::kBytesOutBox;
        const int prow = q * 32 + lane;                               // pixel row of the patch
        unsigned char* row = box + prow * 128;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          uint4 pk;
          __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
          for (int i = 0; i < 4; ++i)
            h[i] = __floats2bfloat162_rn(__uint_as_float(rr[j * 8 + 2 * i]), __uint_as_float(rr[j * 8 + 2 * i + 1]));
          *reinterpret_cast<uint4*>(row + ((j ^ (prow & 7)) << 4)) = pk;      // 128-byte swizzle
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        epilogue_bar();
        if (issuer) {
          tma_store_4d(&map_y, smem_u32(box), cbase, w0, h0, n0);
          tma_store_commit();
        }
        ++boxes;
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&bars[2 * S + 2 + acc])) : "memory");
    }
    if (issuer) tma_store_wait_all();
  }
  if (warp == 0 && lane == 0 && *failed) {
    const int first = armed > S ? armed - S : 0;
    for (int it = first; it < armed; ++it) {
      const unsigned long long t0 = now_ns();
      while (!mbar_try(smem_u32(&bars[it % S]), (it / S) & 1) && now_ns() - t0 < kWaitLimitNs) {}
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Cfg::kCols) : "memory");
  }
  if (threadIdx.x == 0 && failed_s && status != nullptr) atomicExch(status, 1u);
}

bool MakeMap4d(CUtensorMap* map, const void* base, int C, int W, int H, int N, int bw, int bh, int bn) {
  const cuuint64_t dims[4] = {cuuint64_t(C), cuuint64_t(W), cuuint64_t(H), cuuint64_t(N)};
  const cuuint64_t strides[3] = {cuuint64_t(C) * 2, cuuint64_t(W) * C * 2, cuuint64_t(H) * W * C * 2};
  const cuuint32_t box[4] = {64, cuuint32_t(bw), cuuint32_t(bh), cuuint32_t(bn)};
  return EncodeTiled(map, 4, base, dims, strides, box);
}

bool MakeMap2d(CUtensorMap* map, const void* base, int rows, int cols, int box_rows) {
  const cuuint64_t dims[2] = {cuuint64_t(cols), cuuint64_t(rows)};
  const cuuint64_t strides[1] = {cuuint64_t(cols) * 2};
  const cuuint32_t box[2] = {64, cuuint32_t(box_rows)};
  return EncodeTiled(map, 2, base, dims, strides, box);
}

int SmCount() {
  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (sm_count <= 0) sm_count = 148;
  }
  return sm_count;
}

template <int BN_, int BMODE>
cudaError_t Launch(const CUtensorMap& mx, const CUtensorMap& mw, const CUtensorMap& my, const ConvGeom& g,
                   unsigned int* status, cudaStream_t stream) {
  using Cfg = ConvCfg<BN_>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(conv3x3_nhwc_kernel<BN_, BMODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(Cfg::kSmem));
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  const int tiles = g.tiles_w * g.tiles_h * g.tiles_img * g.tiles_co;
  const int sms = SmCount();
  conv3x3_nhwc_kernel<BN_, BMODE><<<tiles < sms ? tiles : sms, kThreads, Cfg::kSmem, stream>>>(mx, mw, my, g, status);
  CountKernelLaunch();
  return cudaGetLastError();
}

}  // namespace

bool Conv3x3Patch(int N, int H, int W, int* bw, int* bh, int* bn) {
  if (N <= 0 || H <= 0 || W <= 0 || W > 128) return false;
  int w = W, h = 128 / W;
  if (h > H) h = H;
  const int th = (H + h - 1) / h;
  h = (H + th - 1) / th;                 // same number of patches, least overhang
  int n = 1;
  if (h == H) {
    n = 128 / (w * h);
    if (n > N) n = N;
    if (n < 1) n = 1;
    const int tn = (N + n - 1) / n;
    n = (N + tn - 1) / tn;
  }
  *bw = w;
  *bh = h;
  *bn = n;
  return true;
}

bool Conv3x3Supported(int N, int H, int W, int Cin, int Cout) {
  int bw, bh, bn;
  return GetEncodeFn() != nullptr && Cin >= 64 && (Cin % 64) == 0 && Cout >= 64 && (Cout % 8) == 0 &&
         Conv3x3Patch(N, H, W, &bw, &bh, &bn);
}

cudaError_t LaunchConv3x3Nhwc(const void* x, const void* w, void* y, int N, int H, int W, int Cin, int Cout,
                              int flip_taps, int filter_mode, unsigned int* status, cudaStream_t stream) {
  if (filter_mode < 0 || filter_mode > 1) return cudaErrorInvalidValue;
  if (!Conv3x3Supported(N, H, W, Cin, Cout)) return cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15) || (reinterpret_cast<uintptr_t>(y) & 15))
    return cudaErrorInvalidValue;
  ConvGeom g;
  g.N = N; g.H = H; g.W = W; g.Cin = Cin; g.Cout = Cout;
  g.flip_taps = flip_taps ? 1 : 0;
  Conv3x3Patch(N, H, W, &g.bw, &g.bh, &g.bn);
  g.tiles_w = (W + g.bw - 1) / g.bw;
  g.tiles_h = (H + g.bh - 1) / g.bh;
  g.tiles_img = (N + g.bn - 1) / g.bn;
  const int spatial = g.tiles_w * g.tiles_h * g.tiles_img;
  // widest N tile that still occupies most of the SMs (a 256-wide tile streams half as many weight
  // bytes per FLOP through shared memory); narrow outputs take the narrow tile
  int bn_tile = 256;
  if (Cout <= 64) bn_tile = 64;
  else if (Cout <= 128 || spatial * ((Cout + 255) / 256) < (SmCount() * 3) / 4) bn_tile = 128;
  g.tiles_co = (Cout + bn_tile - 1) / bn_tile;
  CUtensorMap mx, mw, my;
  // filter map: K-major [Cout rows, 9*Cin], or (MN-major modes) the forward filter [Cin rows, 9*Cout] in boxes of 64 x 64
  const bool mw_ok = filter_mode == 0 ? MakeMap2d(&mw, w, Cout, 9 * Cin, bn_tile) : MakeMap2d(&mw, w, Cin, 9 * Cout, 64);
  if (!MakeMap4d(&mx, x, Cin, W, H, N, g.bw, g.bh, g.bn) || !mw_ok || !MakeMap4d(&my, y, Cout, W, H, N, g.bw, g.bh, g.bn))
    return cudaErrorInvalidValue;
#define BFB_CONV_LAUNCH(BNV) \
  (filter_mode == 0 ? Launch<BNV, 0>(mx, mw, my, g, status, stream) : Launch<BNV, 1>(mx, mw, my, g, status, stream))
  if (bn_tile == 64) return BFB_CONV_LAUNCH(64);
  if (bn_tile == 128) return BFB_CONV_LAUNCH(128);
  return BFB_CONV_LAUNCH(256);
#undef BFB_CONV_LAUNCH
}

}  // namespace bfb
