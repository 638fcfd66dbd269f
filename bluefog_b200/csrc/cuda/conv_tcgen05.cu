// Convolutions of NHWC bf16 activations as implicit GEMMs on tcgen05.
//
// Forward / input-gradient kernel (conv_igemm_kernel):
//
//   y[n, a*os + ph, b*os + pw, co] = sum_{t, ci} x[n, a*is + dh[t], b*is + dw[t], ci] * wgt[co, wt[t], ci]
//
// for a list of at most 16 taps t.  A 3x3 / pad 1 convolution has the nine taps (r - 1, s - 1); its input
// gradient is the same sum over the output gradient with taps (1 - r, 1 - s) and the filter's channel axes
// exchanged; a stride-2 convolution reads with is = 2; its input gradient splits into the four parity classes
// of the input position, each a stride-1 sum over a subset of the taps whose result is stored with os = 2; the
// 7x7 / stride 2 stem, folded to a 4x4 filter over 2x2 pixel blocks of 16 channels, has four taps (r, 0) whose
// reduction slice is the 64 consecutive values of four neighbouring pixels.
//
// The GEMM view is  M = output positions, N = Cout, K = taps * Cin,  and no im2col matrix is ever
// written: one CTA owns a patch of  bn images x bh rows x bw columns  (at most 128 positions, the M
// extent of one tcgen05.mma), and for every tap and every 64-channel slice the producer warp fetches the
// *shifted* input patch with one 4-D tiled TMA load (traversal stride `is` along width and height).
// Coordinates outside the image read zeros, which is exactly the padding.  The box lands in shared memory
// as [positions x 128 bytes] in the 128-byte swizzle, i.e. the K-major A tile that the matrix descriptor
// expects.  The filter arrives through 2-D TMA loads, K-major ([Cout, taps * Cin]) or, for input gradients,
// MN-major straight from the forward filter ([Cred, taps * Cout]).  No load uses cluster multicast.
//
// As in the persistent GEMM: warp 0 produces, warp 1 issues tcgen05.mma into one of two
// accumulator buffers in tensor memory, warps 2-5 drain the other buffer, convert to bf16 and either
// stage [positions x 64 channels] boxes in shared memory for 4-D TMA stores (which clip patches that hang
// over the image or batch edge) or, for strided placement, store their pixel's 128 bytes directly.
//
// Filter-gradient kernel (conv_wgrad_kernel):
//
//   dw[co, wt[t], ci] = sum_{n, a, b} dy[n, a, b, co] * x[n, a*is + dh[t], b*is + dw[t], ci]
//
// is the GEMM  M = Cout, N = Cin (per tap), K = output positions.  Both operands are position-major in
// memory, which is the MN-major operand form: a patch of positions (a multiple of 16) is one box of
// [positions x 64 channels] per 64 channels, loaded by the same shifted 4-D TMA loads, and one MMA step
// reduces over 16 positions.  A CTA owns (128 output channels) x (BN input channels) x (up to three taps,
// one accumulator each in tensor memory) x (a contiguous share of the patches: split-K).  With more than one
// share per tile the epilogue adds its fp32 partial tile to a zero-initialised workspace with vector
// reductions, and the CTA that arrives last at the tile's counter converts the sum to bf16, writes the filter
// gradient and clears the words it used.
//
// All mbarrier waits have a time limit; on expiry the kernel raises a status word, drains its copies in
// flight, frees its tensor memory and returns.
//
// The reference has no convolution code (its benchmark calls cuDNN through torchvision,
// examples/pytorch_benchmark.py:100).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdio>
#include <cstdlib>

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
  static constexpr int kStages = (BN_ == 256) ? 4 : (BN_ == 128 ? 6 : 8);
  static constexpr uint32_t kBytesA = BM * BK * 2;          // room for 128 positions, the box may be smaller
  static constexpr uint32_t kBytesB = BN_ * BK * 2;
  static constexpr uint32_t kBytesStage = kBytesA + kBytesB;
  static constexpr uint32_t kCols = 2 * BN_ < 32 ? 32 : 2 * BN_;
  static constexpr uint32_t kBytesOutBox = BM * 64 * 2;     // [128 positions x 64 channels]
  static constexpr uint32_t kBytesOut = 2 * kBytesOutBox;
  static constexpr size_t kSmem = 1024 + size_t(kStages) * kBytesStage + kBytesOut + 256;
  static constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(BN_ >> 3) << 17) | (uint32_t(BM >> 4) << 24);
};

struct ConvGeom {
  int N, Ho, Wo, Cin, Cout;  // Cin: reduction channels per tap
  int Hy, Wy;                // extent of the output tensor
  int bw, bh, bn;            // patch extent (bw * bh * bn <= 128)
  int tiles_w, tiles_h, tiles_img, tiles_co;
  int T, in_stride, out_stride, out_ph, out_pw;
  signed char dh[kConvMaxTaps], dw[kConvMaxTaps];
  unsigned char wt[kConvMaxTaps];
};

__device__ __forceinline__ void epilogue_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// BMODE 0: the filter is [Cout, taps, Cin] and supplies K-major B tiles.  BMODE 1 (input-gradient form): the
// filter stays in the layout of the forward pass, [Cred, taps, Cout'] with the reduction channels outermost,
// and supplies MN-major B tiles: BN_/64 boxes of [64 reduction rows x 64 output channels] per stage.
// DIRECT 1: the epilogue stores each position's channels straight to y at (a*os + ph, b*os + pw).
constexpr int kIgemmThreads = 224;     // warps 0 and 6 produce, warp 1 issues the MMAs, warps 2-5 are the epilogue

template <int BN_, int BMODE, int DIRECT>
__global__ void __launch_bounds__(kIgemmThreads, 1)
conv_igemm_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                  const __grid_constant__ CUtensorMap map_y, const ConvGeom g, __nv_bfloat16* __restrict__ y,
                  unsigned int* __restrict__ status) {
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
  const int num_kb = g.T * cblocks;
  const uint32_t bytes_a = uint32_t(g.bw * g.bh * g.bn) * 128u;      // what one A box delivers

  if (threadIdx.x == 0) {
    failed_s = 0;
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(&bars[s]), 2);                // the activation producer and the filter producer
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

  // Two producer threads: the activation boxes and the filter boxes of a stage are issued by different warps, so
  // the two TMA instructions of a stage do not wait for one another; each arms the stage's barrier with its bytes.
  int armed = 0;
  if (warp == 0 || warp == 6) {
    if (lane == 0) {
      const bool filter_side = warp == 6;
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int co0, n0, h0, w0;
        tile_coords(tile, co0, n0, h0, w0);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int tap = kb / cblocks;
          const int ci0 = (kb % cblocks) * BK;
          const int s = it % S;
          if (!mbar_wait(smem_u32(&bars[S + s]), ((it / S) & 1) ^ 1, failed)) { ok = false; break; }
          const uint32_t full = smem_u32(&bars[s]);
          if (!filter_side) {
            mbar_expect_tx(full, bytes_a);
            tma_load_4d(smem_u32(stage_a + size_t(s) * Cfg::kBytesA), &map_x, full, ci0, w0 * g.in_stride + g.dw[tap],
                        h0 * g.in_stride + g.dh[tap], n0);
          } else {
            mbar_expect_tx(full, Cfg::kBytesB);
            const int wtap = g.wt[tap];
            if (BMODE == 0) {
              tma_load_2d(smem_u32(stage_b + size_t(s) * Cfg::kBytesB), &map_w, full, wtap * g.Cin + ci0, co0);
            } else {
#pragma unroll
              for (int j = 0; j < BN_ / 64; ++j)
                tma_load_2d(smem_u32(stage_b + size_t(s) * Cfg::kBytesB + size_t(j) * 8192), &map_w, full,
                            wtap * g.Cout + co0 + j * 64, ci0);
            }
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
  } else if (warp >= 2 && warp <= 5) {
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
      const int prow = q * 32 + lane;                                 // position of the patch
      // DIRECT: where this thread's position lands in y (null when it hangs over the grid)
      __nv_bfloat16* ypix = nullptr;
      if (DIRECT) {
        const int pw_ = prow % g.bw;
        const int ph_ = (prow / g.bw) % g.bh;
        const int pn_ = prow / (g.bw * g.bh);
        const int a = h0 + ph_, b = w0 + pw_, n = n0 + pn_;
        if (pn_ < g.bn && a < g.Ho && b < g.Wo && n < g.N) {
          const int hy = a * g.out_stride + g.out_ph, wy = b * g.out_stride + g.out_pw;
          if (hy < g.Hy && wy < g.Wy) ypix = y + ((size_t(n) * g.Hy + hy) * g.Wy + wy) * g.Cout;
        }
      }
#pragma unroll 1
      for (int c = 0; c < BN_ / 64; ++c) {
        const int cbase = co0 + c * 64;
        if (cbase >= g.Cout) break;                                   // uniform over the CTA
        uint32_t rr[64];
        const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + uint32_t(acc * BN_ + c * 64);
        tmem_ld32(taddr, rr);
        tmem_ld32(taddr + 32, rr + 32);
        if (DIRECT) {
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (ypix != nullptr) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              if (cbase + j * 8 < g.Cout) {                           // Cout is a multiple of 8
                uint4 pk;
                __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
                for (int i = 0; i < 4; ++i)
                  h[i] = __floats2bfloat162_rn(__uint_as_float(rr[j * 8 + 2 * i]), __uint_as_float(rr[j * 8 + 2 * i + 1]));
                *reinterpret_cast<uint4*>(ypix + cbase + j * 8) = pk;
              }
            }
          }
        } else {
          // the box staged two stores ago must have left shared memory before it is overwritten
          if (issuer) tma_store_wait_read<1>();
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          epilogue_bar();
          unsigned char* box = stage_out + size_t(boxes & 1) * Cfg::kBytesOutBox;
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
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&bars[2 * S + 2 + acc])) : "memory");
    }
    if (!DIRECT && issuer) tma_store_wait_all();
  }
  if ((warp == 0 || warp == 6) && lane == 0 && *failed) {
    // On the failure path a stage may have been armed by one producer only; its barrier then never completes and
    // the wait below runs into its limit, after which this producer's own copies have long landed.
    const int first = armed > S ? armed - S : 0;
    for (int it = first; it < armed; ++it) {
      const unsigned long long t0 = now_ns();
      while (!mbar_try(smem_u32(&bars[it % S]), (it / S) & 1) && now_ns() - t0 < kWaitLimitNs / 8) {}
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

// ------------------------------------------------------------------------------------------------------ //
// Filter gradient.
// ------------------------------------------------------------------------------------------------------ //
template <int BN_>
struct WgradCfg {
  // Shared memory is a pool of 13 boxes of up to 128 positions x 64 channels (16 KiB each), cut at launch into a
  // ring of output-gradient slots (one or two boxes: 64 or 128 output channels) and a ring of input slots (one box
  // per 64 input channels of the tile), as many patches deep as fit: what limits a split-K CTA is the latency of its
  // loads, so every byte of shared memory should be in flight.
  static constexpr int kPoolBoxes = 13;
  static constexpr uint32_t kBoxBytes = 128 * 128;
  static constexpr int kMaxBars = 64;
  static constexpr size_t kSmem = 1024 + size_t(kPoolBoxes) * kBoxBytes + kMaxBars * 8;
  // D fp32, A and B bf16, both MN-major (bits 15, 16), N = BN_, M = 128
  static constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | (1u << 16) |
                                     (uint32_t(BN_ >> 3) << 17) | (uint32_t(BM >> 4) << 24);
};

struct WgradGeom {
  int N, Ho, Wo, Cout, Cin;
  int bw, bh, bn, tiles_w, tiles_h, tiles_img;
  int T, in_stride;
  signed char dh[kConvMaxTaps], dw[kConvMaxTaps];
  unsigned char wt[kConvMaxTaps];
  int tiles_co, tiles_ci, groups, tg, splits;
  int ldw;                   // elements between filter-gradient rows: w_taps * Cin
  unsigned int tmem_cols;    // power of two >= tg * BN_
  int slots_a, slots_b;      // ring depths
  int boxes_a, boxes_b;      // boxes per slot
};

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.relaxed.gpu.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

template <int BN_>
__global__ void __launch_bounds__(kThreads, 1)
conv_wgrad_kernel(const __grid_constant__ CUtensorMap map_dy, const __grid_constant__ CUtensorMap map_x, const WgradGeom g,
                  __nv_bfloat16* __restrict__ dwt, float* __restrict__ ws, unsigned int* __restrict__ counters,
                  unsigned int* __restrict__ status) {
  using Cfg = WgradCfg<BN_>;
  const int SA = g.slots_a, SB = g.slots_b;
  const uint32_t bytes_slot_a = uint32_t(g.boxes_a) * Cfg::kBoxBytes, bytes_slot_b = uint32_t(g.boxes_b) * Cfg::kBoxBytes;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* stage_a = smem;
  unsigned char* stage_b = smem + size_t(SA) * bytes_slot_a;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + size_t(Cfg::kPoolBoxes) * Cfg::kBoxBytes);
  uint64_t* full_a = bars;
  uint64_t* empty_a = bars + SA;
  uint64_t* full_b = bars + 2 * SA;
  uint64_t* empty_b = bars + 2 * SA + SB;
  uint64_t* acc_full = bars + 2 * SA + 2 * SB;
  uint64_t* acc_empty = acc_full + 1;
  __shared__ uint32_t tmem_base_s;
  __shared__ int failed_s;
  __shared__ int go_s;
  __shared__ unsigned int ticket_s;
  volatile int* failed = &failed_s;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int patches = g.tiles_w * g.tiles_h * g.tiles_img;
  const int out_tiles = g.tiles_co * g.tiles_ci * g.groups;
  const int items = out_tiles * g.splits;
  const int positions = g.bw * g.bh * g.bn;                  // a multiple of 16
  const int ksteps = positions / kUmmaK;
  const uint32_t box_bytes = uint32_t(positions) * 128u;

  if (threadIdx.x == 0) {
    failed_s = 0;
    for (int s = 0; s < SA; ++s) {
      mbar_init(smem_u32(&full_a[s]), 1);
      mbar_init(smem_u32(&empty_a[s]), 1);
    }
    for (int s = 0; s < SB; ++s) {
      mbar_init(smem_u32(&full_b[s]), 1);
      mbar_init(smem_u32(&empty_b[s]), 1);
    }
    mbar_init(smem_u32(acc_full), 1);       // one tcgen05.commit
    mbar_init(smem_u32(acc_empty), 4);      // one arrive per epilogue warp
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(g.tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_s;

  // item -> output tile (co0, ci0, first tap of its group) and its share of the patches
  auto decode = [&](int item, int& co0, int& ci0, int& t0, int& t1, int& p0, int& p1, int& tile_id) {
    tile_id = item % out_tiles;
    const int split = item / out_tiles;
    const int co_t = tile_id % g.tiles_co;
    const int r = tile_id / g.tiles_co;
    const int ci_t = r % g.tiles_ci;
    const int grp = r / g.tiles_ci;
    co0 = co_t * BM;
    ci0 = ci_t * BN_;
    t0 = grp * g.tg;
    t1 = min(g.T, t0 + g.tg);
    p0 = int((long long)patches * split / g.splits);
    p1 = int((long long)patches * (split + 1) / g.splits);
  };
  auto patch_coords = [&](int p, int& n0, int& h0, int& w0) {
    w0 = (p % g.tiles_w) * g.bw;
    h0 = ((p / g.tiles_w) % g.tiles_h) * g.bh;
    n0 = (p / (g.tiles_w * g.tiles_h)) * g.bn;
  };

  int armed_a = 0, armed_b = 0;
  if (warp == 0) {
    if (lane == 0) {
      int ita = 0, itb = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < items && ok; item += gridDim.x) {
        int co0, ci0, t0, t1, p0, p1, tile_id;
        decode(item, co0, ci0, t0, t1, p0, p1, tile_id);
        const int boxes_a = min(2, (g.Cout - co0 + 63) / 64);
        const int boxes_b = min(BN_ / 64, (g.Cin - ci0 + 63) / 64);
        for (int p = p0; p < p1 && ok; ++p) {
          int n0, h0, w0;
          patch_coords(p, n0, h0, w0);
          {
            const int s = ita % SA;
            if (!mbar_wait(smem_u32(&empty_a[s]), ((ita / SA) & 1) ^ 1, failed)) { ok = false; break; }
            const uint32_t full = smem_u32(&full_a[s]);
            mbar_expect_tx(full, uint32_t(boxes_a) * box_bytes);
            for (int j = 0; j < boxes_a; ++j)
              tma_load_4d(smem_u32(stage_a + size_t(s) * bytes_slot_a + size_t(j) * Cfg::kBoxBytes), &map_dy, full,
                          co0 + j * 64, w0, h0, n0);
            armed_a = ++ita;
          }
          for (int t = t0; t < t1; ++t) {
            const int s = itb % SB;
            if (!mbar_wait(smem_u32(&empty_b[s]), ((itb / SB) & 1) ^ 1, failed)) { ok = false; break; }
            const uint32_t full = smem_u32(&full_b[s]);
            mbar_expect_tx(full, uint32_t(boxes_b) * box_bytes);
            for (int j = 0; j < boxes_b; ++j)
              tma_load_4d(smem_u32(stage_b + size_t(s) * bytes_slot_b + size_t(j) * Cfg::kBoxBytes), &map_x, full,
                          ci0 + j * 64, w0 * g.in_stride + g.dw[t], h0 * g.in_stride + g.dh[t], n0);
            armed_b = ++itb;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int ita = 0, itb = 0, local = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < items && ok; item += gridDim.x, ++local) {
        int co0, ci0, t0, t1, p0, p1, tile_id;
        decode(item, co0, ci0, t0, t1, p0, p1, tile_id);
        // the epilogue must have drained the accumulators of the previous item
        if (!mbar_wait(smem_u32(acc_empty), (local & 1) ^ 1, failed)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        for (int p = p0; p < p1 && ok; ++p) {
          const int sa = ita % SA;
          if (!mbar_wait(smem_u32(&full_a[sa]), (ita / SA) & 1, failed)) { ok = false; break; }
          ++ita;
          const uint64_t adesc = make_desc_mn(smem_u32(stage_a + size_t(sa) * bytes_slot_a), Cfg::kBoxBytes, 1024);
          for (int t = t0; t < t1; ++t) {
            const int sb = itb % SB;
            if (!mbar_wait(smem_u32(&full_b[sb]), (itb / SB) & 1, failed)) { ok = false; break; }
            ++itb;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t bdesc = make_desc_mn(smem_u32(stage_b + size_t(sb) * bytes_slot_b), Cfg::kBoxBytes, 1024);
            const uint32_t tmem_d = tmem_base + uint32_t((t - t0) * BN_);
            // one MMA step reduces over 16 positions = 16 rows of 128 bytes in both operands
            for (int k = 0; k < ksteps; ++k)
              umma_f16(tmem_d, adesc + uint64_t(k) * 128u, bdesc + uint64_t(k) * 128u, Cfg::kIdesc,
                       (p != p0 || k != 0) ? 1u : 0u);
            umma_commit(smem_u32(&empty_b[sb]));
          }
          if (ok) umma_commit(smem_u32(&empty_a[sa]));
        }
        if (ok) umma_commit(smem_u32(acc_full));
      }
    }
  } else {
    const int q = warp & 3;                  // accumulator lanes [32q, 32q + 32) = output channels co0 + 32q ...
    const bool leader = (warp == 2 && lane == 0);
    int local = 0;
    for (int item = blockIdx.x; item < items; item += gridDim.x, ++local) {
      int co0, ci0, t0, t1, p0, p1, tile_id;
      decode(item, co0, ci0, t0, t1, p0, p1, tile_id);
      mbar_wait(smem_u32(acc_full), local & 1, failed);
      epilogue_bar();
      if (leader) go_s = (*failed == 0);
      epilogue_bar();
      if (!*reinterpret_cast<volatile int*>(&go_s)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int co = co0 + q * 32 + lane;
      const bool row_ok = co < g.Cout;
      for (int t = t0; t < t1; ++t) {
        const size_t row_off = size_t(co) * g.ldw + size_t(g.wt[t]) * g.Cin;
#pragma unroll 1
        for (int c = 0; c < BN_ / 32; ++c) {
          const int col = ci0 + c * 32;
          if (col >= g.Cin) break;                                   // uniform; Cin is a multiple of 64
          uint32_t r[32];
          tmem_ld32(tmem_base + (uint32_t(q * 32) << 16) + uint32_t((t - t0) * BN_ + c * 32), r);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (!row_ok) continue;
          if (g.splits == 1) {
            __nv_bfloat16* dst = dwt + row_off + col;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 pk;
              __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
              for (int i = 0; i < 4; ++i)
                h[i] = __floats2bfloat162_rn(__uint_as_float(r[j * 8 + 2 * i]), __uint_as_float(r[j * 8 + 2 * i + 1]));
              *reinterpret_cast<uint4*>(dst + j * 8) = pk;
            }
          } else {
            float* dst = ws + row_off + col;
#pragma unroll
            for (int j = 0; j < 8; ++j)
              red_add_v4(dst + j * 4, __uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]),
                         __uint_as_float(r[4 * j + 3]));
          }
        }
      }
      // hand the accumulators back to the MMA warp
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(acc_empty)) : "memory");
      if (g.splits > 1) {
        // the CTA that adds the last share of this tile turns the fp32 sums into the bf16 filter gradient
        __threadfence();
        epilogue_bar();
        if (leader) ticket_s = atomicAdd(&counters[tile_id], 1u);
        epilogue_bar();
        if (*reinterpret_cast<volatile unsigned int*>(&ticket_s) == unsigned(g.splits - 1)) {
          __threadfence();
          // Every warp converts its 32 rows; a lane owns four consecutive columns.  The loads of a batch are issued
          // together: one L2 round trip per batch instead of one per 16 bytes.
          const int width = min(BN_, g.Cin - ci0);
          const int cchunks = (width + 127) / 128;
          const int ntaps = t1 - t0;
          const int total = 32 * ntaps * cchunks;              // (row, tap, column chunk) triples of this warp
          constexpr int kBatch = 16;
          for (int base = 0; base < total; base += kBatch) {
            float4 v[kBatch];
            size_t off[kBatch];
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
              const int i = base + u;
              const int cc = i % cchunks;
              const int t = t0 + (i / cchunks) % ntaps;
              const int row = co0 + q * 32 + i / (cchunks * ntaps);
              const int col = cc * 128 + lane * 4;
              const bool ok = i < total && row < g.Cout && col < width;
              off[u] = ok ? size_t(row) * g.ldw + size_t(g.wt[t]) * g.Cin + ci0 + col : size_t(-1);
              if (ok) v[u] = __ldcg(reinterpret_cast<const float4*>(ws + off[u]));
            }
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
              if (off[u] == size_t(-1)) continue;
              __stcg(reinterpret_cast<float4*>(ws + off[u]), make_float4(0.f, 0.f, 0.f, 0.f));
              uint2 pk;
              __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
              h[0] = __floats2bfloat162_rn(v[u].x, v[u].y);
              h[1] = __floats2bfloat162_rn(v[u].z, v[u].w);
              *reinterpret_cast<uint2*>(dwt + off[u]) = pk;
            }
          }
          if (leader) counters[tile_id] = 0u;
        }
        epilogue_bar();      // ticket_s is rewritten by the next item
      }
    }
  }
  if (warp == 0 && lane == 0 && *failed) {
    for (int it = armed_a > SA ? armed_a - SA : 0; it < armed_a; ++it) {
      const unsigned long long t0 = now_ns();
      while (!mbar_try(smem_u32(&full_a[it % SA]), (it / SA) & 1) && now_ns() - t0 < kWaitLimitNs) {}
    }
    for (int it = armed_b > SB ? armed_b - SB : 0; it < armed_b; ++it) {
      const unsigned long long t0 = now_ns();
      while (!mbar_try(smem_u32(&full_b[it % SB]), (it / SB) & 1) && now_ns() - t0 < kWaitLimitNs) {}
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(g.tmem_cols) : "memory");
  }
  if (threadIdx.x == 0 && failed_s && status != nullptr) atomicExch(status, 1u);
}

// 4-D map over a view [n, h, w, c]; a box of {64, bw, bh, bn} elements taken with traversal stride `stride`
// along w and h.
bool MakeViewMap(CUtensorMap* map, const ConvView& v, int bw, int bh, int bn, int stride) {
  const cuuint64_t dims[4] = {cuuint64_t(v.c), cuuint64_t(v.w), cuuint64_t(v.h), cuuint64_t(v.n)};
  const cuuint64_t strides[3] = {cuuint64_t(v.pix_pitch) * 2, cuuint64_t(v.row_pitch) * 2, cuuint64_t(v.img_pitch) * 2};
  const cuuint32_t box[4] = {64, cuuint32_t(bw * stride), cuuint32_t(bh * stride), cuuint32_t(bn)};
  const cuuint32_t estr[4] = {1, cuuint32_t(stride), cuuint32_t(stride), 1};
  if (box[1] > 256 || box[2] > 256 || box[3] > 256) return false;
  return EncodeTiled(map, 4, v.base, dims, strides, box, estr);
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

template <int BN_, int BMODE, int DIRECT>
cudaError_t LaunchIgemm(const CUtensorMap& mx, const CUtensorMap& mw, const CUtensorMap& my, const ConvGeom& g, void* y,
                        unsigned int* status, cudaStream_t stream) {
  using Cfg = ConvCfg<BN_>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(conv_igemm_kernel<BN_, BMODE, DIRECT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(Cfg::kSmem));
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  const int tiles = g.tiles_w * g.tiles_h * g.tiles_img * g.tiles_co;
  const int sms = SmCount();
  conv_igemm_kernel<BN_, BMODE, DIRECT><<<tiles < sms ? tiles : sms, kIgemmThreads, Cfg::kSmem, stream>>>(
      mx, mw, my, g, static_cast<__nv_bfloat16*>(y), status);
  CountKernelLaunch();
  return cudaGetLastError();
}

template <int BN_>
cudaError_t LaunchWgrad(const CUtensorMap& mdy, const CUtensorMap& mx, const WgradGeom& g, const WgradProblem& p,
                        unsigned int* status, cudaStream_t stream) {
  using Cfg = WgradCfg<BN_>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(conv_wgrad_kernel<BN_>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(Cfg::kSmem));
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  const int items = g.tiles_co * g.tiles_ci * g.groups * g.splits;
  const int sms = SmCount();
  conv_wgrad_kernel<BN_><<<items < sms ? items : sms, kThreads, Cfg::kSmem, stream>>>(
      mdy, mx, g, static_cast<__nv_bfloat16*>(p.dw), p.workspace, p.counters, status);
  CountKernelLaunch();
  return cudaGetLastError();
}

bool TapsOk(const ConvTaps& t, int w_taps) {
  if (t.T < 1 || t.T > kConvMaxTaps) return false;
  for (int i = 0; i < t.T; ++i)
    if (t.dh[i] < -128 || t.dh[i] > 127 || t.dw[i] < -128 || t.dw[i] > 127 || t.wt[i] < 0 || t.wt[i] >= w_taps) return false;
  return true;
}

bool ViewOk(const ConvView& v) {
  return v.base != nullptr && (reinterpret_cast<uintptr_t>(v.base) & 15) == 0 && v.n > 0 && v.h > 0 && v.w > 0 && v.c > 0 &&
         (v.pix_pitch % 8) == 0 && (v.row_pitch % 8) == 0 && (v.img_pitch % 8) == 0 && v.pix_pitch > 0;
}

}  // namespace

bool ConvPatch(int N, int H, int W, bool multiple_of_16, int* bw, int* bh, int* bn) {
  if (N <= 0 || H <= 0 || W <= 0 || W > 128) return false;
  // candidates: part of one image (bh rows, bh may hang over the last rows), or bn whole images of bh >= H rows
  long long best_cost = -1;
  int best_h = 0, best_n = 0;
  auto consider = [&](int h, int n) {
    const int px = W * h * n;
    if (px > 128 || (multiple_of_16 && (px % 16) != 0)) return;
    const long long th = (H + h - 1) / h, tn = (N + n - 1) / n;
    const long long cost = th * tn * 1000 + (128 - px);       // fewest patches first, then the fuller patch
    if (best_cost < 0 || cost < best_cost) {
      best_cost = cost;
      best_h = h;
      best_n = n;
    }
  };
  for (int h = 1; h <= H && W * h <= 128; ++h) consider(h, 1);
  for (int h = H; W * h <= 128 && h <= H + 15; ++h)
    for (int n = 1; n <= N && n <= 256 && W * h * n <= 128; ++n) consider(h, n);
  if (best_cost < 0) return false;
  *bw = W;
  *bh = best_h;
  *bn = best_n;
  return true;
}

bool ConvIgemmSupported(const ConvProblem& p) {
  int bw, bh, bn;
  if (GetEncodeFn() == nullptr || !ViewOk(p.x)) return false;
  if (p.x.c < 64 || (p.x.c % 64) != 0 || p.Cout < 8 || (p.Cout % 8) != 0) return false;
  if (p.filter_mode < 0 || p.filter_mode > 1 || !TapsOk(p.taps, p.w_taps)) return false;
  if (p.in_stride < 1 || p.in_stride > 2 || p.out_stride < 1 || p.out_stride > 2) return false;
  if (p.Ho <= 0 || p.Wo <= 0 || p.Hy <= 0 || p.Wy <= 0 || p.out_ph < 0 || p.out_pw < 0) return false;
  if (p.col_stats != nullptr) return false;
  return ConvPatch(p.x.n, p.Ho, p.Wo, false, &bw, &bh, &bn) && bw * p.in_stride <= 256 && bh * p.in_stride <= 256;
}

cudaError_t LaunchConvIgemm(const ConvProblem& p, unsigned int* status, cudaStream_t stream) {
  (void)cudaGetLastError();
  if (!ConvIgemmSupported(p) || p.w == nullptr || p.y == nullptr || (reinterpret_cast<uintptr_t>(p.w) & 15) ||
      (reinterpret_cast<uintptr_t>(p.y) & 15))
    return cudaErrorInvalidValue;
  ConvGeom g;
  g.N = p.x.n; g.Ho = p.Ho; g.Wo = p.Wo; g.Cin = p.x.c; g.Cout = p.Cout;
  g.Hy = p.Hy; g.Wy = p.Wy;
  g.T = p.taps.T; g.in_stride = p.in_stride; g.out_stride = p.out_stride; g.out_ph = p.out_ph; g.out_pw = p.out_pw;
  for (int i = 0; i < kConvMaxTaps; ++i) {
    g.dh[i] = static_cast<signed char>(i < g.T ? p.taps.dh[i] : 0);
    g.dw[i] = static_cast<signed char>(i < g.T ? p.taps.dw[i] : 0);
    g.wt[i] = static_cast<unsigned char>(i < g.T ? p.taps.wt[i] : 0);
  }
  ConvPatch(g.N, g.Ho, g.Wo, false, &g.bw, &g.bh, &g.bn);
  g.tiles_w = (g.Wo + g.bw - 1) / g.bw;
  g.tiles_h = (g.Ho + g.bh - 1) / g.bh;
  g.tiles_img = (g.N + g.bn - 1) / g.bn;
  const int spatial = g.tiles_w * g.tiles_h * g.tiles_img;
  // widest N tile that still occupies most of the SMs (a 256-wide tile streams half as many weight
  // bytes per FLOP through shared memory); narrow outputs take the narrow tile
  int bn_tile = 256;
  if (p.Cout <= 64) bn_tile = 64;
  else if (p.Cout <= 128 || spatial * ((p.Cout + 255) / 256) < (SmCount() * 3) / 4) bn_tile = 128;
  g.tiles_co = (p.Cout + bn_tile - 1) / bn_tile;
  const bool direct = !(p.out_stride == 1 && p.out_ph == 0 && p.out_pw == 0 && p.Hy == p.Ho && p.Wy == p.Wo);
  CUtensorMap mx, mw, my;
  // filter map: K-major [Cout rows, w_taps*Cin], or (MN-major mode) the forward filter [Cin rows, w_taps*Cout] in boxes of 64 x 64
  const bool mw_ok = p.filter_mode == 0 ? MakeMap2d(&mw, p.w, p.Cout, p.w_taps * g.Cin, bn_tile)
                                        : MakeMap2d(&mw, p.w, g.Cin, p.w_taps * p.Cout, 64);
  if (!MakeViewMap(&mx, p.x, g.bw, g.bh, g.bn, p.in_stride) || !mw_ok) return cudaErrorInvalidValue;
  ConvView yv{p.y, g.N, p.Hy, p.Wy, p.Cout, p.Cout, (long long)p.Wy * p.Cout, (long long)p.Hy * p.Wy * p.Cout};
  if (!direct) {
    if (!MakeViewMap(&my, yv, g.bw, g.bh, g.bn, 1)) return cudaErrorInvalidValue;
  } else {
    my = mx;       // unused by the direct epilogue
  }
#define BFB_CONV_LAUNCH(BNV)                                                                                          \
  (p.filter_mode == 0                                                                                                 \
       ? (direct ? LaunchIgemm<BNV, 0, 1>(mx, mw, my, g, p.y, status, stream) : LaunchIgemm<BNV, 0, 0>(mx, mw, my, g, p.y, status, stream)) \
       : (direct ? LaunchIgemm<BNV, 1, 1>(mx, mw, my, g, p.y, status, stream) : LaunchIgemm<BNV, 1, 0>(mx, mw, my, g, p.y, status, stream)))
  if (bn_tile == 64) return BFB_CONV_LAUNCH(64);
  if (bn_tile == 128) return BFB_CONV_LAUNCH(128);
  return BFB_CONV_LAUNCH(256);
#undef BFB_CONV_LAUNCH
}

namespace {

// Cuts the pool of 13 boxes into the two rings: as many whole patches (one output-gradient slot + tg input slots)
// as fit, at least two output-gradient slots, the rest to the input ring.
void WgradRings(int cout, int cin, int bn, int tg, int* boxes_a, int* boxes_b, int* slots_a, int* slots_b) {
  const int ba = cout > 64 ? 2 : 1;
  const int bb = (bn < cin ? bn : cin) / 64;
  int depth = 13 / (ba + tg * bb);
  if (depth > 6) depth = 6;
  int sa, sb;
  if (depth >= 2) {
    sa = depth;
    sb = (13 - sa * ba) / bb;
  } else {
    sa = 2;
    sb = (13 - 2 * ba) / bb;
  }
  if (sb > 16) sb = 16;
  *boxes_a = ba;
  *boxes_b = bb;
  *slots_a = sa;
  *slots_b = sb;
}

// Tile shape and split of a filter gradient: BN (input channels per tile), taps per group, shares of the patches.
// Every candidate is priced with a small model of one CTA's time line and the cheapest wins:
//   main loop   = patches of the CTA x max(bytes it loads per patch / what one SM draws from L2, MMA time)
//   reduction   = (more than one share per tile) vector reductions of the partial tile, a fence and a ticket, and the
//                 last CTA's conversion pass in batches of one L2 round trip each.
// Few taps per CTA mean more tiles and fewer shares (cheap reduction, but the output gradient is loaded once per
// tap); many taps per CTA share that load but reduce a wider tile.  BLUEFOG_B200_WGRAD_PLAN=bn,tg,splits overrides.
void WgradPlan(const WgradProblem& p, int patches, int positions, int* bn_tile, int* tg, int* splits) {
  const int cin = p.x.c, cout = p.dy.c, T = p.taps.T;
  const int sms = SmCount();
  if (const char* env = std::getenv("BLUEFOG_B200_WGRAD_PLAN")) {
    int b = 0, t = 0, s = 0;
    if (std::sscanf(env, "%d,%d,%d", &b, &t, &s) == 3 && (b == 64 || b == 128 || b == 256) && t >= 1 && t <= T &&
        t * b <= 512 && s >= 1) {
      *bn_tile = b;
      *tg = t;
      *splits = s > patches ? patches : s;
      return;
    }
  }
  const double kSmBytesPerNs = 150.0;        // what one SM's TMA loads sustain out of L2 (GB/s = bytes/ns)
  const double kClockGhz = 1.9;
  const double kRoundTripNs = 1000.0;        // one dependent L2 round trip under load
  const double kLoadLatencyNs = 1200.0;      // issue of a patch's loads to their arrival
  const double box = double(positions) * 128.0;
  const int ksteps = positions / kUmmaK;
  double best = -1.0;
  for (int b : {64, 128, 256}) {
    if (b > 64 && b > cin) continue;
    for (int t = 1; t <= T && t * b <= 512; ++t) {
      const int groups = (T + t - 1) / t;
      const int tiles_co = (cout + BM - 1) / BM, tiles_ci = (cin + b - 1) / b;
      const int tiles = tiles_co * tiles_ci * groups;
      int s = sms / tiles;
      if (s < 1) s = 1;
      if (s > patches) s = patches;
      const double items_per_cta = double((tiles * s + sms - 1) / sms);
      const double cta_patches = double((patches + s - 1) / s) * items_per_cta;
      const int boxes_a = cout >= BM ? 2 : (cout + 63) / 64;
      const int boxes_b = (b < cin ? b : cin) / 64;
      const double bytes = (boxes_a + double(t) * boxes_b) * box;
      const double mma_ns = double(t) * ksteps * (b / 2.0) / kClockGhz;
      const double load_ns = bytes / kSmBytesPerNs;
      int ba, bb, sa, sb;
      WgradRings(cout, cin, b, t, &ba, &bb, &sa, &sb);
      const double depth = double(sa < sb / t ? sa : (sb / t > 0 ? sb / t : 1));     // patches in flight
      const double latency_ns = (kLoadLatencyNs + mma_ns) / depth;
      double per_patch = load_ns > mma_ns ? load_ns : mma_ns;
      if (latency_ns > per_patch) per_patch = latency_ns;
      double ns = 3000.0 + cta_patches * per_patch + kRoundTripNs;
      if (s > 1) {
        const double reds = double(t) * b / 4.0;                  // 16-byte reductions per epilogue thread
        const double batches = double((32 * t * ((b + 127) / 128) + 15) / 16);
        ns += reds * 15.0 + 3.0 * kRoundTripNs + batches * kRoundTripNs;
      } else {
        ns += double(t) * b * 2.0;                               // direct bf16 stores
      }
      if (best < 0 || ns < best) {
        best = ns;
        *bn_tile = b;
        *tg = t;
        *splits = s;
      }
    }
  }
}

}  // namespace

bool ConvWgradSupported(const WgradProblem& p) {
  int bw, bh, bn;
  if (GetEncodeFn() == nullptr || !ViewOk(p.dy) || !ViewOk(p.x) || p.dy.pix_pitch != p.dy.c) return false;
  if (p.x.c < 64 || (p.x.c % 64) != 0 || p.dy.c < 8 || (p.dy.c % 8) != 0 || p.dy.n != p.x.n) return false;
  if (!TapsOk(p.taps, p.w_taps) || p.in_stride < 1 || p.in_stride > 2) return false;
  if (!ConvPatch(p.dy.n, p.dy.h, p.dy.w, true, &bw, &bh, &bn)) return false;
  return bw * p.in_stride <= 256 && bh * p.in_stride <= 256;
}

cudaError_t LaunchConvWgrad(const WgradProblem& p, unsigned int* status, cudaStream_t stream) {
  (void)cudaGetLastError();
  if (!ConvWgradSupported(p) || p.dw == nullptr || (reinterpret_cast<uintptr_t>(p.dw) & 15)) return cudaErrorInvalidValue;
  WgradGeom g;
  g.N = p.dy.n; g.Ho = p.dy.h; g.Wo = p.dy.w; g.Cout = p.dy.c; g.Cin = p.x.c;
  g.T = p.taps.T; g.in_stride = p.in_stride;
  for (int i = 0; i < kConvMaxTaps; ++i) {
    g.dh[i] = static_cast<signed char>(i < g.T ? p.taps.dh[i] : 0);
    g.dw[i] = static_cast<signed char>(i < g.T ? p.taps.dw[i] : 0);
    g.wt[i] = static_cast<unsigned char>(i < g.T ? p.taps.wt[i] : 0);
  }
  ConvPatch(g.N, g.Ho, g.Wo, true, &g.bw, &g.bh, &g.bn);
  g.tiles_w = (g.Wo + g.bw - 1) / g.bw;
  g.tiles_h = (g.Ho + g.bh - 1) / g.bh;
  g.tiles_img = (g.N + g.bn - 1) / g.bn;
  const int patches = g.tiles_w * g.tiles_h * g.tiles_img;
  int bn_tile;
  WgradPlan(p, patches, g.bw * g.bh * g.bn, &bn_tile, &g.tg, &g.splits);
  g.tiles_co = (g.Cout + BM - 1) / BM;
  g.tiles_ci = (g.Cin + bn_tile - 1) / bn_tile;
  g.groups = (g.T + g.tg - 1) / g.tg;
  g.ldw = p.w_taps * g.Cin;
  unsigned int cols = 32;
  while (cols < unsigned(g.tg * bn_tile)) cols <<= 1;
  g.tmem_cols = cols;
  WgradRings(g.Cout, g.Cin, bn_tile, g.tg, &g.boxes_a, &g.boxes_b, &g.slots_a, &g.slots_b);
  if (g.splits > 1) {
    const long long need = (long long)g.Cout * g.ldw;
    if (p.workspace == nullptr || p.counters == nullptr || p.workspace_floats < need ||
        p.n_counters < g.tiles_co * g.tiles_ci * g.groups || (reinterpret_cast<uintptr_t>(p.workspace) & 15))
      return cudaErrorInvalidValue;
  }
  CUtensorMap mdy, mx;
  if (!MakeViewMap(&mdy, p.dy, g.bw, g.bh, g.bn, 1) || !MakeViewMap(&mx, p.x, g.bw, g.bh, g.bn, p.in_stride))
    return cudaErrorInvalidValue;
  if (bn_tile == 64) return LaunchWgrad<64>(mdy, mx, g, p, status, stream);
  if (bn_tile == 128) return LaunchWgrad<128>(mdy, mx, g, p, status, stream);
  return LaunchWgrad<256>(mdy, mx, g, p, status, stream);
}

bool Conv3x3Supported(int N, int H, int W, int Cin, int Cout) {
  int bw, bh, bn;
  return GetEncodeFn() != nullptr && Cin >= 64 && (Cin % 64) == 0 && Cout >= 64 && (Cout % 8) == 0 &&
         ConvPatch(N, H, W, false, &bw, &bh, &bn);
}

cudaError_t LaunchConv3x3Nhwc(const void* x, const void* w, void* y, int N, int H, int W, int Cin, int Cout,
                              int flip_taps, int filter_mode, unsigned int* status, cudaStream_t stream) {
  if (!Conv3x3Supported(N, H, W, Cin, Cout)) return cudaErrorInvalidValue;
  ConvProblem p{};
  p.x = ConvView{x, N, H, W, Cin, Cin, (long long)W * Cin, (long long)H * W * Cin};
  p.w = w;
  p.filter_mode = filter_mode;
  p.w_taps = 9;
  p.y = y;
  p.Hy = H; p.Wy = W; p.Cout = Cout; p.Ho = H; p.Wo = W;
  p.out_stride = 1; p.out_ph = 0; p.out_pw = 0; p.in_stride = 1;
  p.taps.T = 9;
  for (int t = 0; t < 9; ++t) {
    p.taps.dh[t] = t / 3 - 1;
    p.taps.dw[t] = t % 3 - 1;
    p.taps.wt[t] = flip_taps ? 8 - t : t;
  }
  p.col_stats = nullptr;
  return LaunchConvIgemm(p, status, stream);
}

}  // namespace bfb
