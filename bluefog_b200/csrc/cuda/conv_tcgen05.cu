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
constexpr int kWgradMaxCluster = 8;       // portable cluster size

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
  // The tap tables are copied to shared memory with constant indices: indexing the kernel parameter with a loop
  // variable would move it to local memory, whose loads sit on the producers' critical path.
  __shared__ int tap_dh_s[kConvMaxTaps], tap_dw_s[kConvMaxTaps], tap_wt_s[kConvMaxTaps];
  volatile int* failed = &failed_s;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int spatial = g.tiles_w * g.tiles_h * g.tiles_img;
  const int num_tiles = spatial * g.tiles_co;
  const int cblocks = g.Cin / BK;
  const int num_kb = g.T * cblocks;
  const uint32_t bytes_a = uint32_t(g.bw * g.bh * g.bn) * 128u;      // what one A box delivers

  if (threadIdx.x == 0) {
#pragma unroll
    for (int i = 0; i < kConvMaxTaps; ++i) {
      tap_dh_s[i] = g.dh[i];
      tap_dw_s[i] = g.dw[i];
      tap_wt_s[i] = g.wt[i];
    }
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
        // (tap, 64-channel slice) advance by comparison: cblocks is a run-time value, and a division and a modulo
        // by it per stage are some fifty instructions in a loop that one thread runs alone
        int tap = 0, ci0 = 0;
        for (int kb = 0; kb < num_kb; ++kb, ++it, ci0 += BK) {
          if (ci0 == g.Cin) { ci0 = 0; ++tap; }
          const int s = it % S;
          if (!mbar_wait(smem_u32(&bars[S + s]), ((it / S) & 1) ^ 1, failed)) { ok = false; break; }
          const uint32_t full = smem_u32(&bars[s]);
          if (!filter_side) {
            mbar_expect_tx(full, bytes_a);
            tma_load_4d(smem_u32(stage_a + size_t(s) * Cfg::kBytesA), &map_x, full, ci0, w0 * g.in_stride + tap_dw_s[tap],
                        h0 * g.in_stride + tap_dh_s[tap], n0);
          } else {
            mbar_expect_tx(full, Cfg::kBytesB);
            const int wtap = tap_wt_s[tap];
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
          // (no tcgen05 fence here: the data arrived through the async proxy and its mbarrier, which the wait above
          // observed; the fence orders tcgen05 operations of different threads, e.g. the epilogue's loads of an accumulator)
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
// 3x3 / stride 1 / pad 1 with the input patch loaded once: conv_halo_kernel.
//
// The per-tap kernel above fetches the shifted input patch nine times.  Here a tile is a run of at most 128
// consecutive positions of the image *padded by one pixel on every side* (rows of Wp = W + 2 positions, bh rows
// per tile), and one TMA box of {64 channels, Wp, bh + 2 rows} per 64-channel slice brings the patch with its
// halo into shared memory as [(bh + 2) * Wp rows x 128 bytes].  Output position m of the tile then meets, for tap
// (dh, dw), patch row  m + (dh + 1) * Wp + (dw + 1):  the A operand of the tap is the same patch with the matrix
// descriptor's start address moved by that many rows of 128 bytes.  Such a start is not aligned to the 1024-byte
// period of the 128-byte swizzle; the tensor core applies the swizzle to the absolute shared-memory address, as
// TMA did when it wrote the patch, so the rows line up (base-offset field of the descriptor left at zero).
// Two of every Wp positions of a tile are padding columns: their accumulator rows are computed and dropped.
// The filter arrives tap by tap through its own ring, or - when all nine taps of the output-channel tile fit
// (64 -> 64 channels) - is loaded once per CTA and stays resident.
// ------------------------------------------------------------------------------------------------------ //
struct HaloGeom {
  int N, H, W, Cin, Cout;
  int Wp, bh, tiles_h, tiles_co;
  int T;
  signed char dh[kConvMaxTaps], dw[kConvMaxTaps];
  unsigned char wt[kConvMaxTaps];
  int slots_a, slots_b;            // ring depths (slots_b = 0: resident filter)
  unsigned int slot_bytes_a;       // multiple of 1024; room for the furthest row any tap reads
  unsigned int patch_bytes;        // what one box delivers
};

template <int BN_>
struct HaloCfg {
  static constexpr uint32_t kBytesB = BN_ * BK * 2;               // one tap, one 64-channel slice
  static constexpr uint32_t kCols = 2 * BN_ < 32 ? 32 : 2 * BN_;
  static constexpr int kMaxBars = 48;
  static constexpr size_t kSmemLimit = 226 * 1024;      // dynamic part; the kernel also has a few static words
  static constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(BN_ >> 3) << 17) | (uint32_t(BM >> 4) << 24);
};

#ifdef BFB_HALO_TRACE
__device__ unsigned long long g_halo_trace[160][16];
#define HTRACE(i) do { g_halo_trace[blockIdx.x][i] = now_ns(); } while (0)
#define HTRACE_ADD(i, v) do { g_halo_trace[blockIdx.x][i] += (unsigned long long)(v); } while (0)
#else
#define HTRACE(i) do {} while (0)
#define HTRACE_ADD(i, v) do {} while (0)
#endif

template <int BN_, int BMODE>
__global__ void __launch_bounds__(kIgemmThreads, 1)
conv_halo_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, const HaloGeom g,
                 __nv_bfloat16* __restrict__ y, unsigned int* __restrict__ status) {
  using Cfg = HaloCfg<BN_>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int SA = g.slots_a;
  const bool resident = g.slots_b == 0;
  const int cblocks = g.Cin / BK;
  const int SB = resident ? g.T * cblocks : g.slots_b;
  unsigned char* stage_a = smem;
  unsigned char* stage_b = smem + size_t(SA) * g.slot_bytes_a;
  uint64_t* bars = reinterpret_cast<uint64_t*>(stage_b + size_t(SB) * Cfg::kBytesB);
  uint64_t* full_a = bars;
  uint64_t* empty_a = bars + SA;
  uint64_t* full_b = bars + 2 * SA;            // resident: full_b[0] only
  uint64_t* empty_b = full_b + (resident ? 1 : SB);
  uint64_t* acc_full = empty_b + (resident ? 0 : SB);
  uint64_t* acc_empty = acc_full + 2;
  __shared__ uint32_t tmem_base_s;
  __shared__ int failed_s;
  __shared__ int go_s;
  volatile int* failed = &failed_s;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int spatial = g.N * g.tiles_h;
  const int num_tiles = spatial * g.tiles_co;

  if (threadIdx.x == 0) {
    HTRACE(0);
    failed_s = 0;
    for (int s = 0; s < SA; ++s) {
      mbar_init(smem_u32(&full_a[s]), 1);
      mbar_init(smem_u32(&empty_a[s]), 1);
    }
    if (resident) {
      mbar_init(smem_u32(&full_b[0]), 1);
    } else {
      for (int s = 0; s < SB; ++s) {
        mbar_init(smem_u32(&full_b[s]), 1);
        mbar_init(smem_u32(&empty_b[s]), 1);
      }
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&acc_full[a]), 1);
      mbar_init(smem_u32(&acc_empty[a]), 4);
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

  auto tile_coords = [&](int tile, int& co0, int& n, int& h0) {
    const int sp = tile / g.tiles_co;
    co0 = (tile % g.tiles_co) * BN_;
    h0 = (sp % g.tiles_h) * g.bh;
    n = sp / g.tiles_h;
  };
  // one filter tile: tap wt, 64-channel slice ci0, output channels co0 ...
  auto load_filter = [&](uint32_t dst, uint32_t bar, int wtap, int ci0, int co0) {
    if (BMODE == 0) {
      tma_load_2d(dst, &map_w, bar, wtap * g.Cin + ci0, co0);
    } else {
#pragma unroll
      for (int j = 0; j < BN_ / 64; ++j) tma_load_2d(dst + uint32_t(j) * 8192u, &map_w, bar, wtap * g.Cout + co0 + j * 64, ci0);
    }
  };

  int armed_a = 0, armed_b = 0;
  if (warp == 0) {
    // activation producer: one patch per 64-channel slice
    if (lane == 0) {
      // ring positions are kept as (slot, phase) pairs that wrap by comparison: the depths are run-time values, and
      // a modulo and a division by them per step are some fifty instructions in a loop that one thread runs alone
      int it = 0, s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int co0, n, h0;
        tile_coords(tile, co0, n, h0);
        for (int cb = 0; cb < cblocks; ++cb, ++it) {
          if (!mbar_wait(smem_u32(&empty_a[s]), ph ^ 1, failed)) { ok = false; break; }
          const uint32_t full = smem_u32(&full_a[s]);
          mbar_expect_tx(full, g.patch_bytes);
          tma_load_4d(smem_u32(stage_a + size_t(s) * g.slot_bytes_a), &map_x, full, cb * BK, -1, h0 - 1, n);
          armed_a = it + 1;
          if (++s == SA) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 6) {
    // filter producer
    if (lane == 0) {
      if (resident) {
        int co0, n, h0;
        tile_coords(blockIdx.x, co0, n, h0);
        const uint32_t full = smem_u32(&full_b[0]);
        mbar_expect_tx(full, uint32_t(SB) * Cfg::kBytesB);
#pragma unroll
        for (int t = 0; t < 9; ++t)
          for (int cb = 0; cb < cblocks; ++cb)
            load_filter(smem_u32(stage_b + size_t(t * cblocks + cb) * Cfg::kBytesB), full, g.wt[t], cb * BK, co0);
        armed_b = 1;
      } else {
        int it = 0, s = 0;
        uint32_t ph = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
          int co0, n, h0;
          tile_coords(tile, co0, n, h0);
          for (int cb = 0; cb < cblocks && ok; ++cb) {
#pragma unroll
            for (int t = 0; t < 9; ++t, ++it) {
              if (!mbar_wait(smem_u32(&empty_b[s]), ph ^ 1, failed)) { ok = false; break; }
              const uint32_t full = smem_u32(&full_b[s]);
              mbar_expect_tx(full, Cfg::kBytesB);
              load_filter(smem_u32(stage_b + size_t(s) * Cfg::kBytesB), full, g.wt[t], cb * BK, co0);
              armed_b = it + 1;
              if (++s == SB) { s = 0; ph ^= 1; }
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // This loop is run by one thread, and the tensor core idles while it computes: everything that can be is
      // prepared outside.  Ring positions are (slot, phase) pairs that wrap by comparison; barrier and stage
      // addresses are 32-bit shared-memory addresses kept incrementally; a descriptor is a constant high word and a
      // low word = constant + (address >> 4), so moving to the next tap, filter block or K step is one 32-bit add.
      int ita = 0, sa = 0, sb = 0, local = 0;
      uint32_t pha = 0, phb = 0;
      bool ok = true;
      const uint64_t a_proto = make_desc(0u);
      const uint64_t b_proto = BMODE == 0 ? make_desc(0u) : make_desc_mn(0u, 8192, 1024);
      const uint32_t a_hi = uint32_t(a_proto >> 32), b_hi = uint32_t(b_proto >> 32);
      const uint32_t a_lo0 = uint32_t(a_proto), b_lo0 = uint32_t(b_proto);
      uint32_t tap16[9];                                       // the nine taps' row offsets into the patch, >> 4
#pragma unroll
      for (int t = 0; t < 9; ++t) tap16[t] = uint32_t((g.dh[t] + 1) * g.Wp + (g.dw[t] + 1)) * 8u;
      const uint32_t stage_a16 = smem_u32(stage_a) >> 4, slot_a16 = g.slot_bytes_a >> 4;
      const uint32_t stage_b16 = smem_u32(stage_b) >> 4;
      constexpr uint32_t kB16 = Cfg::kBytesB >> 4;
      const uint32_t full_a0 = smem_u32(full_a), empty_a0 = smem_u32(empty_a);
      const uint32_t full_b0 = smem_u32(full_b), empty_b0 = smem_u32(empty_b);
      uint32_t a_cur16 = stage_a16, b_cur16 = stage_b16;       // follow sa and sb
      constexpr uint32_t idesc = Cfg::kIdesc | (BMODE != 0 ? (1u << 16) : 0u);
      constexpr uint32_t b_step = BMODE == 0 ? 2 : (16 * 128) >> 4;
      if (resident) ok = mbar_wait(full_b0, 0, failed);
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
        const int acc = local & 1;
#ifdef BFB_HALO_TRACE
        long long c0 = clock64();
#endif
        if (!mbar_wait(smem_u32(&acc_empty[acc]), ((local >> 1) & 1) ^ 1, failed)) { ok = false; break; }
#ifdef BFB_HALO_TRACE
        HTRACE_ADD(8, clock64() - c0);
#endif
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_d = tmem_base + uint32_t(acc * BN_);
        for (int cb = 0; cb < cblocks && ok; ++cb, ++ita) {
#ifdef BFB_HALO_TRACE
          c0 = clock64();
#endif
          if (!mbar_wait(full_a0 + 8u * uint32_t(sa), pha, failed)) { ok = false; break; }
#ifdef BFB_HALO_TRACE
          HTRACE_ADD(9, clock64() - c0);
          if (ita == 0) HTRACE(1);
#endif
          const uint32_t a_lo_patch = a_lo0 + a_cur16;
          if (resident) b_cur16 = stage_b16 + uint32_t(cb) * kB16;       // block (t, cb) sits at (t * cblocks + cb)
          // Nine taps, unrolled: the tap tables are then read at constant indices.
#pragma unroll
          for (int t = 0; t < 9; ++t) {
            if (!resident) {
#ifdef BFB_HALO_TRACE
              const long long c1 = clock64();
#endif
              if (!mbar_wait(full_b0 + 8u * uint32_t(sb), phb, failed)) { ok = false; break; }
#ifdef BFB_HALO_TRACE
              HTRACE_ADD(10, clock64() - c1);
#endif
            }
            // the tap's view of the patch: same rows, start moved by (dh + 1) * Wp + (dw + 1) rows of 128 bytes
            const uint32_t a_lo = a_lo_patch + tap16[t];
            const uint32_t b_lo = b_lo0 + b_cur16;
#pragma unroll
            for (int k = 0; k < BK / kUmmaK; ++k)
              umma_f16_split(tmem_d, a_lo + uint32_t(2 * k), a_hi, b_lo + b_step * uint32_t(k), b_hi, idesc,
                             (cb | t | k) != 0 ? 1u : 0u);
            if (resident) {
              b_cur16 += uint32_t(cblocks) * kB16;
            } else {
              umma_commit(empty_b0 + 8u * uint32_t(sb));
              b_cur16 += kB16;
              if (++sb == SB) { sb = 0; phb ^= 1; b_cur16 = stage_b16; }
            }
          }
          if (ok) umma_commit(empty_a0 + 8u * uint32_t(sa));
          a_cur16 += slot_a16;
          if (++sa == SA) { sa = 0; pha ^= 1; a_cur16 = stage_a16; }
        }
        if (ok) umma_commit(smem_u32(&acc_full[acc]));
        if (local < 4) HTRACE(2 + local);
      }
      HTRACE(6);
    }
  } else if (warp >= 2 && warp <= 5) {
    const int q = warp & 3;
    const bool leader = (warp == 2 && lane == 0);
    int local = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
      const int acc = local & 1;
      int co0, n, h0;
      tile_coords(tile, co0, n, h0);
      mbar_wait(smem_u32(&acc_full[acc]), (local >> 1) & 1, failed);
      epilogue_bar();
      if (leader) go_s = (*failed == 0);
      epilogue_bar();
      if (!*reinterpret_cast<volatile int*>(&go_s)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int m = q * 32 + lane;
      const int hh = h0 + m / g.Wp, ww = m % g.Wp;
      __nv_bfloat16* ypix = nullptr;
      if (m < g.bh * g.Wp && ww < g.W && hh < g.H) ypix = y + ((size_t(n) * g.H + hh) * g.W + ww) * g.Cout;
#pragma unroll 1
      for (int c = 0; c < BN_ / 64; ++c) {
        const int cbase = co0 + c * 64;
        if (cbase >= g.Cout) break;
        uint32_t rr[64];
        const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + uint32_t(acc * BN_ + c * 64);
        tmem_ld32(taddr, rr);
        tmem_ld32(taddr + 32, rr + 32);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (ypix != nullptr) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (cbase + j * 8 < g.Cout) {
              uint4 pk;
              __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
              for (int i = 0; i < 4; ++i)
                h[i] = __floats2bfloat162_rn(__uint_as_float(rr[j * 8 + 2 * i]), __uint_as_float(rr[j * 8 + 2 * i + 1]));
              *reinterpret_cast<uint4*>(ypix + cbase + j * 8) = pk;
            }
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&acc_empty[acc])) : "memory");
    }
  }
  if (*failed) {
    if (warp == 0 && lane == 0) {
      for (int it = armed_a > SA ? armed_a - SA : 0; it < armed_a; ++it) {
        const unsigned long long t0 = now_ns();
        while (!mbar_try(smem_u32(&full_a[it % SA]), (it / SA) & 1) && now_ns() - t0 < kWaitLimitNs / 8) {}
      }
    }
    if (warp == 6 && lane == 0) {
      const int nb = resident ? 1 : SB;
      for (int it = armed_b > nb ? armed_b - nb : 0; it < armed_b; ++it) {
        const unsigned long long t0 = now_ns();
        while (!mbar_try(smem_u32(&full_b[it % nb]), (it / nb) & 1) && now_ns() - t0 < kWaitLimitNs / 8) {}
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Cfg::kCols) : "memory");
  }
  if (threadIdx.x == 0 && failed_s && status != nullptr) atomicExch(status, 1u);
  if (threadIdx.x == 0) HTRACE(7);
}

// ------------------------------------------------------------------------------------------------------ //
// Filter gradient.
// ------------------------------------------------------------------------------------------------------ //
template <int BN_>
struct WgradCfg {
  // Shared memory is one pool cut at launch into ring stages of (output-gradient boxes + input boxes of the taps
  // of a group), as many as fit: what limits a split-K CTA is the latency of its loads, so every byte should be in
  // flight.  A box holds up to 128 positions x 64 channels.
  static constexpr uint32_t kPoolBytes = 216 * 1024;
  static constexpr int kMaxStages = 8;
  static constexpr size_t kSmem = 1024 + size_t(kPoolBytes) + (2 * kMaxStages + 5) * 8;
};

struct WgradGeom {
  int N, Ho, Wo, Cout, Cin;
  int bw, bh, bn, tiles_w, tiles_h, tiles_img;
  int T, in_stride;
  signed char dh[kConvMaxTaps], dw[kConvMaxTaps];
  unsigned char wt[kConvMaxTaps];
  int tiles_co, tiles_ci, groups, tg, splits;
  int spread;                // 1: every CTA of a tile converts a slice of it at the end (cooperative launch, one item per CTA)
  int cs, gs;                // splits = cs * gs: cs CTAs of one cluster reduce through shared memory, gs such clusters
                             // per tile add up in the fp32 workspace
  int ldw;                   // elements between filter-gradient rows: w_taps * Cin
  unsigned int tmem_cols;    // power of two >= tg * BN_
  int stages;                // ring depth
  int boxes_a, boxes_b;      // boxes per stage: output gradient (1 or 2), input per tap (BN_/64 at most)
  unsigned int box_stride;   // bytes between boxes
};

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.relaxed.gpu.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

__device__ __forceinline__ void st_cluster_v4(uint32_t cluster_addr, float a, float b, float c, float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(cluster_addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// Last step of the cluster reduction: the CS CTAs of the cluster have pushed their partial sums of this CTA's
// 128 / CS rows into its shared memory ([sender][row][pitch] floats); add them up and write them out (bf16 filter
// gradient, or fp32 reductions into the workspace when several clusters share the tile).
struct ClusterRows {
  const float* rx;          // receive buffer
  int n_cols, pitch;        // columns of the tile, floats per row
  int rank, co0, ci0, t0, te;
  int Cout, Cin, ldw;
  bool last;                // true: store bf16; false: reduce into the workspace
  const int* tap_wt;
  __nv_bfloat16* dwt;
  float* ws;
};
template <int BN_, int CS>
__device__ __forceinline__ void cluster_add_rows(const ClusterRows& c) {
  constexpr int rows_share = BM / CS;
  const int nf4 = c.n_cols >> 2;
  const int total = rows_share * nf4;
  for (int idx = c.te; idx < total; idx += 128) {
    const int row = idx / nf4, col = (idx % nf4) * 4;
    const float* at = c.rx + size_t(row) * c.pitch + col;
    float4 acc = *reinterpret_cast<const float4*>(at);
#pragma unroll
    for (int r = 1; r < CS; ++r) {
      const float4 v = *reinterpret_cast<const float4*>(at + size_t(r) * rows_share * c.pitch);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    const int co = c.co0 + c.rank * rows_share + row;
    const int ci = c.ci0 + col % BN_;
    if (co >= c.Cout || ci >= c.Cin) continue;
    const size_t off = size_t(co) * c.ldw + size_t(c.tap_wt[c.t0 + col / BN_]) * c.Cin + ci;
    if (c.last) {
      uint2 pk;
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
      h[0] = __floats2bfloat162_rn(acc.x, acc.y);
      h[1] = __floats2bfloat162_rn(acc.z, acc.w);
      *reinterpret_cast<uint2*>(c.dwt + off) = pk;
    } else {
      red_add_v4(c.ws + off, acc.x, acc.y, acc.z, acc.w);
    }
  }
}

#ifdef BFB_WGRAD_TRACE
__device__ unsigned long long g_wgrad_trace[160][16];
#define WTRACE(i) do { g_wgrad_trace[blockIdx.x][i] = now_ns(); } while (0)
#define WTRACE_ADD(i, v) do { g_wgrad_trace[blockIdx.x][i] += (v); } while (0)
#else
#define WTRACE(i) do {} while (0)
#define WTRACE_ADD(i, v) do {} while (0)
#endif

template <int BN_>
__global__ void __launch_bounds__(kThreads, 1)
conv_wgrad_kernel(const __grid_constant__ CUtensorMap map_dy, const __grid_constant__ CUtensorMap map_x, const WgradGeom g,
                  __nv_bfloat16* __restrict__ dwt, float* __restrict__ ws, unsigned int* __restrict__ counters,
                  unsigned int* __restrict__ status) {
  using Cfg = WgradCfg<BN_>;
  const int S = g.stages;
  const uint32_t box_stride = g.box_stride;                 // bytes between boxes: the box size rounded up to 1 KiB
  const uint32_t stage_bytes = uint32_t(g.boxes_a + g.tg * g.boxes_b) * box_stride;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kPoolBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + S;
  uint64_t* acc_full = bars + 2 * S;
  uint64_t* acc_empty = acc_full + 1;
  uint64_t* red_full = acc_full + 2;      // every CTA of the cluster is through with its MMAs (cs * 4 warp arrivals)
  uint64_t* red_done = acc_full + 3;      // every warp of the cluster has pushed its rows (cs * 4 arrivals)
  uint64_t* rd_done = acc_full + 4;       // this CTA's epilogue warps have read the receive buffer (4 arrivals)
  const int cs = g.cs;
  const uint32_t rank = cs > 1 ? cluster_ctarank() : 0u;
  __shared__ uint32_t tmem_base_s;
  __shared__ int failed_s;
  __shared__ int go_s;
  __shared__ unsigned int ticket_s;
  __shared__ int tap_dh_s[kConvMaxTaps], tap_dw_s[kConvMaxTaps], tap_wt_s[kConvMaxTaps];   // see conv_igemm_kernel
  volatile int* failed = &failed_s;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int patches = g.tiles_w * g.tiles_h * g.tiles_img;
  const int out_tiles = g.tiles_co * g.tiles_ci * g.groups;
  const int items = out_tiles * g.gs;
  const int positions = g.bw * g.bh * g.bn;                  // a multiple of 16
  const int ksteps = positions / kUmmaK;
  const uint32_t box_bytes = uint32_t(positions) * 128u;

  if (threadIdx.x == 0) {
    WTRACE(0);
#pragma unroll
    for (int i = 0; i < kConvMaxTaps; ++i) {
      tap_dh_s[i] = g.dh[i];
      tap_dw_s[i] = g.dw[i];
      tap_wt_s[i] = g.wt[i];
    }
    failed_s = 0;
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(&full[s]), 1);
      mbar_init(smem_u32(&empty[s]), 1);
    }
    mbar_init(smem_u32(acc_full), 1);       // one tcgen05.commit
    mbar_init(smem_u32(acc_empty), 4);      // one arrive per epilogue warp
    mbar_init(smem_u32(red_full), uint32_t(cs) * 4u);
    mbar_init(smem_u32(red_done), uint32_t(cs) * 4u);
    mbar_init(smem_u32(rd_done), 4);
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
  if (threadIdx.x == 0) WTRACE(1);
  if (cs > 1) {
    // no CTA may signal a peer's barriers before that peer has initialised them
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  }

  // item -> output tile (co0, ci0, first tap of its group) and its share of the patches
  // CTAs are numbered cluster by cluster; a cluster walks the (tile, share-of-the-clusters) items together and its
  // CTA `rank` takes share number (item / out_tiles) * cs + rank of the patches
  const int first_item = int(blockIdx.x) / cs, item_step = int(gridDim.x) / cs;
  auto decode = [&](int item, int& co0, int& ci0, int& t0, int& t1, int& p0, int& p1, int& tile_id) {
    tile_id = item % out_tiles;
    const int split = (item / out_tiles) * cs + int(rank);
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

  // One ring stage = one patch: the output-gradient boxes (64 channels each) followed by the input boxes of the
  // group's taps, tap after tap, every tap taking boxes_b boxes.  The taps of a group therefore form ONE B operand
  // of N = taps * BN_ columns (64-column groups box_stride apart), and a patch costs positions/16 MMAs in all
  // instead of that many per tap: with 64 input channels a 128x64x16 MMA keeps the tensor core a third busy,
  // a 128x192x16 one fully.
  int armed = 0;
  if (warp == 0) {
    if (lane == 0) {
      int it = 0, local = 0, s = 0;       // (slot, phase) wrap by comparison: S is a run-time value, see conv_halo_kernel
      uint32_t ph = 0;
      bool ok = true;
      for (int item = first_item; item < items && ok; item += item_step, ++local) {
        int co0, ci0, t0, t1, p0, p1, tile_id;
        decode(item, co0, ci0, t0, t1, p0, p1, tile_id);
        // the ring doubles as the receive buffer of the cluster reduction: what the peers pushed for the previous
        // item must have been read before new patches land on it
        if (cs > 1 && local > 0) {
          if (!mbar_wait(smem_u32(rd_done), (local - 1) & 1, failed)) break;
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // generic accesses before, TMA writes after
        }
        const int boxes_a = min(g.boxes_a, (g.Cout - co0 + 63) / 64);
        const int boxes_b = min(g.boxes_b, (g.Cin - ci0 + 63) / 64);
        for (int p = p0; p < p1; ++p, ++it) {
          int n0, h0, w0;
          patch_coords(p, n0, h0, w0);
#ifdef BFB_WGRAD_TRACE
          const unsigned long long tw0 = now_ns();
#endif
          if (!mbar_wait(smem_u32(&empty[s]), ph ^ 1, failed)) { ok = false; break; }
#ifdef BFB_WGRAD_TRACE
          WTRACE_ADD(10, now_ns() - tw0);
          if (it == 0) WTRACE(2);
#endif
          const uint32_t bar = smem_u32(&full[s]);
          unsigned char* stage = smem + size_t(s) * stage_bytes;
          mbar_expect_tx(bar, uint32_t(boxes_a + (t1 - t0) * boxes_b) * box_bytes);
          for (int j = 0; j < boxes_a; ++j)
            tma_load_4d(smem_u32(stage + size_t(j) * box_stride), &map_dy, bar, co0 + j * 64, w0, h0, n0);
          unsigned char* stage_b = stage + size_t(g.boxes_a) * box_stride;
          for (int t = t0; t < t1; ++t)
            for (int j = 0; j < boxes_b; ++j)
              tma_load_4d(smem_u32(stage_b + size_t((t - t0) * g.boxes_b + j) * box_stride), &map_x, bar, ci0 + j * 64,
                          w0 * g.in_stride + tap_dw_s[t], h0 * g.in_stride + tap_dh_s[t], n0);
          armed = it + 1;
          if (++s == S) { s = 0; ph ^= 1; }
        }
      }
      WTRACE(3);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int it = 0, local = 0, s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int item = first_item; item < items && ok; item += item_step, ++local) {
        int co0, ci0, t0, t1, p0, p1, tile_id;
        decode(item, co0, ci0, t0, t1, p0, p1, tile_id);
        // the epilogue must have drained the accumulators of the previous item
        if (!mbar_wait(smem_u32(acc_empty), (local & 1) ^ 1, failed)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // D fp32, A and B bf16, both MN-major (bits 15, 16), N = taps * BN_, M = 128
        const uint32_t n_cols = uint32_t(t1 - t0) * BN_;
        const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | (1u << 16) | ((n_cols >> 3) << 17) |
                               (uint32_t(BM >> 4) << 24);
        for (int p = p0; p < p1; ++p, ++it) {
#ifdef BFB_WGRAD_TRACE
          const unsigned long long tw0 = now_ns();
#endif
          if (!mbar_wait(smem_u32(&full[s]), ph, failed)) { ok = false; break; }
#ifdef BFB_WGRAD_TRACE
          WTRACE_ADD(11, now_ns() - tw0);
          if (it == 0) WTRACE(4);
#endif
          const uint32_t stage = smem_u32(smem + size_t(s) * stage_bytes);
          const uint64_t adesc = make_desc_mn(stage, box_stride, 1024);
          const uint64_t bdesc = make_desc_mn(stage + uint32_t(g.boxes_a) * box_stride, box_stride, 1024);
          // one MMA step reduces over 16 positions = 16 rows of 128 bytes in both operands
          for (int k = 0; k < ksteps; ++k)
            umma_f16(tmem_base, adesc + uint64_t(k) * 128u, bdesc + uint64_t(k) * 128u, idesc, (p != p0 || k != 0) ? 1u : 0u);
          umma_commit(smem_u32(&empty[s]));
          if (++s == S) { s = 0; ph ^= 1; }
        }
        if (ok) umma_commit(smem_u32(acc_full));
        WTRACE(5);
      }
    }
  } else {
    const int q = warp & 3;                  // accumulator lanes [32q, 32q + 32) = output channels co0 + 32q ...
    const bool leader = (warp == 2 && lane == 0);
    int local = 0;
    for (int item = first_item; item < items; item += item_step, ++local) {
      int co0, ci0, t0, t1, p0, p1, tile_id;
      decode(item, co0, ci0, t0, t1, p0, p1, tile_id);
      mbar_wait(smem_u32(acc_full), local & 1, failed);
      epilogue_bar();
      if (leader) go_s = (*failed == 0);
      epilogue_bar();
      if (!*reinterpret_cast<volatile int*>(&go_s)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (leader) WTRACE(6);
      if (cs > 1) {
        // ---- cluster reduction.  Rows [j * 128 / cs, (j + 1) * 128 / cs) of the tile belong to CTA j of the cluster.
        // 1: every CTA announces that its MMAs are done, i.e. that its ring may be overwritten by its peers
        const int n_cols = (t1 - t0) * BN_;
        const int pitch = n_cols + 4;       // four extra words keep the 16-byte stores of a warp (one row per lane) off each other's banks
        float* rx = reinterpret_cast<float*>(smem);
        __syncwarp();
        if (lane == 0)
          for (int r = 0; r < cs; ++r) mbar_arrive_cluster(mapa_u32(smem_u32(red_full), uint32_t(r)));
        mbar_wait_cluster(smem_u32(red_full), local & 1, failed);
        epilogue_bar();
        if (leader) go_s = (*failed == 0);
        epilogue_bar();
        if (!*reinterpret_cast<volatile int*>(&go_s)) break;
        // 2: the accumulator rows go straight from tensor memory into the owner's receive buffer
        // ([sender][row of the owner's share][pitch] floats) with remote shared-memory stores
        {
          const int rows_share = BM / cs;
          const int row = q * 32 + lane;
          const uint32_t owner = uint32_t(row / rows_share);
          const uint32_t dst = mapa_u32(smem_u32(rx + size_t(int(rank) * rows_share + row % rows_share) * pitch), owner);
#pragma unroll 1
          for (int c = 0; c < n_cols / 32; ++c) {
            uint32_t r[32];
            tmem_ld32(tmem_base + (uint32_t(q * 32) << 16) + uint32_t(c * 32), r);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int j = 0; j < 8; ++j)
              st_cluster_v4(dst + uint32_t(c * 32 + j * 4) * 4u, __uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                            __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
          }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        asm volatile("fence.acq_rel.cluster;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
          asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(acc_empty)) : "memory");
          for (int r = 0; r < cs; ++r) mbar_arrive_cluster(mapa_u32(smem_u32(red_done), uint32_t(r)));
        }
        // 3: when every warp of the cluster has pushed, this CTA adds up what it received
        mbar_wait_cluster(smem_u32(red_done), local & 1, failed);
        epilogue_bar();
        if (leader) go_s = (*failed == 0);
        epilogue_bar();
        if (!*reinterpret_cast<volatile int*>(&go_s)) break;
        if (leader) WTRACE(7);
        const int te = int(threadIdx.x) - 64;                    // 0..127 over the four epilogue warps
        const ClusterRows cr{rx, n_cols, pitch, int(rank), co0, ci0, t0, te, g.Cout, g.Cin, g.ldw, g.gs == 1,
                             tap_wt_s, dwt, ws};
        if (cs == 2) cluster_add_rows<BN_, 2>(cr);
        else if (cs == 4) cluster_add_rows<BN_, 4>(cr);
        else cluster_add_rows<BN_, 8>(cr);
        // the ring may take the next item's patches once these reads are over
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(rd_done)) : "memory");
      } else {
      const int co = co0 + q * 32 + lane;
      const bool row_ok = co < g.Cout;
      for (int t = t0; t < t1; ++t) {
        const size_t row_off = size_t(co) * g.ldw + size_t(tap_wt_s[t]) * g.Cin;
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
      if (leader) WTRACE(7);
      }
      if (g.gs > 1) {
        // fp32 sums of `rows` tile rows from `row_lo` on -> bf16 filter gradient, workspace words back to zero.  The
        // four warps interleave over (row, tap, 128-column chunk) triples; a lane owns four consecutive columns.
        // The loads of a batch are issued together: one L2 round trip per batch instead of one per 16 bytes.
        auto convert_rows = [&](int row_lo, int rows) {
          const int width = min(BN_, g.Cin - ci0);
          const int cchunks = (width + 127) / 128;
          const int ntaps = t1 - t0;
          const int total = rows * ntaps * cchunks;
          constexpr int kBatch = 16;
          for (int base = q; base < total; base += 4 * kBatch) {
            float4 v[kBatch];
            size_t off[kBatch];
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
              const int i = base + 4 * u;
              const int cc = i % cchunks;
              const int t = t0 + (i / cchunks) % ntaps;
              const int row = co0 + row_lo + i / (cchunks * ntaps);
              const int col = cc * 128 + lane * 4;
              const bool ok = i < total && row < g.Cout && col < width;
              off[u] = ok ? size_t(row) * g.ldw + size_t(tap_wt_s[t]) * g.Cin + ci0 + col : size_t(-1);
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
        };
        __threadfence();
        epilogue_bar();
        if (leader) ticket_s = atomicAdd(&counters[tile_id], 1u);
        epilogue_bar();
        if (g.spread) {
          // Cooperative launch, one item per CTA: all CTAs that share the tile are running, so each waits (bounded)
          // until every share has been added and converts its own slice of the rows, instead of the last one
          // converting the whole tile while the others have gone.
          if (leader) {
            bool ok = true;
            const long long t_start = clock64();
            unsigned polls = 0;
            for (;;) {
              unsigned seen;
              asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(counters + tile_id) : "memory");
              if (seen >= unsigned(g.splits)) break;
              if ((++polls & 31u) == 0u && (*failed || clock64() - t_start > kWaitLimitCycles)) {
                *failed = 1;
                ok = false;
                break;
              }
            }
            go_s = ok ? 1 : 0;
          }
          epilogue_bar();
          if (!*reinterpret_cast<volatile int*>(&go_s)) break;
          __threadfence();
          const int share = item / out_tiles;
          const int rows_share = (BM + g.splits - 1) / g.splits;
          const int row_lo = share * rows_share;
          convert_rows(row_lo, max(0, min(rows_share, BM - row_lo)));
          epilogue_bar();
          if (leader) {
            // the CTA that finishes its slice last re-arms the tile's counter
            const unsigned done = atomicAdd(&counters[tile_id], 1u);
            if (done == unsigned(2 * g.splits - 1)) counters[tile_id] = 0u;
          }
        } else if (*reinterpret_cast<volatile unsigned int*>(&ticket_s) == unsigned(g.splits - 1)) {
          // the CTA that adds the last share of this tile turns the fp32 sums into the bf16 filter gradient
          __threadfence();
          convert_rows(0, BM);
          if (leader) counters[tile_id] = 0u;
        }
        epilogue_bar();      // ticket_s is rewritten by the next item
        if (leader) WTRACE(8);
      }
    }
    // (a CTA leaves only after everything addressed to it has arrived, and nothing is pushed to a CTA that has
    // not announced its next item, so no shared memory is touched after its owner has gone)
  }
  if (warp == 0 && lane == 0 && *failed) {
    for (int it = armed > S ? armed - S : 0; it < armed; ++it) {
      const unsigned long long t0 = now_ns();
      while (!mbar_try(smem_u32(&full[it % S]), (it / S) & 1) && now_ns() - t0 < kWaitLimitNs) {}
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(g.tmem_cols) : "memory");
  }
  if (threadIdx.x == 0) WTRACE(9);
  if (threadIdx.x == 0 && failed_s && status != nullptr) atomicExch(status, 1u);
  if (threadIdx.x == 0) HTRACE(7);
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
  const int items = g.tiles_co * g.tiles_ci * g.groups * g.gs;          // each taken by one cluster of cs CTAs
  cudaLaunchConfig_t cfg{};
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = Cfg::kSmem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(g.cs);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g.cs > 1 ? 1 : 0;
  if (g.spread) {                                                       // never together with a cluster
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.numAttrs = 1;
  }
  int resident = SmCount();                                             // clusters (or single CTAs) that run at once
  if (g.cs > 1) {
    static int max_clusters[kWgradMaxCluster + 1] = {0};
    if (max_clusters[g.cs] == 0) {
      cfg.gridDim = dim3(static_cast<unsigned>(g.cs));
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, conv_wgrad_kernel<BN_>, &cfg) != cudaSuccess || n < 1) n = 1;
      (void)cudaGetLastError();
      max_clusters[g.cs] = n;
    }
    resident = max_clusters[g.cs];
  }
  const int clusters = items < resident ? items : resident;
  cfg.gridDim = dim3(static_cast<unsigned>(clusters * g.cs));
  cudaError_t e = cudaLaunchKernelEx(&cfg, conv_wgrad_kernel<BN_>, mdy, mx, g, static_cast<__nv_bfloat16*>(p.dw), p.workspace,
                                     p.counters, status);
  if (e != cudaSuccess && g.spread) {
    // the cooperative launch was refused: the same work with the last CTA of a tile converting all of it
    (void)cudaGetLastError();
    WgradGeom plain = g;
    plain.spread = 0;
    cfg.numAttrs = 0;
    e = cudaLaunchKernelEx(&cfg, conv_wgrad_kernel<BN_>, mdy, mx, plain, static_cast<__nv_bfloat16*>(p.dw), p.workspace,
                           p.counters, status);
  }
  CountKernelLaunch();
  return e != cudaSuccess ? e : cudaGetLastError();
}

// Clusters of `cs` CTAs (one CTA per SM) that the device runs at once, for the planner.  A cluster sits inside one
// GPC, so eight-CTA clusters leave some SMs idle.
int WgradResidentClusters(int cs) {
  static int cached[kWgradMaxCluster + 1] = {0};
  if (cs <= 1) return SmCount();
  if (cached[cs] == 0) {
    cudaLaunchConfig_t cfg{};
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = WgradCfg<64>::kSmem;
    cfg.gridDim = dim3(static_cast<unsigned>(cs));
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = static_cast<unsigned>(cs);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    (void)cudaFuncSetAttribute(conv_wgrad_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(WgradCfg<64>::kSmem));
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, conv_wgrad_kernel<64>, &cfg) != cudaSuccess || n < 1) n = SmCount() / cs / 2;
    (void)cudaGetLastError();
    cached[cs] = n < 1 ? 1 : n;
  }
  return cached[cs];
}

template <int BN_, int BMODE>
cudaError_t LaunchHalo(const CUtensorMap& mx, const CUtensorMap& mw, HaloGeom g, void* y, unsigned int* status,
                       cudaStream_t stream) {
  using Cfg = HaloCfg<BN_>;
  const int cblocks = g.Cin / BK;
  // filter: resident when all taps of the (single) output-channel tile fit beside a useful activation ring
  const size_t resident_bytes = size_t(g.T) * cblocks * Cfg::kBytesB;
  const bool resident = g.tiles_co == 1 && resident_bytes <= 80 * 1024;
  // Ring depths.  A patch feeds 36 MMAs (nine taps x four K steps), a filter block only four, so at the same
  // latency of a load the filter ring has to be about nine times as deep in blocks: three patch slots, and all the
  // rest of the shared memory for filter blocks (with four slots of 16 KB the 128-channel 28x28 layer waited for
  // filter blocks: 18 blocks per tile at four per load latency).  BLUEFOG_B200_HALO_SLOTS=a,b overrides.
  int want_a = 3;
  int want_b = 0;
  if (const char* env = std::getenv("BLUEFOG_B200_HALO_SLOTS")) {
    int a = 0, b = 0;
    if (std::sscanf(env, "%d,%d", &a, &b) == 2 && a >= 2 && a <= 6 && b >= 2 && b <= 16) { want_a = a; want_b = b; }
  }
  const size_t bars_bytes = Cfg::kMaxBars * 8;
  if (resident) {
    g.slots_b = 0;
  } else if (want_b > 0) {
    g.slots_b = want_b;
  } else {
    const size_t left = Cfg::kSmemLimit - 1024 - bars_bytes - size_t(want_a) * g.slot_bytes_a;
    int sb = int(left / Cfg::kBytesB);
    if (sb > 16) sb = 16;
    if (sb < 2) sb = 2;
    g.slots_b = sb;
  }
  if (!resident && 2 * (want_a + g.slots_b) + 4 > Cfg::kMaxBars) g.slots_b = (Cfg::kMaxBars - 4) / 2 - want_a;
  const size_t bytes_b = resident ? resident_bytes : size_t(g.slots_b) * Cfg::kBytesB;
  const size_t fixed = 1024 + bytes_b + bars_bytes;
  if (fixed + 2 * size_t(g.slot_bytes_a) > Cfg::kSmemLimit) return cudaErrorInvalidValue;
  int sa = int((Cfg::kSmemLimit - fixed) / g.slot_bytes_a);
  if (sa > (resident ? 6 : want_a)) sa = resident ? 6 : want_a;
  g.slots_a = sa;
  const size_t smem = fixed + size_t(sa) * g.slot_bytes_a;
  static size_t attr_bytes = 0;
  if (smem > attr_bytes) {
    cudaError_t e = cudaFuncSetAttribute(conv_halo_kernel<BN_, BMODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(Cfg::kSmemLimit));
    if (e != cudaSuccess) return e;
    attr_bytes = Cfg::kSmemLimit;
  }
  const int tiles = g.N * g.tiles_h * g.tiles_co;
  const int sms = SmCount();
  conv_halo_kernel<BN_, BMODE><<<tiles < sms ? tiles : sms, kIgemmThreads, smem, stream>>>(
      mx, mw, g, static_cast<__nv_bfloat16*>(y), status);
  CountKernelLaunch();
  return cudaGetLastError();
}

// Whether the problem is a dense 3x3-neighbourhood convolution the halo kernel covers well: unit strides, taps within
// one pixel, the whole padded row inside one box, and tiles that are at least three quarters real positions.
bool HaloApplies(const ConvProblem& p, int* bh_out) {
  if (p.in_stride != 1 || p.out_stride != 1 || p.out_ph != 0 || p.out_pw != 0) return false;
  if (p.Hy != p.Ho || p.Wy != p.Wo || p.x.h != p.Ho || p.x.w != p.Wo || p.x.pix_pitch != p.x.c) return false;
  if (p.taps.T != 9) return false;            // the kernel's tap loop is unrolled for a 3x3 filter
  for (int t = 0; t < p.taps.T; ++t)
    if (p.taps.dh[t] < -1 || p.taps.dh[t] > 1 || p.taps.dw[t] < -1 || p.taps.dw[t] > 1) return false;
  const int Wp = p.Wo + 2;
  if (Wp > 128) return false;
  int bh = 128 / Wp;
  if (bh > p.Ho) bh = p.Ho;
  if (bh < 1 || bh * p.Wo < 96) return false;
  static const bool off = [] { const char* e = std::getenv("BLUEFOG_B200_CONV_HALO"); return e != nullptr && e[0] == '0'; }();
  if (off) return false;
  *bh_out = bh;
  return true;
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
  int halo_bh = 0;
  if (HaloApplies(p, &halo_bh)) {
    HaloGeom hg;
    hg.N = g.N; hg.H = p.Ho; hg.W = p.Wo; hg.Cin = g.Cin; hg.Cout = p.Cout;
    hg.Wp = p.Wo + 2; hg.bh = halo_bh;
    hg.tiles_h = (p.Ho + halo_bh - 1) / halo_bh;
    hg.T = g.T;
    for (int i = 0; i < kConvMaxTaps; ++i) { hg.dh[i] = g.dh[i]; hg.dw[i] = g.dw[i]; hg.wt[i] = g.wt[i]; }
    const int spatial_h = g.N * hg.tiles_h;
    int bn_h = 256;
    if (p.Cout <= 64) bn_h = 64;
    else if (p.Cout <= 128 || spatial_h * ((p.Cout + 255) / 256) < (SmCount() * 3) / 4) bn_h = 128;
    hg.tiles_co = (p.Cout + bn_h - 1) / bn_h;
    const int patch_rows = (halo_bh + 2) * hg.Wp;
    int slot_rows = 2 * hg.Wp + 2 + 128;
    if (slot_rows < patch_rows) slot_rows = patch_rows;
    hg.slot_bytes_a = (unsigned(slot_rows) * 128u + 1023u) & ~1023u;
    hg.patch_bytes = unsigned(patch_rows) * 128u;
    hg.slots_a = hg.slots_b = 0;
    CUtensorMap hx, hw;
    const bool hw_ok = p.filter_mode == 0 ? MakeMap2d(&hw, p.w, p.Cout, p.w_taps * g.Cin, bn_h)
                                          : MakeMap2d(&hw, p.w, g.Cin, p.w_taps * p.Cout, 64);
    if (MakeViewMap(&hx, p.x, hg.Wp, halo_bh + 2, 1, 1) && hw_ok) {
      cudaError_t e;
      if (bn_h == 64) e = p.filter_mode == 0 ? LaunchHalo<64, 0>(hx, hw, hg, p.y, status, stream) : LaunchHalo<64, 1>(hx, hw, hg, p.y, status, stream);
      else if (bn_h == 128) e = p.filter_mode == 0 ? LaunchHalo<128, 0>(hx, hw, hg, p.y, status, stream) : LaunchHalo<128, 1>(hx, hw, hg, p.y, status, stream);
      else e = p.filter_mode == 0 ? LaunchHalo<256, 0>(hx, hw, hg, p.y, status, stream) : LaunchHalo<256, 1>(hx, hw, hg, p.y, status, stream);
      return e;
    }
  }
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

// Ring geometry of a filter gradient: boxes per stage and how many stages fit into the pool.
void WgradRings(int cout, int cin, int bn, int tg, int positions, int* boxes_a, int* boxes_b, unsigned* box_stride,
                int* stages) {
  const int ba = cout > 64 ? 2 : 1;
  const int bb = (bn < cin ? bn : cin) / 64;
  const unsigned stride = (unsigned(positions) * 128u + 1023u) & ~1023u;
  int s = int(WgradCfg<64>::kPoolBytes / (size_t(ba + tg * bb) * stride));
  if (s > WgradCfg<64>::kMaxStages) s = WgradCfg<64>::kMaxStages;
  *boxes_a = ba;
  *boxes_b = bb;
  *box_stride = stride;
  *stages = s;
}

// Tile shape and split of a filter gradient: BN (input channels per tile), taps per group, and how the patches are
// shared out: cs CTAs of one cluster, times gs clusters.  The taps of a group are columns of one MMA (N = taps * BN
// <= 256), so more taps per group cost no extra MMA instructions and share the load of the output gradient; they
// widen the tile that is reduced at the end.  Every candidate is priced with a small model of one CTA's time line and
// the cheapest wins:
//   main loop   = patches of the CTA x max(bytes per patch / what one SM draws from L2, MMA time, load latency / depth)
//   reduction   = within a cluster: park the tile in shared memory, add up a 1/cs share of its rows from the peers;
//                 across clusters (gs > 1): vector reductions of that share into the workspace, a fence and a ticket,
//                 and the last CTA's conversion pass in batches of one L2 round trip each.
// BLUEFOG_B200_WGRAD_PLAN=bn,tg,cs,gs overrides.
void WgradPlan(const WgradProblem& p, int patches, int positions, int* bn_tile, int* tg, int* cs_out, int* gs_out) {
  const int cin = p.x.c, cout = p.dy.c, T = p.taps.T;
  if (const char* env = std::getenv("BLUEFOG_B200_WGRAD_PLAN")) {
    int b = 0, t = 0, c = 0, s = 0;
    if (std::sscanf(env, "%d,%d,%d,%d", &b, &t, &c, &s) == 4 && (b == 64 || b == 128 || b == 256) && t >= 1 && t <= T &&
        t * b <= 256 && (c == 1 || c == 2 || c == 4 || c == 8) && s >= 1 && c * s <= patches) {
      int ba, bb, st;
      unsigned stride;
      WgradRings(cout, cin, b, t, positions, &ba, &bb, &stride, &st);
      if (st >= 2) {
        *bn_tile = b;
        *tg = t;
        *cs_out = c;
        *gs_out = s;
        return;
      }
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
    for (int t = 1; t <= T && t * b <= 256; ++t) {
      int ba, bb, stages;
      unsigned stride;
      WgradRings(cout, cin, b, t, positions, &ba, &bb, &stride, &stages);
      if (stages < 2) continue;
      const int groups = (T + t - 1) / t;
      const int tiles_co = (cout + BM - 1) / BM, tiles_ci = (cin + b - 1) / b;
      const int tiles = tiles_co * tiles_ci * groups;
      for (int cs = 1; cs <= kWgradMaxCluster; cs *= 2) {
        if (cs > patches) break;
        const int resident = WgradResidentClusters(cs);       // clusters running at once
        int gs = resident / tiles;
        if (gs < 1) gs = 1;
        if (cs * gs > patches) gs = patches / cs;
        if (gs < 1) continue;
        // Measured: the cluster form wins where a CTA's share of the reduction is short (at most 16 patches) and the
        // cluster alone gives all the splits the tile needs; clusters of eight and clusters combined with workspace
        // splits lost against plain workspace splits on every ResNet-50 and GPT-2 shape tried.
        if (cs > 1 && (cs > 4 || gs != 1 || (patches + cs - 1) / cs > 16)) continue;
        const int s = cs * gs;
        const double rounds = double((tiles * gs + resident - 1) / resident);
        const double cta_patches = double((patches + s - 1) / s) * rounds;
        const double bytes = (ba + double(t) * bb) * box;
        double mma_clk = double(t) * b / 2.0;                      // one 128 x (t*b) x 16 MMA
        if (mma_clk < 60.0) mma_clk = 60.0;                        // floor of a small MMA
        const double mma_ns = ksteps * mma_clk / kClockGhz;
        const double load_ns = bytes / kSmBytesPerNs;
        const double latency_ns = (kLoadLatencyNs + mma_ns) / stages;
        double per_patch = load_ns > mma_ns ? load_ns : mma_ns;
        if (latency_ns > per_patch) per_patch = latency_ns;
        double ns = 3000.0 + cta_patches * per_patch + kRoundTripNs;
        const double tile_floats = 128.0 * t * b;
        // pushing (cs - 1) / cs of the tile through distributed shared memory runs at some 15 bytes/ns per SM in the
        // all-to-all pattern of this step; the constants are scaled like those of the workspace path below, which
        // this model prices at about half of what it measures
        if (cs > 1) ns += 700.0 + tile_floats * 4.0 * (cs - 1) / cs / 32.0 + tile_floats / cs * 0.18;
        if (gs > 1) {
          const double reds = tile_floats / cs / 4.0 / 128.0;      // 16-byte reductions per epilogue thread
          double batches = double((32 * t * ((b + 127) / 128) + 15) / 16);
          if (cs == 1 && tiles * gs <= SmCount()) batches = double(int(batches) / gs + 1);     // every CTA converts a slice
          ns += reds * 15.0 + 3.0 * kRoundTripNs + batches * kRoundTripNs;
        } else if (cs == 1) {
          ns += double(t) * b * 2.0;                               // direct bf16 stores
        }
        if (best < 0 || ns < best) {
          best = ns;
          *bn_tile = b;
          *tg = t;
          *cs_out = cs;
          *gs_out = gs;
        }
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
  WgradPlan(p, patches, g.bw * g.bh * g.bn, &bn_tile, &g.tg, &g.cs, &g.gs);
  g.splits = g.cs * g.gs;
  g.spread = 0;      // set below
  g.tiles_co = (g.Cout + BM - 1) / BM;
  g.tiles_ci = (g.Cin + bn_tile - 1) / bn_tile;
  g.groups = (g.T + g.tg - 1) / g.tg;
  g.ldw = p.w_taps * g.Cin;
  {
    static const bool spread_off = [] { const char* e = std::getenv("BLUEFOG_B200_WGRAD_SPREAD"); return e != nullptr && e[0] == '0'; }();
    static const bool coop = [] {
      int dev = 0, v = 0;
      cudaGetDevice(&dev);
      cudaDeviceGetAttribute(&v, cudaDevAttrCooperativeLaunch, dev);
      return v != 0;
    }();
    g.spread = (!spread_off && coop && g.cs == 1 && g.gs > 1 && g.tiles_co * g.tiles_ci * g.groups * g.gs <= SmCount()) ? 1 : 0;
  }
  unsigned int cols = 32;
  while (cols < unsigned(g.tg * bn_tile)) cols <<= 1;
  g.tmem_cols = cols;
  WgradRings(g.Cout, g.Cin, bn_tile, g.tg, g.bw * g.bh * g.bn, &g.boxes_a, &g.boxes_b, &g.box_stride, &g.stages);
  if (g.stages < 2) return cudaErrorInvalidValue;
  if (g.gs > 1) {
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
