// bf16 GEMM on Blackwell's 5th-generation tensor cores:  C[M,N] = act(A[M,K] * B[N,K]^T + bias).
//
// One CTA computes one 128 x 128 output tile.  Warp 0 is the TMA producer: it streams
// 128x64 tiles of A and B (K-major, 128-byte swizzle) into a 6-stage shared-memory ring with
// `cp.async.bulk.tensor.2d` (no cluster multicast).  Warp 1 allocates 128 columns of tensor
// memory and issues `tcgen05.mma.cta_group::1.kind::f16` (M=128, N=128, K=16) from one
// elected lane, accumulating in fp32 in TMEM, and releases ring stages with
// `tcgen05.commit`.  Warps 2-5 are the epilogue: once the accumulator is complete they read
// it back with `tcgen05.ld.32x32b.x32`, add the bias, apply the activation, convert to bf16
// and store.  Producer, MMA issuer and epilogue run concurrently and synchronise only
// through mbarriers.  Every mbarrier wait has a time limit: on expiry the kernel records an
// error code, stops issuing work, waits (bounded) for its TMA copies in flight, frees its TMEM
// and returns.
//
// That is the one-tile-per-CTA kernel (gemm_bf16_nt_kernel).  The default is the persistent kernel further
// down: one CTA per SM walks 128 x 128/256 tiles in groups of eight tile rows, the accumulator is
// double-buffered in TMEM so that the epilogue of one tile overlaps the MMAs of the next, the output leaves
// through swizzled staging boxes and TMA stores, and operands may be K-major or MN-major (NT, NN, TN
// products).  Its epilogue mode is a template parameter: bias + activation; pre-activation and GELU in one
// pass; product times GELU'(saved pre-activation); column sums and sums of squares of the output for a
// following BatchNorm.
//
// The reference has no GEMM of its own (its models call cuBLAS through PyTorch,
// examples/pytorch_benchmark.py:76-100); this kernel is what the models of this library use for
// their linear layers and 1x1 convolutions.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdlib>
#include <string>

#include "gemm_tcgen05.h"
#include "tcgen05_common.cuh"
#include "comm_kernels.h"

namespace bfb {
namespace {

using namespace t5;

constexpr int BM = 128, BN = 128, BK = 64;
constexpr int kStages = 6;
constexpr int kUmmaK = 16;
constexpr int kThreads = 192;
constexpr uint32_t kStageBytesA = BM * BK * 2;
constexpr uint32_t kStageBytesB = BN * BK * 2;
constexpr uint32_t kStageBytes = kStageBytesA + kStageBytesB;
constexpr uint32_t kTmemCols = 128;
constexpr size_t kSmemBytes = 1024 /*alignment slack*/ + size_t(kStages) * kStageBytes + 256 /*barriers*/;

// Instruction descriptor: D=f32, A=B=bf16, both K-major, N=128, M=128.
constexpr uint32_t kInstrDesc = (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(BN >> 3) << 17) | (uint32_t(BM >> 4) << 24);

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(kInstrDesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ float act_fn(float x, int act) {
  if (act == kActRelu) return fmaxf(x, 0.f);
  if (act == kActGeluTanh) {
    const float c = 0.7978845608028654f;
    return 0.5f * x * (1.f + tanhf(c * (x + 0.044715f * x * x * x)));
  }
  return x;
}

// Order in which the persistent kernel walks the output tiles: groups of eight tile rows, inside a group the
// row index runs fastest.  The CTAs that are resident together then share 8 A panels and about tiles/8 B panels
// instead of one or two A panels and every B panel, so a B matrix larger than L2 (a 50 304-column classifier)
// is streamed from DRAM once per group of eight tile rows rather than once per tile row.
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  constexpr int kGroup = 8;
  const int per_group = kGroup * tiles_n;
  const int gid = tile / per_group;
  const int first = gid * kGroup;
  const int rows = min(tiles_m - first, kGroup);
  const int r = tile - gid * per_group;
  tm = first + r % rows;
  tn = r / rows;
}

// two floats in one 64-bit register, the operand form of the packed f32x2 instructions
__device__ __forceinline__ unsigned long long pack_f32x2(uint32_t lo_bits, uint32_t hi_bits) {
  unsigned long long v;
  asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "r"(lo_bits), "r"(hi_bits));
  return v;
}
__device__ __forceinline__ void unpack_f32x2(unsigned long long v, float& lo, float& hi) {
  uint32_t a, b;
  asm("mov.b64 {%0, %1}, %2;" : "=r"(a), "=r"(b) : "l"(v));
  lo = __uint_as_float(a);
  hi = __uint_as_float(b);
}

// d/dx of the tanh-approximated GELU of act_fn
__device__ __forceinline__ float gelu_tanh_grad(float x) {
  const float c = 0.7978845608028654f;
  const float u = c * (x + 0.044715f * x * x * x);
  const float t = tanhf(u);
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * c * (1.f + 3.f * 0.044715f * x * x);
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_nt_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ bias, int M, int N, int K,
                    int act, unsigned int* __restrict__ status) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* stage_a = smem;
  unsigned char* stage_b = smem + size_t(kStages) * kStageBytesA;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + size_t(kStages) * kStageBytes);
  // bars[0..S): full, bars[S..2S): empty, bars[2S]: accumulator complete
  __shared__ uint32_t tmem_base_s;
  __shared__ int failed_s;
  volatile int* failed = &failed_s;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * BM;
  const int n0 = blockIdx.x * BN;
  const int num_kb = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    failed_s = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&bars[s]), 1);
      mbar_init(smem_u32(&bars[kStages + s]), 1);
    }
    mbar_init(smem_u32(&bars[2 * kStages]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_s;

  int armed = 0;  // producer: stages whose TMA copies were issued (for the failure path)
  if (warp == 0) {
    if (lane == 0) {
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % kStages;
        const uint32_t parity = ((kb / kStages) & 1) ^ 1;
        if (!mbar_wait(smem_u32(&bars[kStages + s]), parity, failed)) break;
        const uint32_t full = smem_u32(&bars[s]);
        mbar_expect_tx(full, kStageBytes);
        tma_load_2d(smem_u32(stage_a + size_t(s) * kStageBytesA), &map_a, full, kb * BK, m0);
        tma_load_2d(smem_u32(stage_b + size_t(s) * kStageBytesB), &map_b, full, kb * BK, n0);
        armed = kb + 1;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % kStages;
        const uint32_t parity = (kb / kStages) & 1;
        if (!mbar_wait(smem_u32(&bars[s]), parity, failed)) break;
        // (no tcgen05 fence here: the data arrived through the async proxy and its mbarrier; a fence after every
        // stage wait makes the issuing thread wait out the MMAs in flight: 150 instead of 48 cycles per 128x64x16 MMA)
        const uint64_t adesc = make_desc(smem_u32(stage_a + size_t(s) * kStageBytesA));
        const uint64_t bdesc = make_desc(smem_u32(stage_b + size_t(s) * kStageBytesB));
#pragma unroll
        for (int k = 0; k < BK / kUmmaK; ++k) {
          // advancing by 16 bf16 = 32 bytes inside the swizzle atom = +2 in the 16-byte address field
          umma_bf16(tmem_base, adesc + uint64_t(2 * k), bdesc + uint64_t(2 * k), (kb | k) != 0 ? 1u : 0u);
        }
        umma_commit(smem_u32(&bars[kStages + s]));   // frees the stage when these MMAs have read it
      }
      if (!*failed) umma_commit(smem_u32(&bars[2 * kStages]));  // accumulator complete
    }
  } else {
    // Epilogue warps 2..5: TMEM lane group = warp % 4.
    const int q = warp & 3;
    const bool ok = mbar_wait(smem_u32(&bars[2 * kStages]), 0, failed);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok) {
      const int m = m0 + q * 32 + lane;
      const bool vec_ok = (N % 8) == 0;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem_base + (uint32_t(q * 32) << 16) + uint32_t(c * 32), r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const int nbase = n0 + c * 32;
        if (m < M && nbase < N) {
          __nv_bfloat16* dst = out + size_t(m) * N + nbase;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int n = nbase + j * 8;
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              float x = __uint_as_float(r[j * 8 + i]);
              if (bias != nullptr && n + i < N) x += __bfloat162float(bias[n + i]);
              v[i] = act_fn(x, act);
            }
            if (vec_ok && n + 8 <= N) {
              uint4 pk;
              __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
              for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
              *reinterpret_cast<uint4*>(dst + j * 8) = pk;
            } else {
#pragma unroll
              for (int i = 0; i < 8; ++i)
                if (n + i < N) dst[j * 8 + i] = __float2bfloat16_rn(v[i]);
            }
          }
        }
      }
    }
  }
  // Tear-down. On the failure path the producer first waits (bounded) for the copies it issued.
  if (warp == 0 && lane == 0 && *failed) {
    const int first = armed > kStages ? armed - kStages : 0;
    for (int kb = first; kb < armed; ++kb) {
      const unsigned long long t0 = now_ns();
      while (!mbar_try(smem_u32(&bars[kb % kStages]), (kb / kStages) & 1) && now_ns() - t0 < kWaitLimitNs) {}
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
  if (threadIdx.x == 0 && failed_s && status != nullptr) atomicExch(status, 1u);
}


// ------------------------------------------------------------------------------------------ //
// Two-SM variant (tcgen05 cta_group::2): a cluster of two CTAs owns a 256 x 256 output tile.  Each CTA loads its
// own 128 rows of A and HALF of B (128 of the 256 columns) per ring stage; one thread of the leader CTA issues
// 256 x 256 x 16 MMAs that read A from each CTA's own shared memory and both halves of B, and leave 128 rows of
// the accumulator in each CTA's tensor memory.  Per SM and MMA that is 4 KB of A and 4 KB of B out of shared
// memory instead of 4 + 8: a 128 x 256 tile on one SM reads (and TMA writes) more than the 128 bytes per clock an
// SM's shared memory has, which is what held the one-SM kernel at 0.84 of the library on large products.
//   loads     : cp.async.bulk.tensor with .cta_group::2 (no multicast): data lands in the issuing CTA, the byte
//               count is signalled on the LEADER's full barrier, which expects both CTAs' bytes;
//   empty/acc : tcgen05.commit.cta_group::2 ... multicast::cluster arrives on the barrier at the same offset in
//               both CTAs (ring slots free, accumulator complete);
//   acc_empty : the eight epilogue warps of both CTAs arrive on the leader's barrier (count 16, remote arrive).
// Every wait is bounded.  It is the PAIR mode of the persistent kernel below, so every operand mode and epilogue has it.
// ------------------------------------------------------------------------------------------ //
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t leader_bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(leader_bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"((unsigned short)3)
      : "memory");
}

// ------------------------------------------------------------------------------------------ //
// Persistent variant: one CTA per SM walks over output tiles of 128 x BN_; the accumulator is
// double-buffered in tensor memory (2 x BN_ columns) so that the epilogue of tile i runs while
// the MMAs of tile i+1 are issued.  Ring-stage and accumulator hand-over use four kinds of
// mbarriers: full/empty per smem stage, acc_full/acc_empty per accumulator buffer.
// The epilogue leaves through shared memory: every epilogue warp converts [32 rows x 64 columns]
// of its accumulator quarter to bf16, writes them in the 128-byte-swizzle layout and hands the box
// to a TMA store (two boxes per warp in flight), so global memory sees full 128-byte rows and the
// tile edges are clipped by the tensor map.  Row pitches that TMA cannot address (N % 8 != 0)
// take the direct-store epilogue.
// ------------------------------------------------------------------------------------------ //
template <int BN_, int EPI = 0, int PAIR = 0>
struct PersistentCfg {
  // PAIR: two CTAs of a cluster share a (2 * BM) x BN_ tile (tcgen05 cta_group::2); each holds its 128 rows of A and
  // half of B, so a stage is smaller and the ring deeper.
  // the column-statistics epilogue gives one ring stage up for its per-warp partial sums
  // PAIR runs eight epilogue warps, two per 32-lane quarter of tensor memory, each on half of the tile's columns:
  // with a reduction of 1024 the main loop of a 256 x 256 tile takes 4.3 us, and four warps that convert, activate
  // and store 256 columns each (and wait for their own TMA stores and auxiliary loads in turn) took three times
  // that on the GELU epilogues.  Their staging boxes cost one of the six ring stages.
  static constexpr int kEpiWarps = PAIR ? 8 : 4;
  static constexpr int kThreadsP = 64 + 32 * kEpiWarps;
  static constexpr int kStagesP = (PAIR ? 5 : ((BN_ == 256) ? 4 : 6)) - (EPI == kEpiColumnStats ? 1 : 0);
  // per epilogue warp: BN_ column sums and BN_ sums of squares
  static constexpr uint32_t kStatBytes = EPI == kEpiColumnStats ? kEpiWarps * 2 * BN_ * 4 : 0;
  static constexpr int kRowsB = PAIR ? BN_ / 2 : BN_;          // rows (output columns) of B one CTA loads
  static constexpr int kTileM = PAIR ? 2 * BM : BM;
  static constexpr uint32_t kBytesA = BM * BK * 2;
  static constexpr uint32_t kBytesB = kRowsB * BK * 2;
  static constexpr uint32_t kBytesStage = kBytesA + kBytesB;
  static constexpr uint32_t kCols = 2 * BN_;
  // output staging: per epilogue warp two [32 rows x 64 columns] bf16 boxes (4 KiB each, 1024-byte aligned)
  static constexpr uint32_t kBytesOutBox = 32 * 64 * 2;
  static constexpr uint32_t kBytesOut = kEpiWarps * 2 * kBytesOutBox;
  static constexpr size_t kSmem = 1024 + size_t(kStagesP) * kBytesStage + kBytesOut + 256 + kStatBytes;
  static constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(BN_ >> 3) << 17) | (uint32_t(kTileM >> 4) << 24);
};

// BMODE 0: B is [N, K] row-major (K-major operand).  BMODE 1: B is [K, N] row-major and is consumed as an
// MN-major operand: every ring stage holds BN_/64 boxes of [64 K-rows x 64 N-columns] (8 KiB each, 128-byte
// swizzle); the descriptor's leading-dimension stride is the distance between boxes, its stride-dimension
// stride the 1024 bytes between groups of eight K-rows, and one MMA step advances 16 rows = 2048 bytes.
// AMODE 1: A is given as [K, M] row-major (the transposed product dY^T * X of a weight gradient) and is
// consumed MN-major in the same way: two boxes of [64 K-rows x 64 M-columns] per stage, bit 15 of the
// instruction descriptor.
// EPI (GemmEpi) is a template parameter so that the plain epilogue keeps its small register footprint.
// PAIR 1: launched as clusters of two CTAs (see the two-SM notes above): loads signal the
// leader's full barrier, commits are multicast to both CTAs, the leader's MMA thread issues cta_group::2 MMAs and
// waits for the epilogue warps of both CTAs.
template <int BN_, int BMODE = 0, int AMODE = 0, int EPI = 0, int PAIR = 0>
__global__ void __launch_bounds__((PersistentCfg<BN_, EPI, PAIR>::kThreadsP), 1)
gemm_bf16_nt_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                               const __grid_constant__ CUtensorMap map_c, __nv_bfloat16* __restrict__ out,
                               const __nv_bfloat16* __restrict__ bias, int M, int N, int K, int act, int tma_out,
                               unsigned int* __restrict__ status, const __grid_constant__ CUtensorMap map_aux,
                               const __nv_bfloat16* __restrict__ aux_in, float* __restrict__ col_stats) {
  using Cfg = PersistentCfg<BN_, EPI, PAIR>;
  constexpr int S = Cfg::kStagesP;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* stage_a = smem;
  unsigned char* stage_b = smem + size_t(S) * Cfg::kBytesA;
  unsigned char* stage_out = smem + size_t(S) * Cfg::kBytesStage;
  uint64_t* bars = reinterpret_cast<uint64_t*>(stage_out + Cfg::kBytesOut);
  // bars[0..S): full, [S..2S): empty, [2S..2S+2): acc_full, [2S+2..2S+4): acc_empty
  __shared__ uint32_t tmem_base_s;
  __shared__ int failed_s;
  volatile int* failed = &failed_s;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
  const bool leader = rank == 0;
  const int tiles_n = (N + BN_ - 1) / BN_;
  const int tiles_m = (M + Cfg::kTileM - 1) / Cfg::kTileM;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + BK - 1) / BK;
  const int first_tile = PAIR ? int(blockIdx.x >> 1) : int(blockIdx.x);
  const int tile_step = PAIR ? int(gridDim.x >> 1) : int(gridDim.x);

  if (threadIdx.x == 0) {
    failed_s = 0;
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(&bars[s]), 1);
      mbar_init(smem_u32(&bars[S + s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&bars[2 * S + a]), 1);        // one tcgen05.commit
      mbar_init(smem_u32(&bars[2 * S + 2 + a]), (PAIR ? 2 : 1) * Cfg::kEpiWarps);    // one arrive per epilogue warp (of both CTAs)
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    if (PAIR) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(Cfg::kCols) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(Cfg::kCols) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (PAIR) {
    // nobody signals a peer's barrier before the peer has initialised it
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_s;

  int armed = 0;
  if (warp == 0) {
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int tile = first_tile; tile < num_tiles && ok; tile += tile_step) {
        int tm, tn;
        tile_coords(tile, tiles_m, tiles_n, tm, tn);
        const int m0 = tm * Cfg::kTileM + int(rank) * BM;
        const int n0 = tn * BN_ + int(rank) * Cfg::kRowsB;          // PAIR: this CTA's half of the tile's columns
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % S;
          if (!mbar_wait(smem_u32(&bars[S + s]), ((it / S) & 1) ^ 1, failed)) { ok = false; break; }
          // PAIR: the leader's barrier counts the bytes of both CTAs; the leader arms it
          if (leader) mbar_expect_tx(smem_u32(&bars[s]), (PAIR ? 2u : 1u) * Cfg::kBytesStage);
          const uint32_t full = PAIR ? mapa_u32(smem_u32(&bars[s]), 0u) : smem_u32(&bars[s]);
          auto load = [&](uint32_t dst, const CUtensorMap* map, int x, int y) {
            if (PAIR) tma_load_2d_pair(dst, map, full, x, y);
            else tma_load_2d(dst, map, full, x, y);
          };
          if (AMODE == 0) {
            load(smem_u32(stage_a + size_t(s) * Cfg::kBytesA), &map_a, kb * BK, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              load(smem_u32(stage_a + size_t(s) * Cfg::kBytesA + size_t(j) * 8192), &map_a, m0 + j * 64, kb * BK);
          }
          if (BMODE == 0) {
            load(smem_u32(stage_b + size_t(s) * Cfg::kBytesB), &map_b, kb * BK, n0);
          } else {
#pragma unroll
            for (int j = 0; j < Cfg::kRowsB / 64; ++j)
              load(smem_u32(stage_b + size_t(s) * Cfg::kBytesB + size_t(j) * 8192), &map_b, n0 + j * 64, kb * BK);
          }
          armed = it + 1;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      int it = 0, local = 0;
      bool ok = true;
      for (int tile = first_tile; tile < num_tiles && ok; tile += tile_step, ++local) {
        const int acc = local & 1;
        // the epilogue (of both CTAs) must have drained this accumulator buffer (tile local-2)
        if (!(PAIR ? mbar_wait_cluster(smem_u32(&bars[2 * S + 2 + acc]), ((local >> 1) & 1) ^ 1, failed)
                   : mbar_wait(smem_u32(&bars[2 * S + 2 + acc]), ((local >> 1) & 1) ^ 1, failed))) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_d = tmem_base + uint32_t(acc * BN_);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % S;
          if (!mbar_wait(smem_u32(&bars[s]), (it / S) & 1, failed)) { ok = false; break; }
          // (no tcgen05 fence here: the data arrived through the async proxy and its mbarrier; a fence after every
          // stage wait makes the issuing thread wait out the MMAs in flight: 150 instead of 48 cycles per 128x64x16 MMA)
          const uint32_t a_addr = smem_u32(stage_a + size_t(s) * Cfg::kBytesA);
          const uint64_t adesc = AMODE == 0 ? make_desc(a_addr) : make_desc_mn(a_addr, 8192, 1024);
          const uint32_t b_addr = smem_u32(stage_b + size_t(s) * Cfg::kBytesB);
          const uint64_t bdesc = BMODE == 0 ? make_desc(b_addr) : make_desc_mn(b_addr, 8192, 1024);
          // MN-major operands: bits 15 (A) and 16 (B) of the instruction descriptor; 16 K-rows of 128 bytes per MMA step
          constexpr uint32_t idesc = Cfg::kIdesc | (AMODE != 0 ? (1u << 15) : 0u) | (BMODE != 0 ? (1u << 16) : 0u);
          constexpr uint64_t a_step = AMODE == 0 ? 2 : (16 * 128) >> 4;
          constexpr uint64_t b_step = BMODE == 0 ? 2 : (16 * 128) >> 4;
#pragma unroll
          for (int k = 0; k < BK / kUmmaK; ++k) {
            if (PAIR) {
              asm volatile(
                  "{\n\t.reg .pred p;\n\t"
                  "setp.ne.b32 p, %4, 0;\n\t"
                  "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
                  ::"r"(tmem_d), "l"(adesc + a_step * uint64_t(k)), "l"(bdesc + b_step * uint64_t(k)), "r"(idesc),
                    "r"((kb | k) != 0 ? 1u : 0u), "r"(0u)
                  : "memory");
            } else {
              asm volatile(
                  "{\n\t.reg .pred p;\n\t"
                  "setp.ne.b32 p, %4, 0;\n\t"
                  "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                  ::"r"(tmem_d), "l"(adesc + a_step * uint64_t(k)), "l"(bdesc + b_step * uint64_t(k)), "r"(idesc),
                    "r"((kb | k) != 0 ? 1u : 0u)
                  : "memory");
            }
          }
          if (PAIR) umma_commit_pair(smem_u32(&bars[S + s]));
          else umma_commit(smem_u32(&bars[S + s]));
        }
        if (ok) {
          if (PAIR) umma_commit_pair(smem_u32(&bars[2 * S + acc]));
          else umma_commit(smem_u32(&bars[2 * S + acc]));
        }
      }
    }
  } else {
    const int q = warp & 3;                // the quarter of tensor memory (32 lanes = 32 rows) this warp can read
    const int ew = warp - 2;               // epilogue warp index
    // eight warps: warps 2-5 take the first half of the columns, warps 6-9 the second
    constexpr int kChunks = BN_ / 64;
    constexpr int kChunksW = Cfg::kEpiWarps == 8 ? kChunks / 2 : kChunks;
    const int c_first = Cfg::kEpiWarps == 8 ? (ew >> 2) * kChunksW : 0;
    const bool vec_ok = (N % 8) == 0;
    unsigned char* my_out = stage_out + size_t(ew) * 2 * Cfg::kBytesOutBox;
    int local = 0;
    int boxes = 0;                       // TMA stores issued by this warp
    // kEpiColumnStats: this warp's partial column sums [BN_] and sums of squares [BN_] of the current column
    // block live in shared memory (lanes 0-7 each own eight columns of every 64-column chunk, so no atomics)
    // and go to col_stats with vector reductions when the column block changes and at the end: adding every
    // box to global memory directly serialises thousands of reductions per address.
    float* wstat = reinterpret_cast<float*>(stage_out + Cfg::kBytesOut + 256) + (EPI == kEpiColumnStats ? ew * 2 * BN_ : 0);
    int stat_n0 = -1;
    auto flush_stats = [&]() {
      if (stat_n0 >= 0 && lane < 8) {
#pragma unroll 1
        for (int c = c_first; c < c_first + kChunksW; ++c) {
          const int col = c * 64 + lane * 8;
          const int n = stat_n0 + col;
          float4* ws = reinterpret_cast<float4*>(wstat + col);
          float4* wq = reinterpret_cast<float4*>(wstat + BN_ + col);
          if (n < N) {                   // N is a multiple of 8 in this mode: the whole group is inside
            atomicAdd(reinterpret_cast<float4*>(col_stats + n), ws[0]);
            atomicAdd(reinterpret_cast<float4*>(col_stats + n) + 1, ws[1]);
            atomicAdd(reinterpret_cast<float4*>(col_stats + N + n), wq[0]);
            atomicAdd(reinterpret_cast<float4*>(col_stats + N + n) + 1, wq[1]);
          }
          ws[0] = ws[1] = wq[0] = wq[1] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
    };
    if constexpr (EPI == kEpiColumnStats) {
      for (int i = lane; i < 2 * BN_; i += 32) wstat[i] = 0.f;
      __syncwarp();
    }
    for (int tile = first_tile; tile < num_tiles; tile += tile_step, ++local) {
      const int acc = local & 1;
      int tm, tn;
      tile_coords(tile, tiles_m, tiles_n, tm, tn);
      const int m0 = tm * Cfg::kTileM + int(rank) * BM;         // this CTA's 128 rows, all BN_ columns
      const int n0 = tn * BN_;
      if (!mbar_wait(smem_u32(&bars[2 * S + acc]), (local >> 1) & 1, failed)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int m = m0 + q * 32 + lane;
      if constexpr (EPI == kEpiColumnStats) {
        if (n0 != stat_n0) {
          flush_stats();
          stat_n0 = n0;
        }
      }
      if (tma_out) {
#pragma unroll 1
        for (int c = c_first; c < c_first + kChunksW; ++c) {
          const int nbase = n0 + c * 64;
          if (nbase >= N || m0 + q * 32 >= M) break;           // warp-uniform
          uint32_t r[64];
          const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + uint32_t(acc * BN_ + c * 64);
          tmem_ld32(taddr, r);
          tmem_ld32(taddr + 32, r + 32);
          // the box written two stores ago must have been read out of shared memory
          if (lane == 0) tma_store_wait_read<1>();
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          __syncwarp();
          if constexpr (EPI == kEpiNone || EPI == kEpiColumnStats) {
            unsigned char* box = my_out + size_t(boxes & 1) * Cfg::kBytesOutBox;
            unsigned char* row = box + lane * 128;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float v[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                float x = __uint_as_float(r[j * 8 + i]);
                if (bias != nullptr) {
                  const int n = nbase + j * 8 + i;
                  x += n < N ? __bfloat162float(bias[n]) : 0.f;
                }
                v[i] = act_fn(x, act);
              }
              uint4 pk;
              __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
              for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
              *reinterpret_cast<uint4*>(row + ((j ^ (lane & 7)) << 4)) = pk;      // 128-byte swizzle
            }
            if constexpr (EPI == kEpiColumnStats) {
              // Statistics of the staged (rounded) box: lane l reads the eight columns (l & 7)*8.. of rows
              // (l >> 3) + 4i back with 16-byte loads that follow the swizzle, sums them as packed float pairs, the
              // four row groups are folded with shuffles and eight lanes add the result to this warp's partial sums.
              // Rows past M hold exact zeros (zero-filled A rows, no bias, no activation).  The chunk loop stays
              // rolled: as straight-line code the epilogue ran out of the instruction cache.
              __syncwarp();
              unsigned long long s2[4] = {0ull, 0ull, 0ull, 0ull}, q2[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int rr = (lane >> 3) + 4 * i;
                const uint4 wv = *reinterpret_cast<const uint4*>(box + rr * 128 + (((lane & 7) ^ (rr & 7)) << 4));
                const uint32_t w4[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                  const unsigned long long f = pack_f32x2(w4[k] << 16, w4[k] & 0xffff0000u);   // two bf16 -> two floats
                  asm("add.rn.f32x2 %0, %0, %1;" : "+l"(s2[k]) : "l"(f));
                  asm("fma.rn.f32x2 %0, %1, %1, %0;" : "+l"(q2[k]) : "l"(f));
                }
              }
              float v[16];
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                unpack_f32x2(s2[k], v[2 * k], v[2 * k + 1]);
                unpack_f32x2(q2[k], v[8 + 2 * k], v[8 + 2 * k + 1]);
              }
#pragma unroll
              for (int k = 0; k < 16; ++k) {
                v[k] += __shfl_xor_sync(0xffffffffu, v[k], 8);
                v[k] += __shfl_xor_sync(0xffffffffu, v[k], 16);
              }
              if (lane < 8) {
                float4* ws = reinterpret_cast<float4*>(wstat + c * 64 + lane * 8);
                float4* wq = reinterpret_cast<float4*>(wstat + BN_ + c * 64 + lane * 8);
                float4 t;
                t = ws[0]; t.x += v[0]; t.y += v[1]; t.z += v[2]; t.w += v[3]; ws[0] = t;
                t = ws[1]; t.x += v[4]; t.y += v[5]; t.z += v[6]; t.w += v[7]; ws[1] = t;
                t = wq[0]; t.x += v[8]; t.y += v[9]; t.z += v[10]; t.w += v[11]; wq[0] = t;
                t = wq[1]; t.x += v[12]; t.y += v[13]; t.z += v[14]; t.w += v[15]; wq[1] = t;
              }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&map_c, smem_u32(box), nbase, m0 + q * 32);
              tma_store_commit();
            }
            ++boxes;
          } else if constexpr (EPI == kEpiMulGeluGrad || EPI == kEpiAddAux) {
            // kEpiMulGeluGrad: out = accumulator * GELU'(aux), the backward of a fused Linear+GELU (aux = the saved
            // pre-activation).  kEpiAddAux: out = accumulator + aux (aux = a gradient that joins this one).
            unsigned char* box = my_out + size_t(boxes & 1) * Cfg::kBytesOutBox;
            unsigned char* row = box + lane * 128;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              uint4 av = make_uint4(0u, 0u, 0u, 0u);
              if (m < M && nbase + j * 8 < N) av = __ldg(reinterpret_cast<const uint4*>(aux_in + size_t(m) * N + nbase + j * 8));
              const __nv_bfloat162* ah = reinterpret_cast<const __nv_bfloat162*>(&av);
              float v[8];
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const float2 t2 = __bfloat1622float2(ah[i]);
                if constexpr (EPI == kEpiAddAux) {
                  float b0 = 0.f, b1 = 0.f;
                  if (bias != nullptr) {                       // out = accumulator + bias + aux (a layer with a residual)
                    const int n = nbase + j * 8 + 2 * i;
                    b0 = n < N ? __bfloat162float(bias[n]) : 0.f;
                    b1 = n + 1 < N ? __bfloat162float(bias[n + 1]) : 0.f;
                  }
                  v[2 * i] = __uint_as_float(r[j * 8 + 2 * i]) + b0 + t2.x;
                  v[2 * i + 1] = __uint_as_float(r[j * 8 + 2 * i + 1]) + b1 + t2.y;
                } else {
                  v[2 * i] = __uint_as_float(r[j * 8 + 2 * i]) * gelu_tanh_grad(t2.x);
                  v[2 * i + 1] = __uint_as_float(r[j * 8 + 2 * i + 1]) * gelu_tanh_grad(t2.y);
                }
              }
              uint4 pk;
              __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
              for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
              *reinterpret_cast<uint4*>(row + ((j ^ (lane & 7)) << 4)) = pk;      // 128-byte swizzle
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&map_c, smem_u32(box), nbase, m0 + q * 32);
              tma_store_commit();
            }
            ++boxes;
          } else {
            // kEpiStorePreact: two boxes leave per chunk, x = accumulator + bias through map_aux and act(x)
            // through map_c; both staging boxes are in use, so every earlier store must have been read
            if (lane == 0) tma_store_wait_read<0>();
            __syncwarp();
            unsigned char* row_raw = my_out + lane * 128;
            unsigned char* row_act = my_out + Cfg::kBytesOutBox + lane * 128;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float x[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                x[i] = __uint_as_float(r[j * 8 + i]);
                if (bias != nullptr) {
                  const int n = nbase + j * 8 + i;
                  x[i] += n < N ? __bfloat162float(bias[n]) : 0.f;
                }
              }
              uint4 pk_raw, pk_act;
              __nv_bfloat162* hr = reinterpret_cast<__nv_bfloat162*>(&pk_raw);
              __nv_bfloat162* ha = reinterpret_cast<__nv_bfloat162*>(&pk_act);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                hr[i] = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
                // the activation sees the rounded pre-activation, as a separate activation kernel would
                const float2 xr = __bfloat1622float2(hr[i]);
                ha[i] = __floats2bfloat162_rn(act_fn(xr.x, act), act_fn(xr.y, act));
              }
              const int off = (j ^ (lane & 7)) << 4;                                // 128-byte swizzle
              *reinterpret_cast<uint4*>(row_raw + off) = pk_raw;
              *reinterpret_cast<uint4*>(row_act + off) = pk_act;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&map_aux, smem_u32(my_out), nbase, m0 + q * 32);
              tma_store_2d(&map_c, smem_u32(my_out + Cfg::kBytesOutBox), nbase, m0 + q * 32);
              tma_store_commit();
            }
            boxes += 2;
          }
        }
      } else {
#pragma unroll 1
        for (int c = 2 * c_first; c < 2 * (c_first + kChunksW); ++c) {
          uint32_t r[32];
          tmem_ld32(tmem_base + (uint32_t(q * 32) << 16) + uint32_t(acc * BN_ + c * 32), r);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          const int nbase = n0 + c * 32;
          if (m < M && nbase < N) {
            __nv_bfloat16* dst = out + size_t(m) * N + nbase;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int n = nbase + j * 8;
              float v[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                float x = __uint_as_float(r[j * 8 + i]);
                if (bias != nullptr && n + i < N) x += __bfloat162float(bias[n + i]);
                v[i] = act_fn(x, act);
              }
              if (vec_ok && n + 8 <= N) {
                uint4 pk;
                __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
                for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                *reinterpret_cast<uint4*>(dst + j * 8) = pk;
              } else {
#pragma unroll
                for (int i = 0; i < 8; ++i)
                  if (n + i < N) dst[j * 8 + i] = __float2bfloat16_rn(v[i]);
              }
            }
          }
        }
      }
      // hand the accumulator buffer back to the MMA warp
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        if (PAIR) mbar_arrive_cluster(mapa_u32(smem_u32(&bars[2 * S + 2 + acc]), 0u));
        else asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&bars[2 * S + 2 + acc])) : "memory");
      }
    }
    if constexpr (EPI == kEpiColumnStats) flush_stats();
    // the stores of this warp must be complete before its shared memory goes away
    if (lane == 0) tma_store_wait_all();
  }
  if (warp == 0 && lane == 0 && *failed && leader) {
    const int first = armed > S ? armed - S : 0;
    for (int it = first; it < armed; ++it) {
      const unsigned long long t0 = now_ns();
      while (!mbar_try(smem_u32(&bars[it % S]), (it / S) & 1) && now_ns() - t0 < kWaitLimitNs) {}
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (PAIR) {
    // neither CTA leaves (or frees tensor memory) while the other may still read its shared memory or signal it
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Cfg::kCols) : "memory");
    else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Cfg::kCols) : "memory");
  }
  if (threadIdx.x == 0 && failed_s && status != nullptr) atomicExch(status, 1u);
}

bool MakeMap(CUtensorMap* map, const void* base, int rows, int cols /*K*/, int box_rows) {
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 2};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(BK), static_cast<cuuint32_t>(box_rows)};
  return EncodeTiled(map, 2, base, dims, strides, box);
}

// Launches one instantiation of the persistent kernel on min(tiles, SMs) CTAs; PAIR: on clusters of two CTAs, one
// cluster per (2 * BM) x BN_ tile at a time.
template <int BN_, int BMODE, int AMODE, int EPI, int PAIR = 0>
cudaError_t LaunchPersistent(const CUtensorMap& map_a, const CUtensorMap& map_b, const CUtensorMap& map_c,
                             const CUtensorMap& map_aux, __nv_bfloat16* out, const __nv_bfloat16* bias,
                             const __nv_bfloat16* aux_in, int M, int N, int K, int act, int tma_out, int sm_count,
                             unsigned int* status, cudaStream_t stream, float* col_stats = nullptr) {
  using Cfg = PersistentCfg<BN_, EPI, PAIR>;
  auto kernel = gemm_bf16_nt_persistent_kernel<BN_, BMODE, AMODE, EPI, PAIR>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(Cfg::kSmem));
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  const int tiles = ((M + Cfg::kTileM - 1) / Cfg::kTileM) * ((N + BN_ - 1) / BN_);
  if (!PAIR) {
    kernel<<<tiles < sm_count ? tiles : sm_count, Cfg::kThreadsP, Cfg::kSmem, stream>>>(map_a, map_b, map_c, out, bias, M, N, K, act,
                                                                               tma_out, status, map_aux, aux_in, col_stats);
    return cudaSuccess;
  }
  const int pairs = tiles < sm_count / 2 ? tiles : sm_count / 2;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs));
  cfg.blockDim = dim3(Cfg::kThreadsP);
  cfg.dynamicSmemBytes = Cfg::kSmem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, map_a, map_b, map_c, out, bias, M, N, K, act, tma_out, status, map_aux, aux_in, col_stats);
}

// Whether a plain product goes to the two-SM kernel: TMA-storable output, at least one full pair tile in each
// direction, enough tiles to occupy the pairs, and a reduction long enough for the main loop to matter (measured:
// +8 % at 8192^3, +11 % on 8192 x 50304 x 1024, +4-5 % on GPT-2's 8192 x {1024, 3072, 4096} x {1024, 4096}; with
// K <= 256 the product is bound by its epilogue and the larger tile is 20-30 % slower).
// BLUEFOG_B200_GEMM_PAIR=0 keeps everything on the one-SM kernel, =1 sends every eligible shape to the pair.
bool UsePair(int M, int N, int K, int sm_count) {
  static const int mode = [] {
    const char* v = std::getenv("BLUEFOG_B200_GEMM_PAIR");
    return v == nullptr ? -1 : std::atoi(v);
  }();
  if (mode == 0) return false;
  if ((N % 8) != 0 || N < 256 || M < 256) return false;
  if (mode > 0) return true;
  const long long tiles = (long long)((M + 255) / 256) * ((N + 255) / 256);
  return K >= 1024 && tiles >= sm_count / 4;
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

}  // namespace

bool GemmSupported() { return GetEncodeFn() != nullptr; }

cudaError_t LaunchGemmBf16NT(const void* a, const void* b, void* out, const void* bias, int M, int N, int K, int act,
                             unsigned int* status, cudaStream_t stream, void* preact_out, float* col_stats,
                             const void* addend) {
  (void)cudaGetLastError();   // the value returned below must be this launch's own, not an older error of the calling thread
  if (M <= 0 || N <= 0 || K <= 0) return cudaErrorInvalidValue;
  // TMA needs 16-byte aligned bases and row pitches: K must be a multiple of 8 bf16 elements.
  if ((K % 8) != 0 || (reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 15))
    return cudaErrorInvalidValue;
  static const int variant = [] {
    const char* v = std::getenv("BLUEFOG_B200_GEMM_VARIANT");   // "tile" = one tile per CTA, default persistent
    return (v != nullptr && std::string(v) == "tile") ? 0 : 1;
  }();
  const int sm_count = SmCount();
  __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out);
  const __nv_bfloat16* bp = static_cast<const __nv_bfloat16*>(bias);
  CUtensorMap map_a, map_b, map_c;
  const int tma_out = (N % 8) == 0 ? 1 : 0;        // TMA needs a 16-byte row pitch
  if (variant != 0) {
    // output boxes of [32 rows x 64 columns]; without a usable pitch the map is a valid dummy over A
    if (!(tma_out ? MakeMap(&map_c, out, M, N, 32) : MakeMap(&map_c, a, M, K, 32))) return cudaErrorInvalidValue;
  }
  CUtensorMap map_aux = map_c;
  const bool preact = preact_out != nullptr;
  if (preact) {
    if (variant == 0 || !tma_out || (reinterpret_cast<uintptr_t>(preact_out) & 15)) return cudaErrorInvalidValue;
    if (!MakeMap(&map_aux, preact_out, M, N, 32)) return cudaErrorInvalidValue;
  }
  cudaError_t e = cudaSuccess;
  if (addend != nullptr) {
    // out = a b^T + bias + addend (a layer whose output joins a residual stream): the addend is read in the epilogue
    if (variant == 0 || !tma_out || preact || col_stats != nullptr || act != 0 || (reinterpret_cast<uintptr_t>(addend) & 15))
      return cudaErrorInvalidValue;
    const __nv_bfloat16* add = static_cast<const __nv_bfloat16*>(addend);
    if (UsePair(M, N, K, sm_count)) {
      if (!MakeMap(&map_a, a, M, K, BM) || !MakeMap(&map_b, b, N, K, 128)) return cudaErrorInvalidValue;
      e = LaunchPersistent<256, 0, 0, kEpiAddAux, 1>(map_a, map_b, map_c, map_c, o, bp, add, M, N, K, 0, 1, sm_count, status, stream);
    } else if (N > 128) {
      if (!MakeMap(&map_a, a, M, K, BM) || !MakeMap(&map_b, b, N, K, 256)) return cudaErrorInvalidValue;
      e = LaunchPersistent<256, 0, 0, kEpiAddAux>(map_a, map_b, map_c, map_c, o, bp, add, M, N, K, 0, 1, sm_count, status, stream);
    } else {
      if (!MakeMap(&map_a, a, M, K, BM) || !MakeMap(&map_b, b, N, K, 128)) return cudaErrorInvalidValue;
      e = LaunchPersistent<128, 0, 0, kEpiAddAux>(map_a, map_b, map_c, map_c, o, bp, add, M, N, K, 0, 1, sm_count, status, stream);
    }
  } else if (col_stats != nullptr) {
    // column statistics of the plain product only: the kernel relies on rows past M being exact zeros
    if (variant == 0 || !tma_out || preact || bias != nullptr || act != 0) return cudaErrorInvalidValue;
    const int bn = N > 128 ? 256 : 128;
    if (!MakeMap(&map_a, a, M, K, BM) || !MakeMap(&map_b, b, N, K, bn)) return cudaErrorInvalidValue;
    e = N > 128 ? LaunchPersistent<256, 0, 0, kEpiColumnStats>(map_a, map_b, map_c, map_aux, o, nullptr, nullptr, M, N, K, 0, 1,
                                                               sm_count, status, stream, col_stats)
                : LaunchPersistent<128, 0, 0, kEpiColumnStats>(map_a, map_b, map_c, map_aux, o, nullptr, nullptr, M, N, K, 0, 1,
                                                               sm_count, status, stream, col_stats);
  } else if (variant == 0) {
    if (!MakeMap(&map_a, a, M, K, BM) || !MakeMap(&map_b, b, N, K, BN)) return cudaErrorInvalidValue;
    static bool attr_set = false;
    if (!attr_set) {
      e = cudaFuncSetAttribute(gemm_bf16_nt_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmemBytes));
      if (e != cudaSuccess) return e;
      attr_set = true;
    }
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    gemm_bf16_nt_kernel<<<grid, kThreads, kSmemBytes, stream>>>(map_a, map_b, o, bp, M, N, K, act, status);
  } else if (tma_out && UsePair(M, N, K, sm_count)) {
    if (!MakeMap(&map_a, a, M, K, BM) || !MakeMap(&map_b, b, N, K, 128)) return cudaErrorInvalidValue;
    e = preact ? LaunchPersistent<256, 0, 0, kEpiStorePreact, 1>(map_a, map_b, map_c, map_aux, o, bp, nullptr, M, N, K, act, 1,
                                                                 sm_count, status, stream)
               : LaunchPersistent<256, 0, 0, kEpiNone, 1>(map_a, map_b, map_c, map_aux, o, bp, nullptr, M, N, K, act, 1, sm_count,
                                                          status, stream);
  } else if (N > 128) {
    if (!MakeMap(&map_a, a, M, K, BM) || !MakeMap(&map_b, b, N, K, 256)) return cudaErrorInvalidValue;
    e = preact ? LaunchPersistent<256, 0, 0, kEpiStorePreact>(map_a, map_b, map_c, map_aux, o, bp, nullptr, M, N, K, act, tma_out,
                                                              sm_count, status, stream)
               : LaunchPersistent<256, 0, 0, kEpiNone>(map_a, map_b, map_c, map_aux, o, bp, nullptr, M, N, K, act, tma_out,
                                                       sm_count, status, stream);
  } else {
    if (!MakeMap(&map_a, a, M, K, BM) || !MakeMap(&map_b, b, N, K, 128)) return cudaErrorInvalidValue;
    e = preact ? LaunchPersistent<128, 0, 0, kEpiStorePreact>(map_a, map_b, map_c, map_aux, o, bp, nullptr, M, N, K, act, tma_out,
                                                              sm_count, status, stream)
               : LaunchPersistent<128, 0, 0, kEpiNone>(map_a, map_b, map_c, map_aux, o, bp, nullptr, M, N, K, act, tma_out,
                                                       sm_count, status, stream);
  }
  if (e != cudaSuccess) return e;
  CountKernelLaunch();
  return cudaGetLastError();
}

// out[M,N] = a[M,K] * b[K,N]: the B operand is consumed MN-major straight from its row-major memory, so a
// product with a transposed weight (an input gradient) needs no transposed copy.  With gelu_preact the result
// is multiplied elementwise by GELU'(gelu_preact[M,N]) in the epilogue (the backward of a fused Linear+GELU).
cudaError_t LaunchGemmBf16NN(const void* a, const void* b, void* out, int M, int N, int K, unsigned int* status,
                             cudaStream_t stream, const void* gelu_preact, const void* addend) {
  (void)cudaGetLastError();   // the value returned below must be this launch's own, not an older error of the calling thread
  if (M <= 0 || N <= 0 || K <= 0 || (K % 8) != 0 || (N % 8) != 0) return cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15) || (reinterpret_cast<uintptr_t>(out) & 15) ||
      (reinterpret_cast<uintptr_t>(gelu_preact) & 15) || (reinterpret_cast<uintptr_t>(addend) & 15) ||
      (gelu_preact != nullptr && addend != nullptr))
    return cudaErrorInvalidValue;
  const int sm_count = SmCount();
  CUtensorMap map_a, map_b, map_c;
  // B: [K rows, N columns]; boxes of 64 columns (128 bytes) x 64 rows
  if (!MakeMap(&map_a, a, M, K, BM) || !MakeMap(&map_b, b, K, N, 64) || !MakeMap(&map_c, out, M, N, 32))
    return cudaErrorInvalidValue;
  __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out);
  const __nv_bfloat16* aux = static_cast<const __nv_bfloat16*>(gelu_preact);
  cudaError_t e;
  if (UsePair(M, N, K, sm_count)) {
    const __nv_bfloat16* add = static_cast<const __nv_bfloat16*>(addend);
    if (add != nullptr)
      e = LaunchPersistent<256, 1, 0, kEpiAddAux, 1>(map_a, map_b, map_c, map_c, o, nullptr, add, M, N, K, 0, 1, sm_count, status, stream);
    else if (aux != nullptr)
      e = LaunchPersistent<256, 1, 0, kEpiMulGeluGrad, 1>(map_a, map_b, map_c, map_c, o, nullptr, aux, M, N, K, 0, 1, sm_count, status,
                                                          stream);
    else
      e = LaunchPersistent<256, 1, 0, kEpiNone, 1>(map_a, map_b, map_c, map_c, o, nullptr, nullptr, M, N, K, 0, 1, sm_count, status,
                                                   stream);
  } else if (addend != nullptr) {
    const __nv_bfloat16* add = static_cast<const __nv_bfloat16*>(addend);
    e = N > 128 ? LaunchPersistent<256, 1, 0, kEpiAddAux>(map_a, map_b, map_c, map_c, o, nullptr, add, M, N, K, 0, 1, sm_count,
                                                          status, stream)
                : LaunchPersistent<128, 1, 0, kEpiAddAux>(map_a, map_b, map_c, map_c, o, nullptr, add, M, N, K, 0, 1, sm_count,
                                                          status, stream);
  } else if (N > 128) {
    e = aux != nullptr ? LaunchPersistent<256, 1, 0, kEpiMulGeluGrad>(map_a, map_b, map_c, map_c, o, nullptr, aux, M, N, K, 0, 1,
                                                                      sm_count, status, stream)
                       : LaunchPersistent<256, 1, 0, kEpiNone>(map_a, map_b, map_c, map_c, o, nullptr, nullptr, M, N, K, 0, 1,
                                                               sm_count, status, stream);
  } else {
    e = aux != nullptr ? LaunchPersistent<128, 1, 0, kEpiMulGeluGrad>(map_a, map_b, map_c, map_c, o, nullptr, aux, M, N, K, 0, 1,
                                                                      sm_count, status, stream)
                       : LaunchPersistent<128, 1, 0, kEpiNone>(map_a, map_b, map_c, map_c, o, nullptr, nullptr, M, N, K, 0, 1,
                                                               sm_count, status, stream);
  }
  if (e != cudaSuccess) return e;
  CountKernelLaunch();
  return cudaGetLastError();
}

// out[M,N] = a[K,M]^T * b[K,N]: both operands row-major with the reduction dimension outermost (the weight
// gradient dW = dY^T X of a linear layer: a = dY [rows, N_out], b = X [rows, K_in]); both are consumed MN-major.
cudaError_t LaunchGemmBf16TN(const void* a, const void* b, void* out, int M, int N, int K, unsigned int* status,
                             cudaStream_t stream) {
  (void)cudaGetLastError();   // the value returned below must be this launch's own, not an older error of the calling thread
  if (M <= 0 || N <= 0 || K <= 0 || (M % 8) != 0 || (N % 8) != 0) return cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15) || (reinterpret_cast<uintptr_t>(out) & 15))
    return cudaErrorInvalidValue;
  const int sm_count = SmCount();
  CUtensorMap map_a, map_b, map_c;
  // A: [K rows, M columns], B: [K rows, N columns]; boxes of 64 columns (128 bytes) x 64 rows
  if (!MakeMap(&map_a, a, K, M, 64) || !MakeMap(&map_b, b, K, N, 64) || !MakeMap(&map_c, out, M, N, 32))
    return cudaErrorInvalidValue;
  __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out);
  const cudaError_t e =
      UsePair(M, N, K, sm_count)
          ? LaunchPersistent<256, 1, 1, kEpiNone, 1>(map_a, map_b, map_c, map_c, o, nullptr, nullptr, M, N, K, 0, 1, sm_count, status,
                                                     stream)
      : N > 128 ? LaunchPersistent<256, 1, 1, kEpiNone>(map_a, map_b, map_c, map_c, o, nullptr, nullptr, M, N, K, 0, 1, sm_count,
                                                      status, stream)
              : LaunchPersistent<128, 1, 1, kEpiNone>(map_a, map_b, map_c, map_c, o, nullptr, nullptr, M, N, K, 0, 1, sm_count,
                                                      status, stream);
  if (e != cudaSuccess) return e;
  CountKernelLaunch();
  return cudaGetLastError();
}

}  // namespace bfb
