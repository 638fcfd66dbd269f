// Device-side communication protocol and launchers for the peer-memory kernels.
//
// Every rank owns a "channel": a control block plus a double-buffered payload area
// ("arena") that live in memory mapped into every peer's address space (CUDA IPC over
// NVLink/NVSwitch).  A rank *publishes* version v of its payload in arena half v % 2 and
// then stores epoch = v + 1 with release semantics; a reader spins (bounded) on the
// owner's epoch with acquire loads, streams the payload with 16-byte loads straight out
// of the owner's memory, and finally adds 1 to the owner's done[v % 2] counter.  Before a
// rank overwrites arena half v % 2 with version v it waits until done[v % 2] has reached
// the number of readers of all earlier versions with that parity.  Every dependency
// points at an earlier version, so the protocol cannot deadlock, and every wait has a time
// limit after which the kernel records an error code in a host-visible status word and
// returns normally.
//
// What this replaces in the reference: the grouped ncclSend/ncclRecv exchange, the
// cudaMemcpyAsync fusion-buffer pack/unpack, the per-destination scaled copies and the
// per-neighbor ATen mul_/add_ combine (bluefog/common/nccl_controller.cc:710-949,
// 1013-1204, 1915-2064; bluefog/torch/mpi_ops.cc:99-164).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace bfb {

constexpr int kMaxWorld = 64;   // ranks addressable by one channel
constexpr int kMaxSrc = 64;     // sources one pull kernel can read
constexpr int kMaxSeg = 40;     // tensors handled by one launch (fused groups are chunked)

// Error codes written to the status word (0 = healthy).
enum CommError : uint32_t {
  kCommOk = 0,
  kCommTimeoutEpoch = 1,   // a source never published the awaited version
  kCommTimeoutDone = 2,    // readers of an old version never finished
  kCommBadArgument = 3,
  kCommPeerFailed = 4,     // a source published a version it could not complete (its own wait had expired)
  kCommTimeoutLock = 5,    // a window mutex word stayed taken for longer than the limit
  kCommLayoutMismatch = 6, // a source published from registered memory that this reader has no matching pointer for
};

struct alignas(256) ChannelCtrl {
  unsigned long long epoch;             // versions published so far
  unsigned long long done[2];           // finished readers per arena half (cumulative)
  unsigned int block_counter[4];        // last-block detection, local use only
  unsigned int reserved[2];
  unsigned long long payload_bytes[2];  // size of the published payload per half
  double dst_weight[2][kMaxWorld];      // weight the owner attaches per destination rank
  // Versions (epoch values) up to which dst_weight[] of the half being *read* is valid: the adapt-with-combine
  // bucket step announces the destination weights of a step when that step starts, after the data they scale.
  unsigned long long weight_epoch;
  // Epoch value of a version whose owner gave up while producing it (a wait ran out): published all the same, so
  // that nobody hangs, but marked; readers report kCommPeerFailed and leave their outputs alone.
  unsigned long long failed_epoch;
  unsigned int launch_failed;           // set by any block of the owner's launches of the current version
  // Where the payload of each half's version lives: 0 = in the arena half; otherwise the key of a registered
  // tensor (symmetric buffer id and byte offset, see RegisteredLoc) that the owner published in place, without a
  // copy into the arena.  Written with the header of every version.
  unsigned long long payload_loc[2];
};

// Host-visible status block (pinned, mapped): kernels write, the host reads after the
// completion event.
struct CommStatus {
  unsigned int error;       // CommError
  unsigned int peer;        // rank that was waited for
  unsigned long long want;  // awaited value
  unsigned long long seen;  // last observed value
};

enum ElemType : int {
  kF32 = 0, kF64 = 1, kF16 = 2, kBF16 = 3, kI32 = 4, kI64 = 5, kU8 = 6, kI8 = 7, kI16 = 8,
};
int ElemSize(int elem_type);

struct PackParams {
  ChannelCtrl* ctrl;            // my control block
  unsigned char* arena_half;    // my arena + half offset
  CommStatus* status;
  unsigned long long need_done; // wait until ctrl->done[half] >= need_done before writing
  unsigned long long publish_epoch;  // value stored to ctrl->epoch when publish != 0
  unsigned long long timeout_ns;
  unsigned long long payload_bytes;
  unsigned long long loc;       // ChannelCtrl::payload_loc of this version
  int half;
  int wait_done;                // 1: perform the done-wait (first launch of a version)
  int publish;                  // 1: store the header and the epoch (last launch of a version)
  int world;
  int my_rank;
  int n_seg;
  int has_dst_weight;
  const void* src[kMaxSeg];
  unsigned long long dst_off[kMaxSeg];
  unsigned long long nbytes[kMaxSeg];
  unsigned long long chunk_start[kMaxSeg + 1];  // prefix sum of 16-byte chunks
  double dst_weight[kMaxWorld];
};

struct PullSync {
  int n_src;
  int my_rank;
  int half;
  int use_dst_weight;           // 1: scale by the sources' dst_weight[half][my_rank]; 2: wait for their weight_epoch first
  int signal_done;              // 1: add 1 to every source's done[half] when the grid is finished
  int counter_slot;             // which block_counter of my ctrl to use
  unsigned long long wait_epoch;
  unsigned long long timeout_ns;
  ChannelCtrl* my_ctrl;
  CommStatus* status;
  ChannelCtrl* src_ctrl[kMaxSrc];           // peer-mapped control blocks
  const unsigned char* src_arena[kMaxSrc];  // peer-mapped arena + half offset
  int src_rank[kMaxSrc];
};

// out[seg] = post_scale * (self_w * self[seg] + sum_j w_j * dstw_j * src_j[seg])
struct CombineParams {
  PullSync sync;
  const unsigned char* self_arena;   // my arena + half offset (self term), may be null if self_w == 0
  double self_w;
  double post_scale;
  double src_w[kMaxSrc];
  int elem_type;
  int n_seg;
  void* out[kMaxSeg];
  unsigned long long off[kMaxSeg];      // byte offset of the segment inside every arena half
  unsigned long long numel[kMaxSeg];
  unsigned long long chunk_start[kMaxSeg + 1];
  // Registered payloads (one tensor, published in place): my_loc is the key this rank published with (0 = arena)
  // and alt_src[j] the address of the same tensor in source j's registered buffer.  A source whose version says
  // "arena" is read from its arena, one that says my_loc from alt_src[j]; anything else is kCommLayoutMismatch.
  unsigned long long my_loc;
  const unsigned char* alt_src[kMaxSrc];
  // Bytes of a source's payload this launch reads (largest segment end).  A source whose version is shorter than that
  // was published with another layout (ranks that disagree about sizes while negotiation is skipped): the reader
  // reports kCommLayoutMismatch instead of reading past what was written.
  unsigned long long need_bytes;
};
static_assert(sizeof(CombineParams) <= 4000, "kernel parameters are limited to 4 KB");

// Plain copies out of sources' arenas (allgather / neighbor_allgather / broadcast).
struct GatherParams {
  PullSync sync;
  const unsigned char* self_arena;
  int n_copy;
  int copy_src[kMaxSeg];                 // index into sync.src_*, or -1 for my own arena
  void* out[kMaxSeg];
  unsigned long long src_off[kMaxSeg];
  unsigned long long nbytes[kMaxSeg];
  unsigned long long chunk_start[kMaxSeg + 1];
};

// kOptRMSprop: beta2 = alpha, amsgrad = centered; state1 square_avg, state2 momentum_buffer, state3 grad_avg.
// kOptAdagrad: lr = the step's decayed rate; state1 sum.  kOptAdadelta: beta2 = rho; state1 square_avg, state2 acc_delta.
enum BucketOpt : int { kOptNone = 0, kOptSGD = 1, kOptAdam = 2, kOptRMSprop = 3, kOptAdagrad = 4, kOptAdadelta = 5 };
enum BucketMode : int {
  // c = self_w*P + sum_j w_j*pub_j(v);  P' = c - step(g, c);  pub(v+1) = P'   (adapt-with-combine)
  kModeAWC = 0,
  // a = P - step(g, P);  P = a;  pub(v) = a   (first half of adapt-then-combine; no remote reads)
  kModeAdaptPublish = 1,
  // P' = self_w*P + sum_j w_j*pub_j(v)   (second half of adapt-then-combine; P holds the adapted value)
  kModeCombineOnly = 2,
  // gbar = post_scale*(g_self + sum_j pub_j(v));  P' = P - step(gbar, P)   (gradient allreduce)
  kModeGradReduce = 3,
  // pub(v) = src (P or g): plain publish of a local buffer
  kModePublishOnly = 4,
  // only announces this step's destination weights for the version the neighbors are about to pull (what an
  // adapt-with-combine launch does at its start; as a launch of its own for ranks emulated on one GPU, whose
  // kernels run one after the other and cannot wait for each other's start)
  kModeAnnounceWeights = 5,
};

struct BucketParams {
  PullSync sync;                 // unused fields are zero when the mode reads no peers
  int mode;
  int opt;
  int pub_elem;                  // kF32 or kBF16: element type of the published copy
  int grad_elem;                 // kF32 or kBF16
  int nesterov, adamw, amsgrad, first_step, maximize;
  float lr, momentum, dampening, weight_decay, beta1, beta2, eps, bias1, bias2, grad_scale;
  float self_w, post_scale;
  float src_w[kMaxSrc];
  unsigned long long numel;
  float* master;                 // P (private fp32)
  const void* grad;              // flat gradient bucket, or null when grad_ptrs is used
  // Gradients left where autograd put them: grad_ptrs[s] is the gradient of the s-th parameter of
  // the bucket (null = no gradient), which occupies elements [seg_start[s], seg_start[s] + seg_numel[s]).
  const void* const* grad_ptrs;
  const unsigned long long* seg_start;
  const unsigned long long* seg_numel;
  int n_seg;
  float* state1;                 // momentum / exp_avg
  float* state2;                 // exp_avg_sq
  float* state3;                 // max_exp_avg_sq (amsgrad)
  void* shadow;                  // bf16 copy used by forward/backward (optional)
  const unsigned char* pub_read_self;  // my published half of the version that is pulled (kept for reference; the own term is read from master)
  unsigned char* pub_write;      // my published half that is written (or null)
  // publishing the written half
  int publish;
  int wait_done;
  int write_half;
  unsigned long long need_done;
  unsigned long long publish_epoch;
  // Destination weights of this step (world entries, 1 where unused).  dst_weight_mode 1: they belong to the
  // version this launch publishes and are stored beside it.  2: they belong to the version this launch *reads*
  // (adapt-with-combine: the neighbors pull what the previous step published) and are announced at kernel start
  // through weight_epoch.
  int dst_weight_mode;
  int world;
  float dst_weight[kMaxWorld];
};

// Launchers. Each returns cudaGetLastError() of the launch.
cudaError_t LaunchPack(const PackParams& p, cudaStream_t stream);
cudaError_t LaunchCombine(const CombineParams& p, cudaStream_t stream);
cudaError_t LaunchGather(const GatherParams& p, cudaStream_t stream);
// One thread waits (bounded) until ctrl->done[half] >= need: every reader of the versions published so far in that
// half has finished.  A rank that published a tensor in place runs it behind its own pull, so that the operation is
// complete - and the tensor the caller's again - only when no neighbor still reads it.
cudaError_t LaunchWaitReaders(ChannelCtrl* ctrl, int half, unsigned long long need, unsigned long long timeout_ns,
                              CommStatus* status, int my_rank, cudaStream_t stream);
cudaError_t LaunchBucketStep(const BucketParams& p, cudaStream_t stream);
// buf[i] *= s for any supported element type (K1/K2 of the reference, kept as a utility).
cudaError_t LaunchScale(void* buf, unsigned long long numel, double s, int elem_type, cudaStream_t stream);
// Number of kernels launched by this library in this process (all launchers count).
unsigned long long KernelLaunchCount();
void CountKernelLaunch();

}  // namespace bfb
