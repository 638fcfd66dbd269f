// One-sided window kernels: a window is a block of peer-mapped device memory per rank,
// laid out as [WinHeader | self tensor | slot 0 | slot 1 | ...]; slot k receives what the
// k-th in-neighbor puts or accumulates.  The kernels write (or atomically add) straight
// into the destination's slots over NVLink and bump its per-source version counter with
// a release reduction, so the target's host and device do nothing ("passive target").
// They replace the request/ack handshake + 2-rank ncclSend/ncclRecv/ncclReduce emulation
// of the reference (bluefog/common/nccl_controller.cc:1261-1386, 1503-1887) and the ATen
// combine/reset of win_update (bluefog/torch/mpi_win_ops.cc:185-341).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "comm_kernels.h"

namespace bfb {

struct alignas(256) WinHeader {
  unsigned long long version[kMaxWorld];  // version[s]: transfers from source s since the last update
  double p[kMaxWorld];                    // push-sum weights: p[own rank] = own value, p[s] = received from s
  // Device-side mutex words of GPU windows: lock[s] guards the slot that source s writes on this rank (and
  // lock[own rank] the self tensor).  0 = free, otherwise 1 + the holder's rank.  Taken with a compare-and-swap
  // from a kernel of the holder (win_lock_kernel), which waits at most a given time.
  unsigned int lock[kMaxWorld];
};

// Outcome of the last lock launch of a rank on a window; lives next to the window's block counter.
struct WinLockState {
  unsigned int failed;        // 1: the wait for some word ran out; nothing is held, guarded kernels do nothing
  unsigned int failed_rank;   // owner of the word that could not be taken
  unsigned int held;          // words currently held by this rank's lock launch
  unsigned int pad;
};

constexpr int kMaxWinPeers = 64;

struct WinPutParams {
  const void* src;                  // local tensor that is sent
  void* self_scale_target;          // tensor scaled by self_weight afterwards (usually == src), or null
  unsigned long long numel;
  int elem_type;
  int accumulate;                   // 0: overwrite the slot, 1: atomically add
  int n_dst;
  int my_rank;
  int with_p;
  double self_weight;
  double weight[kMaxWinPeers];
  void* dst_slot[kMaxWinPeers];         // peer-mapped slot for this rank at every destination
  WinHeader* dst_header[kMaxWinPeers];  // peer-mapped headers
  WinHeader* my_header;
  unsigned int* block_counter;
  const WinLockState* lock_state;   // optional: when its `failed` is set the kernel does nothing
};

struct WinGetParams {
  unsigned long long numel;
  int elem_type;
  int n_src;
  double weight[kMaxWinPeers];
  const void* src_self[kMaxWinPeers];  // peer-mapped self tensors
  void* local_slot[kMaxWinPeers];
  int src_rank[kMaxWinPeers];
  WinHeader* my_header;
  unsigned int* block_counter;
  const WinLockState* lock_state;
};

struct WinUpdateParams {
  void* self;                       // window's self tensor (updated in place)
  void* out;                        // where the result is written (self or a clone)
  unsigned long long numel;
  int elem_type;
  int n_src;
  int reset;
  int with_p;
  int my_rank;
  double self_weight;
  double weight[kMaxWinPeers];
  void* slot[kMaxWinPeers];
  int src_rank[kMaxWinPeers];
  WinHeader* my_header;
  unsigned int* block_counter;
  const WinLockState* lock_state;
};

// Takes (acquire != 0) or frees the words lock[index[i]] of the headers header[i], in the given order (callers
// sort by owner rank, so two ranks locking overlapping sets cannot wait for each other in a cycle).
struct WinLockParams {
  int acquire;
  int n;
  int my_rank;
  unsigned long long timeout_ns;
  WinHeader* header[kMaxWinPeers];
  int index[kMaxWinPeers];
  int owner[kMaxWinPeers];           // rank that owns header[i], for the error report
  WinLockState* state;
  CommStatus* status;                // optional pinned status block: error kCommTimeoutLock, peer = owner
};

cudaError_t LaunchWinPut(const WinPutParams& p, cudaStream_t stream);
cudaError_t LaunchWinGet(const WinGetParams& p, cudaStream_t stream);
cudaError_t LaunchWinUpdate(const WinUpdateParams& p, cudaStream_t stream);
cudaError_t LaunchWinLock(const WinLockParams& p, cudaStream_t stream);

}  // namespace bfb
