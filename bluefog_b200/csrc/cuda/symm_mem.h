// Symmetric device memory: every rank allocates a buffer of the same size and maps all
// peers' buffers into its own address space, so kernels can load/store/reduce directly
// into any rank's HBM over NVLink.  Two providers:
//   * AllocateIpc   - one process per GPU; cudaMalloc + cudaIpcGetMemHandle, handles
//                     exchanged over the TCP control plane, cudaIpcOpenMemHandle on peers.
//   * AllocateLocal - all "ranks" are buffers of one process on one GPU; used to run the
//                     multi-rank kernels rank by rank on a single device.
// This layer has no counterpart in the reference, whose GPU path hands buffers to NCCL
// (bluefog/common/nccl_controller.cc:73-116).
#pragma once
#include <cuda_runtime.h>

#include <memory>
#include <string>
#include <vector>

#include "../common/control_plane.h"
#include "../common/status.h"

namespace bfb {

struct SymmBuffer {
  int rank = 0;
  int world = 1;
  int device = 0;
  size_t bytes = 0;
  std::vector<void*> ptrs;  // ptrs[r]: rank r's buffer in this process' address space
  bool ipc = false;         // true: peers are IPC mappings that must be closed
  bool owner = true;        // local mode: only the first view frees the memory
  std::shared_ptr<std::vector<void*>> local_owned;  // local mode: shared ownership of all buffers
  void* local() const { return ptrs[rank]; }
  ~SymmBuffer();
};

Status AllocateIpc(ControlPlane* cp, int channel, int device, size_t bytes, std::shared_ptr<SymmBuffer>* out);
Status AllocateLocal(int world, int device, size_t bytes, std::vector<std::shared_ptr<SymmBuffer>>* out);
// Symmetric memory shared by this rank and one peer only (world = 2; index 0 is the lower of the two ranks).
// Only the two ranks take part in the exchange of handles, so it can be set up while the others do other work.
Status AllocateIpcPair(ControlPlane* cp, int channel, int peer, int device, size_t bytes,
                       std::shared_ptr<SymmBuffer>* out);

std::string CudaErrorString(cudaError_t e);
#define BFB_CUDA_OK(expr)                                                              \
  do {                                                                                 \
    cudaError_t _e = (expr);                                                           \
    if (_e != cudaSuccess)                                                             \
      return ::bfb::Status::UnknownError(std::string(#expr) + " failed: " + ::bfb::CudaErrorString(_e)); \
  } while (0)

}  // namespace bfb
