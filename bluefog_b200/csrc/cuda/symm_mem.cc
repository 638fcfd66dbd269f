#include "symm_mem.h"

#include <cstring>

#include "../common/logging.h"

namespace bfb {

std::string CudaErrorString(cudaError_t e) { return std::string(cudaGetErrorName(e)) + ": " + cudaGetErrorString(e); }

SymmBuffer::~SymmBuffer() {
  if (ptrs.empty()) return;
  int prev = 0;
  cudaGetDevice(&prev);
  cudaSetDevice(device);
  if (ipc) {
    for (int r = 0; r < world; ++r) {
      if (r == rank || ptrs[r] == nullptr) continue;
      cudaIpcCloseMemHandle(ptrs[r]);
    }
    if (ptrs[rank]) cudaFree(ptrs[rank]);
  } else if (local_owned && local_owned.use_count() == 1) {
    for (void* p : *local_owned)
      if (p) cudaFree(p);
  }
  cudaSetDevice(prev);
}

Status AllocateIpc(ControlPlane* cp, int channel, int device, size_t bytes, std::shared_ptr<SymmBuffer>* out) {
  auto buf = std::make_shared<SymmBuffer>();
  buf->rank = cp->rank();
  buf->world = cp->size();
  buf->device = device;
  buf->bytes = bytes;
  buf->ipc = true;
  buf->ptrs.assign(buf->world, nullptr);
  BFB_CUDA_OK(cudaSetDevice(device));
  void* mine = nullptr;
  BFB_CUDA_OK(cudaMalloc(&mine, bytes));
  BFB_CUDA_OK(cudaMemset(mine, 0, bytes));
  BFB_CUDA_OK(cudaDeviceSynchronize());
  buf->ptrs[buf->rank] = mine;
  if (buf->world > 1) {
    cudaIpcMemHandle_t handle;
    BFB_CUDA_OK(cudaIpcGetMemHandle(&handle, mine));
    std::string blob(reinterpret_cast<const char*>(&handle), sizeof(handle));
    uint64_t sz = bytes;
    blob.append(reinterpret_cast<const char*>(&sz), sizeof(sz));
    std::vector<std::string> all;
    Status s = cp->AllgatherBytes(channel, blob, &all);
    if (!s.ok()) return s;
    for (int r = 0; r < buf->world; ++r) {
      if (r == buf->rank) continue;
      if (all[r].size() != blob.size()) return Status::UnknownError("symmetric memory: malformed handle from rank " + std::to_string(r));
      uint64_t peer_sz;
      std::memcpy(&peer_sz, all[r].data() + sizeof(handle), sizeof(peer_sz));
      if (peer_sz != sz)
        return Status::PreconditionError("symmetric memory: rank " + std::to_string(r) + " allocated " +
                                         std::to_string(peer_sz) + " bytes, this rank " + std::to_string(sz));
      cudaIpcMemHandle_t h;
      std::memcpy(&h, all[r].data(), sizeof(h));
      void* p = nullptr;
      BFB_CUDA_OK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
      buf->ptrs[r] = p;
    }
    // Nobody may touch a peer buffer before every rank has finished zeroing its own.
    s = cp->Barrier(channel);
    if (!s.ok()) return s;
  }
  *out = buf;
  return Status::OK();
}

Status AllocateIpcPair(ControlPlane* cp, int channel, int peer, int device, size_t bytes,
                       std::shared_ptr<SymmBuffer>* out) {
  if (peer < 0 || peer >= cp->size() || peer == cp->rank()) return Status::InvalidArgument("invalid peer for pair memory");
  auto buf = std::make_shared<SymmBuffer>();
  buf->rank = cp->rank() > peer ? 1 : 0;
  buf->world = 2;
  buf->device = device;
  buf->bytes = bytes;
  buf->ipc = true;
  buf->ptrs.assign(2, nullptr);
  BFB_CUDA_OK(cudaSetDevice(device));
  void* mine = nullptr;
  BFB_CUDA_OK(cudaMalloc(&mine, bytes));
  BFB_CUDA_OK(cudaMemset(mine, 0, bytes));
  BFB_CUDA_OK(cudaDeviceSynchronize());     // zeroed before the peer can learn the handle
  buf->ptrs[buf->rank] = mine;
  struct Blob {
    cudaIpcMemHandle_t handle;
    uint64_t bytes;
  } out_blob, in_blob;
  std::memset(&out_blob, 0, sizeof(out_blob));
  std::memset(&in_blob, 0, sizeof(in_blob));
  BFB_CUDA_OK(cudaIpcGetMemHandle(&out_blob.handle, mine));
  out_blob.bytes = bytes;
  Status s = cp->Exchange(channel, {{peer, &out_blob, sizeof(out_blob)}}, {{peer, &in_blob, sizeof(in_blob)}});
  if (!s.ok()) return s;
  if (in_blob.bytes != bytes)
    return Status::PreconditionError("pair memory: rank " + std::to_string(peer) + " allocated " +
                                     std::to_string(in_blob.bytes) + " bytes, this rank " + std::to_string(bytes));
  void* theirs = nullptr;
  BFB_CUDA_OK(cudaIpcOpenMemHandle(&theirs, in_blob.handle, cudaIpcMemLazyEnablePeerAccess));
  buf->ptrs[1 - buf->rank] = theirs;
  *out = buf;
  return Status::OK();
}

Status AllocateLocal(int world, int device, size_t bytes, std::vector<std::shared_ptr<SymmBuffer>>* out) {
  BFB_CUDA_OK(cudaSetDevice(device));
  auto owned = std::make_shared<std::vector<void*>>(world, nullptr);
  for (int r = 0; r < world; ++r) {
    BFB_CUDA_OK(cudaMalloc(&(*owned)[r], bytes));
    BFB_CUDA_OK(cudaMemset((*owned)[r], 0, bytes));
  }
  BFB_CUDA_OK(cudaDeviceSynchronize());
  out->clear();
  for (int r = 0; r < world; ++r) {
    auto buf = std::make_shared<SymmBuffer>();
    buf->rank = r;
    buf->world = world;
    buf->device = device;
    buf->bytes = bytes;
    buf->ipc = false;
    buf->ptrs = *owned;
    buf->local_owned = owned;
    out->push_back(buf);
  }
  return Status::OK();
}

}  // namespace bfb
