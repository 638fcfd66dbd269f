// One-sided windows: registry, memory, mutexes, and the CPU/GPU implementations of
// create / free / put / accumulate / get / update.
//
// A window named N holds, on every rank, its "self" tensor, one slot per in-neighbor, a
// version counter and a push-sum weight p per source rank, and one mutex word per source
// rank.  CPU windows live in POSIX shared memory mapped by every rank of the box, so a
// put is a weighted copy into the target's mapping; GPU windows live in CUDA-IPC memory
// and are written by kernels (cuda/window_kernels.cu).  The mutex words of CPU windows live in host shared
// memory and are taken by the host with compare-and-swap; those of GPU windows live in the window's device
// header and are taken by a one-thread kernel on the stream of the operation (bounded wait, error status), so an
// operation under a mutex is three stream-ordered launches and never a host synchronisation.
// The target never takes part in a transfer, which is the passive-target behaviour of
// the reference's MPI-RMA windows (bluefog/common/mpi_controller.cc:795-1183,
// 1594-1663; bluefog/common/mpi_context.cc:53-170; bluefog/torch/mpi_win_ops.cc:83-426).
#pragma once
#include <torch/extension.h>

#include <atomic>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "control_plane.h"
#include "status.h"

namespace bfb {

struct SymmBuffer;
struct OpSpec;

struct ShmSegment {
  std::string name;
  void* base = nullptr;
  size_t bytes = 0;
  bool created = false;
  ~ShmSegment();
};

struct Window {
  std::string name;
  int id = 0;
  bool on_gpu = false;
  int device = -1;
  at::ScalarType dtype = at::kFloat;
  std::vector<int64_t> shape;
  uint64_t numel = 0, nbytes = 0, padded = 0;
  int num_slots = 0;
  std::vector<int> in_neighbors;   // slot k belongs to in_neighbors[k]
  // host shared memory of every rank (mutex words; for CPU windows also header + data)
  std::vector<std::shared_ptr<ShmSegment>> shm;
  // device symmetric memory (GPU windows)
  std::shared_ptr<SymmBuffer> dev;
  at::Tensor self_view;            // tensor aliasing the self region
  unsigned int* block_counter = nullptr;  // device scratch for the kernels (GPU windows)

  size_t data_offset() const;      // offset of the window data block (WinHeader) inside shm (CPU)
  unsigned char* data_base(int rank) const;   // start of [WinHeader | self | slots] of a rank
  unsigned char* self_ptr(int rank) const;
  unsigned char* slot_ptr(int rank, int k) const;
  std::atomic<int>* mutex_word(int owner, int source) const;
  // Guard words: the last 16 bytes of every region (self and each slot) of this rank's block lie behind the tensor
  // and behind anything a kernel may write for it (whole 16-byte vectors); they hold a fixed pattern from win_create
  // to win_free, where a changed pattern means that some rank wrote past the end of a region.
  static constexpr size_t kGuardBytes = 16;
  void WriteGuards(int rank) const;
  int DamagedGuards(int rank) const;          // how many regions of the rank's block have a changed guard
};

class WindowManager {
 public:
  WindowManager(ControlPlane* cp, int rank, int size, const std::string& job_tag)
      : cp_(cp), rank_(rank), size_(size), job_tag_(job_tag) {}
  ~WindowManager();

  // Collective (run on the background thread after negotiation).
  Status Create(const OpSpec& spec, int channel);
  Status Free(const std::string& name, int channel);   // empty name = all windows
  // One-sided transfers (background thread). stream = cudaStream_t for GPU windows.
  Status Put(const OpSpec& spec, void* stream);
  Status Get(const OpSpec& spec, void* stream);
  // Local combine (calling thread).
  Status Update(const std::string& name, at::Tensor out, double self_weight, const std::vector<int>& src_ranks,
                const std::vector<double>& src_weights, bool reset, bool require_mutex, void* stream);

  Status MutexAcquire(const std::string& name, const std::vector<int>& ranks, bool for_self);
  Status MutexRelease(const std::string& name, const std::vector<int>& ranks, bool for_self);
  Status Versions(const std::string& name, std::vector<int64_t>* versions);
  Status GetAssociatedP(const std::string& name, double* p);
  Status SetAssociatedP(const std::string& name, double p);
  void set_with_associated_p(bool v) { with_p_.store(v); }
  bool with_associated_p() const { return with_p_.load(); }
  at::Tensor SelfView(const std::string& name);
  std::vector<std::string> Names();
  size_t Count();
  double mutex_timeout_s = 120.0;
  // Error left by a device-side mutex wait that ran out since the last call (OK when none); clears it.
  Status TakeDeviceError();

 private:
  // Launches the lock (acquire) or unlock kernel for the words `ranks` of a GPU window on `stream`.
  // for_self: words lock[r] of my own header (win_update); otherwise word lock[my rank] of every rank r's header.
  // user: the state block of explicit win_mutex calls instead of the one that guards the operation kernels.
  Status DeviceLock(Window& w, const std::vector<int>& ranks, bool for_self, bool acquire, bool user, void* stream);
  void* dev_status_host_ = nullptr;   // pinned, mapped CommStatus written by the lock kernel
  void* dev_status_dev_ = nullptr;
  std::shared_ptr<Window> Find(const std::string& name);
  Status FreeOne(std::shared_ptr<Window> w);
  ControlPlane* cp_;
  int rank_, size_;
  std::string job_tag_;
  std::mutex mu_;
  std::map<std::string, std::shared_ptr<Window>> windows_;
  int next_id_ = 0;
  std::atomic<bool> with_p_{false};
};

}  // namespace bfb
