// Host side of a communication channel (see comm_kernels.h for the device protocol):
// owns the symmetric control block and arena, hands out version numbers, keeps the
// reader accounting that tells a publisher when an arena half may be overwritten, and
// turns tensor lists into kernel launches.
#pragma once
#include <memory>
#include <vector>

#include "comm_kernels.h"
#include "symm_mem.h"

namespace bfb {

struct SegSpec {
  const void* in = nullptr;   // publish: source of the payload
  void* out = nullptr;        // pull: destination
  uint64_t nbytes = 0;        // payload bytes of this tensor
  uint64_t numel = 0;
  uint64_t elem_offset = 0;   // pull: first element of the published tensor that is combined
};

struct Round {
  uint64_t version = 0;
  int half = 0;
  std::vector<uint64_t> offsets;  // per tensor, byte offset inside the arena half
};

// A tensor that lives in registered symmetric memory (the same allocation on every rank, all of them mapped into
// this process): it is published in place - no copy into the arena - and neighbors pull it from where it is.
struct RegisteredLoc {
  uint64_t key = 0;                // (buffer id + 1) << 40 | byte offset inside the buffer; 0 = not registered
  std::vector<const void*> ptrs;   // ptrs[r]: the tensor's address in rank r's buffer
};

// The registered buffers of one rank, in allocation order (allocation is collective, so ids agree across ranks).
class SymmRegistry {
 public:
  int Add(std::shared_ptr<SymmBuffer> buf);
  // Whether [p, p + nbytes) lies inside one of this rank's registered buffers and starts on a 16-byte boundary.
  bool Find(const void* p, uint64_t nbytes, RegisteredLoc* loc) const;
  size_t size() const { return bufs_.size(); }
  void Clear() { bufs_.clear(); }

 private:
  std::vector<std::shared_ptr<SymmBuffer>> bufs_;
};

class Channel {
 public:
  Channel(std::shared_ptr<SymmBuffer> ctrl, std::shared_ptr<SymmBuffer> arena, size_t half_bytes);
  ~Channel();
  int rank() const { return ctrl_->rank; }
  int world() const { return ctrl_->world; }
  size_t half_bytes() const { return half_bytes_; }
  uint64_t next_version() const { return version_; }
  void set_timeout_ms(double ms) { timeout_ns_ = static_cast<unsigned long long>(ms * 1e6); }
  // Replaces the arena after a collective re-allocation; all in-flight work must be finished.
  void ResetArena(std::shared_ptr<SymmBuffer> arena, size_t half_bytes);

  static uint64_t PaddedSize(uint64_t nbytes) { return (nbytes + 255) & ~uint64_t(255); }
  static uint64_t RequiredBytes(const std::vector<SegSpec>& segs);

  // Publishes one version holding the given tensors (possibly none). n_readers = how many
  // ranks will pull this version. dst_weight: world entries or nullptr.
  // loc != 0: the (single) tensor of this version stays where it is, in registered memory with that key; segs
  // still describes it (sizes and layout are the same on every rank) but nothing is copied.
  Status Publish(const std::vector<SegSpec>& segs, const double* dst_weight, int n_readers,
                 cudaStream_t stream, Round* round, uint64_t loc = 0);
  // out = post_scale * (self_w * mine + sum_j w_j * [dstw_j] * src_j) for every tensor of the round.
  Status PullCombine(const Round& round, const std::vector<SegSpec>& segs, int elem_type, double self_w,
                     const std::vector<int>& src_ranks, const std::vector<double>& src_w,
                     bool use_dst_weight, double post_scale, cudaStream_t stream, const RegisteredLoc* reg = nullptr);
  // Returns (on the stream) once every reader of the versions published so far in the round's half has finished.
  Status WaitReaders(const Round& round, cudaStream_t stream);
  // Copies: for each item, nbytes from rank src's (or my own) version of tensor `seg_index`
  // starting at src_byte_off into out.
  struct CopySpec {
    int src_rank;
    uint64_t arena_off;
    uint64_t nbytes;
    void* out;
  };
  Status PullGather(const Round& round, const std::vector<int>& src_ranks, const std::vector<CopySpec>& copies,
                    cudaStream_t stream);

  // Status word written by kernels; valid after the stream work has completed.
  CommStatus ReadStatus() const { return *status_; }
  void ClearStatus() { *status_ = CommStatus{0, 0, 0, 0}; }
  Status StatusToError() const;

  ChannelCtrl* ctrl_ptr(int r) const { return static_cast<ChannelCtrl*>(ctrl_->ptrs[r]); }
  unsigned char* arena_ptr(int r, int half) const {
    return static_cast<unsigned char*>(arena_->ptrs[r]) + static_cast<size_t>(half) * half_bytes_;
  }
  CommStatus* status_ptr() const { return status_; }
  unsigned long long timeout_ns() const { return timeout_ns_; }

  // Version / reader bookkeeping shared with the bucket path.
  uint64_t TakeVersion(int n_readers, uint64_t* need_done);
  // Bucket path: the readers of a version are only known when the *next* step is issued
  // (dynamic topologies), so they are added separately from taking the version.
  void AddReaders(uint64_t version, int n_readers) { readers_cum_[version & 1] += static_cast<uint64_t>(n_readers); }
  std::shared_ptr<SymmBuffer> arena() const { return arena_; }

 private:
  void FillSync(PullSync* s, const Round& round, const std::vector<int>& src_ranks, bool signal_done);
  std::shared_ptr<SymmBuffer> ctrl_;
  std::shared_ptr<SymmBuffer> arena_;
  size_t half_bytes_;
  uint64_t version_ = 0;
  uint64_t readers_cum_[2] = {0, 0};
  CommStatus* status_ = nullptr;
  unsigned long long timeout_ns_ = 30ull * 1000 * 1000 * 1000;
};

}  // namespace bfb
