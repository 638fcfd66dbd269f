// Parameter buckets: the optimizer fast path.
//
// A bucket is a flat fp32 "master" buffer that holds many parameters back to back (what
// the reference calls a fusion group, bluefog/common/operations.cc:990-1008, except that
// the tensors live there permanently, so nothing is packed or unpacked per step).  Each
// bucket owns a channel whose arena halves hold the *published* copy of the bucket (fp32
// or bf16) that the neighbors read.  One kernel launch per bucket and step reads the
// in-neighbors' published copies over NVLink, forms the weighted combine, applies the
// SGD/Adam update, and writes the new master, the new published copy and the bf16 shadow
// used by forward/backward (K5+K6+K7 of the reference fused into one pass).
#pragma once
#include <memory>
#include <vector>

#include "gpu_channel.h"

namespace bfb {

struct BucketStepArgs {
  int mode = kModeAWC;
  int opt = kOptNone;
  int grad_elem = kF32;
  bool nesterov = false, adamw = false, amsgrad = false, first_step = false, maximize = false;
  double lr = 0, momentum = 0, dampening = 0, weight_decay = 0, beta1 = 0.9, beta2 = 0.999, eps = 1e-8;
  double bias1 = 1, bias2 = 1, grad_scale = 1, self_weight = 1, post_scale = 1;
  std::vector<int> src_ranks;
  std::vector<double> src_weights;
  int n_readers = 0;            // ranks that read the version this step consumes (my dst list)
  // Destination weights (world entries; empty = not used).  When used, every rank of the step must use them:
  // the readers then wait for and apply their sources' weights.
  std::vector<double> dst_weights;
  bool read_dst_weights = false;   // the sources attach destination weights to the version this step reads
  void* master = nullptr;
  const void* grad = nullptr;
  const void* const* grad_ptrs = nullptr;              // device array, see BucketParams
  const unsigned long long* seg_start = nullptr;       // device arrays of n_seg entries
  const unsigned long long* seg_numel = nullptr;
  int n_seg = 0;
  void* state1 = nullptr;
  void* state2 = nullptr;
  void* state3 = nullptr;
  void* shadow = nullptr;
};

class Bucket {
 public:
  Bucket(std::unique_ptr<Channel> channel, uint64_t numel, int pub_elem);
  uint64_t numel() const { return numel_; }
  int pub_elem() const { return pub_elem_; }
  Channel* channel() { return channel_.get(); }
  uint64_t versions_published() const { return channel_->next_version(); }
  Status Step(const BucketStepArgs& a, cudaStream_t stream);
  static uint64_t PubBytes(uint64_t numel, int pub_elem) {
    const uint64_t padded = (numel + 63) & ~uint64_t(63);
    return padded * static_cast<uint64_t>(ElemSize(pub_elem));
  }

 private:
  std::unique_ptr<Channel> channel_;
  uint64_t numel_;
  int pub_elem_;
};

}  // namespace bfb
