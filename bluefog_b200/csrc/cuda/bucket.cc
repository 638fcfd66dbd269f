#include "bucket.h"

#include <cstring>

namespace bfb {

Bucket::Bucket(std::unique_ptr<Channel> channel, uint64_t numel, int pub_elem)
    : channel_(std::move(channel)), numel_(numel), pub_elem_(pub_elem) {}

Status Bucket::Step(const BucketStepArgs& a, cudaStream_t stream) {
  Channel& ch = *channel_;
  if (a.src_ranks.size() != a.src_weights.size()) return Status::InvalidArgument("bucket step: ranks/weights differ in length");
  if (a.src_ranks.size() > static_cast<size_t>(kMaxSrc)) return Status::InvalidArgument("bucket step: too many sources");
  for (int r : a.src_ranks)
    if (r < 0 || r >= ch.world() || r == ch.rank()) return Status::InvalidArgument("bucket step: invalid source rank");
  const bool reads = a.mode == kModeAWC || a.mode == kModeCombineOnly || a.mode == kModeGradReduce;
  const bool writes_pub = a.mode == kModeAWC || a.mode == kModeAdaptPublish || a.mode == kModePublishOnly;
  if (reads && ch.next_version() == 0) return Status::PreconditionError("bucket step: nothing has been published yet");

  BucketParams p;
  std::memset(&p, 0, sizeof(p));
  p.mode = a.mode;
  p.opt = a.opt;
  p.pub_elem = pub_elem_;
  p.grad_elem = a.grad_elem;
  p.nesterov = a.nesterov;
  p.adamw = a.adamw;
  p.amsgrad = a.amsgrad;
  p.first_step = a.first_step;
  p.maximize = a.maximize;
  p.lr = static_cast<float>(a.lr);
  p.momentum = static_cast<float>(a.momentum);
  p.dampening = static_cast<float>(a.dampening);
  p.weight_decay = static_cast<float>(a.weight_decay);
  p.beta1 = static_cast<float>(a.beta1);
  p.beta2 = static_cast<float>(a.beta2);
  p.eps = static_cast<float>(a.eps);
  p.bias1 = static_cast<float>(a.bias1);
  p.bias2 = static_cast<float>(a.bias2);
  p.grad_scale = static_cast<float>(a.grad_scale);
  p.self_w = static_cast<float>(a.self_weight);
  p.post_scale = static_cast<float>(a.post_scale);
  p.numel = numel_;
  p.master = static_cast<float*>(a.master);
  p.grad = a.grad;
  p.grad_ptrs = a.grad_ptrs;
  p.seg_start = a.seg_start;
  p.seg_numel = a.seg_numel;
  p.n_seg = a.n_seg;
  if (a.grad_ptrs != nullptr && (a.n_seg <= 0 || a.seg_start == nullptr || a.seg_numel == nullptr))
    return Status::InvalidArgument("bucket step: incomplete gradient table");
  p.state1 = static_cast<float*>(a.state1);
  p.state2 = static_cast<float*>(a.state2);
  p.state3 = static_cast<float*>(a.state3);
  p.shadow = a.shadow;
  {
    // the state arrays the chosen optimizer reads and writes (the same table as in bucket_step_kernel) have to exist
    const bool updates = (a.mode == kModeAWC || a.mode == kModeAdaptPublish || a.mode == kModeGradReduce) &&
                         (a.grad != nullptr || a.grad_ptrs != nullptr);
    if (a.opt < kOptNone || a.opt > kOptAdadelta) return Status::InvalidArgument("bucket step: unknown optimizer");
    const bool need1 = (a.opt == kOptSGD && a.momentum != 0.0) || a.opt >= kOptAdam;
    const bool need2 = a.opt == kOptAdam || a.opt == kOptAdadelta || (a.opt == kOptRMSprop && a.momentum > 0.0);
    const bool need3 = (a.opt == kOptAdam || a.opt == kOptRMSprop) && a.amsgrad;
    if (updates && ((need1 && p.state1 == nullptr) || (need2 && p.state2 == nullptr) || (need3 && p.state3 == nullptr)))
      return Status::InvalidArgument("bucket step: an optimizer state buffer is missing");
  }

  PullSync& s = p.sync;
  s.my_rank = ch.rank();
  s.my_ctrl = ch.ctrl_ptr(ch.rank());
  s.status = ch.status_ptr();
  s.timeout_ns = ch.timeout_ns();
  s.counter_slot = 2;
  if (a.mode == kModeAnnounceWeights) {
    if (ch.next_version() == 0) return Status::PreconditionError("bucket step: nothing has been published yet");
    if (a.dst_weights.empty()) return Status::InvalidArgument("bucket step: no destination weights to announce");
    const uint64_t v_read = ch.next_version() - 1;
    s.half = static_cast<int>(v_read & 1);
    s.wait_epoch = v_read + 1;
  }
  if (reads) {
    const uint64_t v_read = ch.next_version() - 1;   // latest published version
    ch.AddReaders(v_read, a.n_readers);
    s.n_src = static_cast<int>(a.src_ranks.size());
    s.half = static_cast<int>(v_read & 1);
    s.wait_epoch = v_read + 1;
    s.signal_done = 1;
    // adapt-with-combine reads a version that was published before this step's weights were known: they are
    // announced separately (mode 2); every other mode finds them stored beside the version it reads
    if (a.read_dst_weights) s.use_dst_weight = a.mode == kModeAWC ? 2 : 1;
    for (size_t j = 0; j < a.src_ranks.size(); ++j) {
      s.src_ctrl[j] = ch.ctrl_ptr(a.src_ranks[j]);
      s.src_arena[j] = ch.arena_ptr(a.src_ranks[j], s.half);
      s.src_rank[j] = a.src_ranks[j];
      p.src_w[j] = static_cast<float>(a.src_weights[j]);
    }
    p.pub_read_self = ch.arena_ptr(ch.rank(), s.half);
  }
  if (writes_pub) {
    uint64_t need_done = 0;
    const uint64_t v_new = ch.TakeVersion(0, &need_done);
    p.pub_write = ch.arena_ptr(ch.rank(), static_cast<int>(v_new & 1));
    p.publish = 1;
    p.wait_done = 1;
    p.write_half = static_cast<int>(v_new & 1);
    p.need_done = need_done;
    p.publish_epoch = v_new + 1;
  }
  if (!a.dst_weights.empty()) {
    if (static_cast<int>(a.dst_weights.size()) != ch.world() || ch.world() > kMaxWorld)
      return Status::InvalidArgument("bucket step: destination weights need one entry per rank");
    p.world = ch.world();
    for (int r = 0; r < ch.world(); ++r) p.dst_weight[r] = static_cast<float>(a.dst_weights[r]);
    if ((a.mode == kModeAWC && reads) || a.mode == kModeAnnounceWeights) p.dst_weight_mode = 2;
    else if (writes_pub) p.dst_weight_mode = 1;
  }
  BFB_CUDA_OK(LaunchBucketStep(p, stream));
  return Status::OK();
}

}  // namespace bfb
