#include "gpu_channel.h"

#include <algorithm>
#include <cstring>

namespace bfb {

Channel::Channel(std::shared_ptr<SymmBuffer> ctrl, std::shared_ptr<SymmBuffer> arena, size_t half_bytes)
    : ctrl_(std::move(ctrl)), arena_(std::move(arena)), half_bytes_(half_bytes) {
  cudaHostAlloc(reinterpret_cast<void**>(&status_), sizeof(CommStatus), cudaHostAllocMapped | cudaHostAllocPortable);
  if (status_) *status_ = CommStatus{0, 0, 0, 0};
  if (const char* t = std::getenv("BLUEFOG_B200_WAIT_TIMEOUT_MS")) set_timeout_ms(std::atof(t));
}

Channel::~Channel() {
  if (status_) cudaFreeHost(status_);
}

void Channel::ResetArena(std::shared_ptr<SymmBuffer> arena, size_t half_bytes) {
  arena_ = std::move(arena);
  half_bytes_ = half_bytes;
}

uint64_t Channel::RequiredBytes(const std::vector<SegSpec>& segs) {
  uint64_t total = 0;
  for (const auto& s : segs) total += PaddedSize(s.nbytes);
  return total;
}

uint64_t Channel::TakeVersion(int n_readers, uint64_t* need_done) {
  const uint64_t v = version_++;
  const int half = static_cast<int>(v & 1);
  *need_done = readers_cum_[half];  // readers of every earlier version stored in this half
  readers_cum_[half] += static_cast<uint64_t>(n_readers);
  return v;
}

Status Channel::StatusToError() const {
  const CommStatus st = *status_;
  if (st.error == kCommOk) return Status::OK();
  std::string what = st.error == kCommTimeoutEpoch
                         ? "timed out waiting for rank " + std::to_string(st.peer) + " to publish version " +
                               std::to_string(st.want) + " (saw " + std::to_string(st.seen) + ")"
                         : st.error == kCommTimeoutDone
                               ? "timed out waiting for the readers of an earlier version (need " +
                                     std::to_string(st.want) + ", saw " + std::to_string(st.seen) + ")"
                               : st.error == kCommLayoutMismatch
                                     ? "the version rank " + std::to_string(st.peer) + " published does not have the layout this "
                                       "rank reads (expected " + std::to_string(st.want) + ", found " + std::to_string(st.seen) +
                                       "): tensor sizes differ between the ranks, or only some ranks passed a tensor of "
                                       "bf.symmetric_empty"
                                     : "invalid kernel argument";
  return Status::Aborted("peer-memory channel on rank " + std::to_string(rank()) + ": " + what +
                         ". The send/recv pattern of the ranks probably does not match.");
}

int SymmRegistry::Add(std::shared_ptr<SymmBuffer> buf) {
  bufs_.push_back(std::move(buf));
  return static_cast<int>(bufs_.size()) - 1;
}

bool SymmRegistry::Find(const void* p, uint64_t nbytes, RegisteredLoc* loc) const {
  const uintptr_t a = reinterpret_cast<uintptr_t>(p);
  if (p == nullptr || (a & 15) != 0) return false;
  for (size_t id = 0; id < bufs_.size(); ++id) {
    const SymmBuffer& b = *bufs_[id];
    const uintptr_t base = reinterpret_cast<uintptr_t>(b.local());
    if (a < base || a + nbytes > base + b.bytes) continue;
    const uint64_t off = a - base;
    loc->key = (static_cast<uint64_t>(id + 1) << 40) | off;
    loc->ptrs.resize(b.world);
    for (int r = 0; r < b.world; ++r) loc->ptrs[r] = static_cast<const unsigned char*>(b.ptrs[r]) + off;
    return true;
  }
  return false;
}

Status Channel::WaitReaders(const Round& round, cudaStream_t stream) {
  BFB_CUDA_OK(LaunchWaitReaders(ctrl_ptr(rank()), round.half, readers_cum_[round.half], timeout_ns_, status_, rank(), stream));
  return Status::OK();
}

Status Channel::Publish(const std::vector<SegSpec>& segs, const double* dst_weight, int n_readers,
                        cudaStream_t stream, Round* round, uint64_t loc) {
  if (loc != 0 && segs.size() != 1) return Status::InvalidArgument("a registered payload is one tensor");
  if (loc == 0 && RequiredBytes(segs) > half_bytes_)
    return Status::PreconditionError("channel arena too small for this payload");
  uint64_t need_done = 0;
  round->version = TakeVersion(n_readers, &need_done);
  round->half = static_cast<int>(round->version & 1);
  round->offsets.clear();
  uint64_t off = 0;
  for (const auto& s : segs) {
    round->offsets.push_back(off);
    off += PaddedSize(s.nbytes);
  }
  const size_t n = segs.size();
  size_t begin = 0;
  bool first = true;
  do {
    const size_t end = std::min(n, begin + static_cast<size_t>(kMaxSeg));
    PackParams p;
    std::memset(&p, 0, sizeof(p));
    p.ctrl = ctrl_ptr(rank());
    p.arena_half = arena_ptr(rank(), round->half);
    p.status = status_;
    p.need_done = need_done;
    p.publish_epoch = round->version + 1;
    p.timeout_ns = timeout_ns_;
    p.payload_bytes = off;
    p.loc = loc;
    p.half = round->half;
    p.wait_done = first ? 1 : 0;
    p.publish = end == n ? 1 : 0;
    p.world = world();
    p.my_rank = rank();
    p.n_seg = static_cast<int>(end - begin);
    p.has_dst_weight = dst_weight != nullptr;
    if (dst_weight)
      for (int r = 0; r < world(); ++r) p.dst_weight[r] = dst_weight[r];
    uint64_t chunks = 0;
    for (size_t i = begin; i < end; ++i) {
      const size_t k = i - begin;
      p.src[k] = segs[i].in;
      p.dst_off[k] = round->offsets[i];
      p.nbytes[k] = segs[i].nbytes;
      p.chunk_start[k] = chunks;
      if (loc == 0) chunks += (segs[i].nbytes + 15) / 16;          // registered: the header alone is published
    }
    p.chunk_start[p.n_seg] = chunks;
    BFB_CUDA_OK(LaunchPack(p, stream));
    begin = end;
    first = false;
  } while (begin < n);
  return Status::OK();
}

void Channel::FillSync(PullSync* s, const Round& round, const std::vector<int>& src_ranks, bool signal_done) {
  s->n_src = static_cast<int>(src_ranks.size());
  s->my_rank = rank();
  s->half = round.half;
  s->signal_done = signal_done ? 1 : 0;
  s->counter_slot = 1;
  s->wait_epoch = round.version + 1;
  s->timeout_ns = timeout_ns_;
  s->my_ctrl = ctrl_ptr(rank());
  s->status = status_;
  for (size_t j = 0; j < src_ranks.size(); ++j) {
    s->src_ctrl[j] = ctrl_ptr(src_ranks[j]);
    s->src_arena[j] = arena_ptr(src_ranks[j], round.half);
    s->src_rank[j] = src_ranks[j];
  }
}

Status Channel::PullCombine(const Round& round, const std::vector<SegSpec>& segs, int elem_type, double self_w,
                            const std::vector<int>& src_ranks, const std::vector<double>& src_w,
                            bool use_dst_weight, double post_scale, cudaStream_t stream, const RegisteredLoc* reg) {
  if (src_ranks.size() > static_cast<size_t>(kMaxSrc)) return Status::InvalidArgument("too many source ranks");
  if (reg != nullptr && (segs.size() != 1 || reg->key == 0 || reg->ptrs.size() != static_cast<size_t>(world())))
    return Status::InvalidArgument("a registered payload is one tensor with one address per rank");
  if (src_ranks.size() != src_w.size()) return Status::InvalidArgument("source ranks and weights differ in length");
  for (int r : src_ranks)
    if (r < 0 || r >= world() || r == rank()) return Status::InvalidArgument("invalid source rank " + std::to_string(r));
  const int esize = ElemSize(elem_type);
  const int per_vec = 16 / esize;
  const size_t n = segs.size();
  size_t begin = 0;
  do {
    const size_t end = std::min(n, begin + static_cast<size_t>(kMaxSeg));
    CombineParams p;
    std::memset(&p, 0, sizeof(p));
    FillSync(&p.sync, round, src_ranks, /*signal_done=*/end == n);
    p.sync.use_dst_weight = use_dst_weight ? 1 : 0;
    p.self_arena = arena_ptr(rank(), round.half);
    if (reg != nullptr) {
      // the own term and the sources that published the same registered tensor are read in place (offset 0 of the
      // round's layout); a source that copied into its arena is read from there
      p.self_arena = static_cast<const unsigned char*>(reg->ptrs[rank()]);
      p.my_loc = reg->key;
      for (size_t j = 0; j < src_ranks.size(); ++j) p.alt_src[j] = static_cast<const unsigned char*>(reg->ptrs[src_ranks[j]]);
    }
    p.self_w = self_w;
    p.post_scale = post_scale;
    for (size_t j = 0; j < src_w.size(); ++j) p.src_w[j] = src_w[j];
    p.elem_type = elem_type;
    p.n_seg = static_cast<int>(end - begin);
    uint64_t chunks = 0;
    for (size_t i = begin; i < end; ++i) {
      const size_t k = i - begin;
      p.out[k] = segs[i].out;
      p.off[k] = round.offsets[i] + segs[i].elem_offset * static_cast<uint64_t>(esize);
      p.numel[k] = segs[i].numel;
      p.chunk_start[k] = chunks;
      chunks += (segs[i].numel + per_vec - 1) / per_vec;
      const uint64_t end_byte = p.off[k] + segs[i].numel * static_cast<uint64_t>(esize);
      if (end_byte > p.need_bytes) p.need_bytes = end_byte;
    }
    p.chunk_start[p.n_seg] = chunks;
    BFB_CUDA_OK(LaunchCombine(p, stream));
    begin = end;
  } while (begin < n);
  return Status::OK();
}

Status Channel::PullGather(const Round& round, const std::vector<int>& src_ranks,
                           const std::vector<CopySpec>& copies, cudaStream_t stream) {
  if (src_ranks.size() > static_cast<size_t>(kMaxSrc)) return Status::InvalidArgument("too many source ranks");
  const size_t n = copies.size();
  size_t begin = 0;
  do {
    const size_t end = std::min(n, begin + static_cast<size_t>(kMaxSeg));
    GatherParams p;
    std::memset(&p, 0, sizeof(p));
    FillSync(&p.sync, round, src_ranks, /*signal_done=*/end == n);
    p.self_arena = arena_ptr(rank(), round.half);
    p.n_copy = static_cast<int>(end - begin);
    uint64_t chunks = 0;
    for (size_t i = begin; i < end; ++i) {
      const size_t k = i - begin;
      int idx = -1;
      if (copies[i].src_rank != rank()) {
        auto it = std::find(src_ranks.begin(), src_ranks.end(), copies[i].src_rank);
        if (it == src_ranks.end()) return Status::InvalidArgument("copy from a rank that is not a source");
        idx = static_cast<int>(it - src_ranks.begin());
      }
      p.copy_src[k] = idx;
      p.out[k] = copies[i].out;
      p.src_off[k] = copies[i].arena_off;
      p.nbytes[k] = copies[i].nbytes;
      p.chunk_start[k] = chunks;
      chunks += (copies[i].nbytes + 15) / 16;
    }
    p.chunk_start[p.n_copy] = chunks;
    BFB_CUDA_OK(LaunchGather(p, stream));
    begin = end;
  } while (begin < n);
  return Status::OK();
}

}  // namespace bfb
