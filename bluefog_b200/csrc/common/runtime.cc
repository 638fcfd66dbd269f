#include "runtime.h"

#include <dlfcn.h>
#include <poll.h>
#include <sys/eventfd.h>
#include <unistd.h>

#include <ATen/Parallel.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "../cuda/gpu_channel.h"
#include "../cuda/symm_mem.h"
#include "logging.h"
#include "windows.h"

namespace bfb {

namespace {

using Clock = std::chrono::steady_clock;

double EnvDouble(const char* name, double fallback) {
  const char* v = std::getenv(name);
  return v ? std::atof(v) : fallback;
}

uint64_t Fnv(uint64_t h, const void* data, size_t n) {
  const unsigned char* p = static_cast<const unsigned char*>(data);
  for (size_t i = 0; i < n; ++i) {
    h ^= p[i];
    h *= 1099511628211ull;
  }
  return h;
}

int ToElem(at::ScalarType t) {
  switch (t) {
    case at::kFloat: return kF32;
    case at::kDouble: return kF64;
    case at::kHalf: return kF16;
    case at::kBFloat16: return kBF16;
    case at::kInt: return kI32;
    case at::kLong: return kI64;
    default: return -1;
  }
}

bool IsReduceOp(OpType t) {
  return t == OpType::ALLREDUCE || t == OpType::NEIGHBOR_ALLREDUCE || t == OpType::PAIR_GOSSIP;
}

const char* ProcActivity(OpType t) {
  switch (t) {
    case OpType::ALLREDUCE: return "PROC_ALLREDUCE";
    case OpType::ALLGATHER: return "PROC_ALLGATHER";
    case OpType::BROADCAST: return "PROC_BROADCAST";
    case OpType::NEIGHBOR_ALLREDUCE: return "PROC_NEIGHBOR_ALLREDUCE";
    case OpType::NEIGHBOR_ALLGATHER: return "PROC_NEIGHBOR_ALLGATHER";
    case OpType::PAIR_GOSSIP: return "PROC_PAIR_GOSSIP";
    case OpType::WIN_CREATE: return "WIN_CREATE";
    case OpType::WIN_FREE: return "WIN_FREE";
    case OpType::WIN_PUT: return "WIN_PUT";
    case OpType::WIN_GET: return "WIN_GET";
    case OpType::WIN_ACCUMULATE: return "WIN_ACCUMULATE";
    case OpType::BARRIER: return "PROC_BARRIER";
    default: return "PROC_UNKNOWN";
  }
}

}  // namespace

DataType ToDataType(at::ScalarType t, bool* ok) {
  *ok = true;
  switch (t) {
    case at::kByte: return DataType::UINT8;
    case at::kChar: return DataType::INT8;
    case at::kShort: return DataType::INT16;
    case at::kInt: return DataType::INT32;
    case at::kLong: return DataType::INT64;
    case at::kHalf: return DataType::FLOAT16;
    case at::kBFloat16: return DataType::BFLOAT16;
    case at::kFloat: return DataType::FLOAT32;
    case at::kDouble: return DataType::FLOAT64;
    case at::kBool: return DataType::BOOL;
    default: *ok = false; return DataType::BYTE;
  }
}

uint64_t NeighborSignature(const OpSpec& spec) {
  uint64_t h = 1469598103934665603ull;
  auto add_vec_i = [&](const std::vector<int>& v) {
    uint64_t n = v.size();
    h = Fnv(h, &n, sizeof(n));
    if (!v.empty()) h = Fnv(h, v.data(), v.size() * sizeof(int));
  };
  auto add_vec_d = [&](const std::vector<double>& v) {
    uint64_t n = v.size();
    h = Fnv(h, &n, sizeof(n));
    if (!v.empty()) h = Fnv(h, v.data(), v.size() * sizeof(double));
  };
  add_vec_i(spec.src_ranks);
  add_vec_d(spec.src_weights);
  add_vec_i(spec.dst_ranks);
  add_vec_d(spec.dst_weights);
  h = Fnv(h, &spec.self_weight, sizeof(double));
  h = Fnv(h, &spec.post_scale, sizeof(double));
  unsigned char flags = (spec.use_dst_weight ? 1 : 0) | (spec.enable_topo_check ? 2 : 0);
  h = Fnv(h, &flags, 1);
  return h;
}

Runtime& Runtime::Get() {
  static Runtime* rt = new Runtime();  // leaked on purpose: outlives static destructors
  return *rt;
}

// ----------------------------------------------------------------------------------------
// lifecycle
// ----------------------------------------------------------------------------------------
Status Runtime::Listen(const std::string& bind_addr, int* port) { return cp_.Listen(bind_addr, port); }

Status Runtime::Init(int rank, int size, int local_rank, int local_size,
                     const std::vector<std::string>& endpoints, int device) {
  if (initialized_.load()) return Status::OK();
  rank_ = rank;
  size_ = size;
  local_rank_ = local_rank;
  local_size_ = local_size;
  device_ = device;
  if (size > kMaxWorld) return Status::InvalidArgument("at most 64 ranks are supported");
  Status s = cp_.Connect(rank, size, endpoints, EnvDouble("BLUEFOG_START_TIMEOUT", 600.0));
  if (!s.ok()) return s;
  fusion_threshold_ = static_cast<int64_t>(EnvDouble("BLUEFOG_FUSION_THRESHOLD", 8.0 * 1024 * 1024));
  cycle_time_ms_ = EnvDouble("BLUEFOG_CYCLE_TIME", 0.5);
  stall_warning_s_ = EnvDouble("BLUEFOG_STALL_WARNING_SECONDS", 60.0);
  if (const char* prefix = std::getenv("BLUEFOG_TIMELINE"))
    timeline_.Initialize(std::string(prefix) + std::to_string(rank) + ".json", size);
  // A job-wide tag for shared-memory names: rank 0's pid and start time, shared with everyone.
  std::string tag;
  if (rank == 0) {
    char buf[64];
    std::snprintf(buf, sizeof(buf), "%d_%lld", static_cast<int>(getpid()),
                  static_cast<long long>(std::chrono::duration_cast<std::chrono::microseconds>(
                                             std::chrono::system_clock::now().time_since_epoch()).count() % 100000000));
    tag = buf;
  }
  s = cp_.BroadcastBytes(kChanUser, 0, &tag);
  if (!s.ok()) return s;
  windows_ = std::make_unique<WindowManager>(&cp_, rank, size, tag);
  windows_->mutex_timeout_s = EnvDouble("BLUEFOG_B200_MUTEX_TIMEOUT_SECONDS", 120.0);
  finalizers_.create(static_cast<int>(EnvDouble("BLUEFOG_NUM_FINALIZER_THREADS", 1)));
  inline_enabled_ = EnvDouble("BLUEFOG_B200_INLINE_OPS", 1.0) != 0.0;
  wake_fd_ = eventfd(0, EFD_NONBLOCK);
  shutdown_requested_.store(false);
  loop_exited_.store(false);
  shutdown_sent_ = false;
  any_shutdown_ = false;
  last_stall_check_ = Clock::now();
  initialized_.store(true);
  thread_ = std::thread([this] { Loop(); });
  return Status::OK();
}

void Runtime::Wake() {
  if (wake_fd_ >= 0) {
    uint64_t one = 1;
    ssize_t r = ::write(wake_fd_, &one, sizeof(one));
    (void)r;
  }
}

void Runtime::KeepUntilShutdown(std::shared_ptr<void> memory) {
  std::lock_guard<std::mutex> g(keep_mu_);
  keep_until_shutdown_.push_back(std::move(memory));
}

Status Runtime::SymmetricAlloc(size_t bytes, std::shared_ptr<SymmBuffer>* out) {
  if (!initialized_.load()) return Status::PreconditionError("bluefog is not initialized");
  if (device_ < 0) return Status::PreconditionError("symmetric memory needs a CUDA device");
  if (bytes == 0) return Status::InvalidArgument("symmetric allocation of zero bytes");
  c10::cuda::CUDAGuard guard(device_);
  Status s = AllocateIpc(&cp_, kChanUser, device_, (bytes + 255) & ~size_t(255), out);
  if (!s.ok()) return s;
  KeepUntilShutdown(*out);
  std::lock_guard<std::mutex> g(reg_mu_);
  if (!registered_) registered_ = std::make_unique<SymmRegistry>();
  registered_->Add(*out);
  return Status::OK();
}

bool Runtime::FindRegistered(const void* p, uint64_t nbytes, RegisteredLoc* loc) {
  std::lock_guard<std::mutex> g(reg_mu_);
  return registered_ != nullptr && registered_->Find(p, nbytes, loc);
}

void Runtime::Shutdown() {
  if (!initialized_.load()) return;
  {
    // fast-path operations nobody waited for: finish them before the channel goes away
    std::vector<int> pending;
    {
      std::lock_guard<std::mutex> g(inline_mu_);
      for (auto& kv : inline_ops_) pending.push_back(kv.first);
    }
    bool finished = false;
    for (int h : pending) CompleteInline(h, /*block=*/true, &finished);
  }
  shutdown_requested_.store(true);
  Wake();
  if (thread_.joinable()) thread_.join();
  finalizers_.reset();
  if (device_ >= 0) {
    cudaSetDevice(device_);
    cudaDeviceSynchronize();
  }
  if (size_ > 1 && cp_.connected()) {
    // Every rank's kernels have finished (device synchronised above) once all ranks are here: only then is peer-
    // mapped memory (windows, channels, bucket arenas) unmapped.  The wait is bounded; a rank that never comes
    // costs the others this long at exit and nothing else.
    double limit_s = 10.0;
    if (const char* v = std::getenv("BLUEFOG_B200_SHUTDOWN_BARRIER_SECONDS")) limit_s = std::atof(v);
    if (limit_s > 0) {
      Status s = cp_.Barrier(kChanData, limit_s);
      if (!s.ok()) BFLOG(WARNING, rank_) << "shutdown barrier not completed (" << s.reason() << "); releasing peer memory anyway";
    }
  }
  if (windows_) {
    windows_.reset();
  }
  {
    std::lock_guard<std::mutex> g(reg_mu_);
    registered_.reset();
  }
  {
    std::lock_guard<std::mutex> g(keep_mu_);
    keep_until_shutdown_.clear();
  }
  gpu_channel_.reset();
  gpu_ctrl_.reset();
  pair_channels_.clear();
  if (comm_stream_) {
    cudaStreamDestroy(static_cast<cudaStream_t>(comm_stream_));
    comm_stream_ = nullptr;
  }
  timeline_.Shutdown();
  cp_.Close();
  if (wake_fd_ >= 0) {
    ::close(wake_fd_);
    wake_fd_ = -1;
  }
  message_table_.clear();
  ready_names_.clear();
  initialized_.store(false);
}

// ----------------------------------------------------------------------------------------
// handles
// ----------------------------------------------------------------------------------------
std::map<std::string, uint64_t> Runtime::StatsSnapshot() const {
  std::map<std::string, uint64_t> out;
  for (int t = 0; t < kStatOpTypes; ++t) {
    const uint64_t n = stats_.enqueued[t].load();
    if (n != 0) out[std::string("enqueued.") + OpTypeName(static_cast<OpType>(t))] = n;
  }
  out["input_bytes"] = stats_.input_bytes.load();
  out["issued_on_calling_thread"] = stats_.inline_issued.load();
  out["responses_executed"] = stats_.responses.load();
  out["tensors_in_fused_responses"] = stats_.fused_tensors.load();
  out["operations_failed"] = stats_.errors.load();
  return out;
}

void Runtime::MarkDone(int handle, const Status& s) {
  if (!s.ok() && !s.in_progress()) stats_.errors.fetch_add(1);
  {
    std::lock_guard<std::mutex> g(handle_mu_);
    auto it = handles_.find(handle);
    if (it != handles_.end()) it->second = s;
  }
  handle_cv_.notify_all();
}

bool Runtime::Poll(int handle) {
  bool finished = false;
  CompleteInline(handle, /*block=*/false, &finished);   // no-op for handles of the queued path
  std::lock_guard<std::mutex> g(handle_mu_);
  auto it = handles_.find(handle);
  if (it == handles_.end()) return true;
  return !it->second.in_progress();
}

Status Runtime::Wait(int handle) {
  bool finished = false;
  CompleteInline(handle, /*block=*/true, &finished);
  std::unique_lock<std::mutex> lk(handle_mu_);
  auto it = handles_.find(handle);
  if (it == handles_.end()) return Status::InvalidArgument("unknown handle " + std::to_string(handle));
  handle_cv_.wait(lk, [&] { return !handles_[handle].in_progress(); });
  Status s = handles_[handle];
  handles_.erase(handle);
  return s;
}

void Runtime::Release(int handle) {
  bool finished = false;
  CompleteInline(handle, /*block=*/true, &finished);
  std::lock_guard<std::mutex> g(handle_mu_);
  handles_.erase(handle);
}

// ----------------------------------------------------------------------------------------
// fast path: issue on the calling thread
// ----------------------------------------------------------------------------------------
thread_local bool Runtime::tls_inline_ = false;

bool Runtime::InlineEligible(const OpSpec& spec) const {
  if (!inline_enabled_ || device_ < 0) return false;
  if (spec.negotiate && !skip_negotiate_.load() && size_ > 1) return false;
  const OpType type = static_cast<OpType>(spec.type);
  if (type != OpType::ALLREDUCE && type != OpType::BROADCAST && type != OpType::ALLGATHER &&
      type != OpType::NEIGHBOR_ALLGATHER && type != OpType::NEIGHBOR_ALLREDUCE && type != OpType::PAIR_GOSSIP)
    return false;
  const at::Tensor* t = spec.input.has_value() ? &*spec.input : (spec.output.has_value() ? &*spec.output : nullptr);
  return t != nullptr && t->is_cuda();
}

bool Runtime::TryRunInline(Entry& e) {
  std::unique_lock<std::mutex> ex(exec_mu_, std::try_to_lock);
  if (!ex.owns_lock()) return false;                 // the background loop is executing something
  {
    // anything queued or waiting for a response keeps its place in front of this operation
    std::lock_guard<std::mutex> q(queue_mu_);
    if (!queue_.empty()) return false;
  }
  {
    std::lock_guard<std::mutex> t(table_mu_);
    if (!table_.empty()) return false;
  }
  const std::string name = e.spec.name;
  const int handle = e.handle;
  {
    std::lock_guard<std::mutex> g(inline_mu_);
    if (inline_names_.count(name)) {
      timeline_.ActivityEnd(name);
      if (e.ready_event) cudaEventDestroy(static_cast<cudaEvent_t>(e.ready_event));
      MarkDone(handle, Status::InvalidArgument(DuplicateNameError(name)));
      return true;
    }
    inline_names_[name] = handle;
  }
  c10::cuda::CUDAGuard guard(device_);
  Response r;
  r.type = static_cast<OpType>(e.spec.type);
  r.names = {name};
  std::vector<Entry> entries;
  entries.push_back(std::move(e));
  tls_inline_ = true;
  ExecuteEntries(entries, r);
  tls_inline_ = false;
  {
    // finished on the spot (an error, or nothing left in flight): the name is free again
    std::lock_guard<std::mutex> g(inline_mu_);
    if (!inline_ops_.count(handle)) inline_names_.erase(name);
  }
  return true;
}

// Finishes a fast-path handle: waits for (block) or queries its completion event, turns a device-side
// wait limit into an error, frees the events and records the final status.
Status Runtime::CompleteInline(int handle, bool block, bool* finished) {
  InlineOp op;
  {
    std::lock_guard<std::mutex> g(inline_mu_);
    auto it = inline_ops_.find(handle);
    if (it == inline_ops_.end()) {
      *finished = true;
      return Status::OK();
    }
    if (!block && cudaEventQuery(static_cast<cudaEvent_t>(it->second.done_event)) == cudaErrorNotReady) {
      *finished = false;
      return Status::OK();
    }
    op = std::move(it->second);
    inline_ops_.erase(it);
  }
  cudaError_t err = cudaEventSynchronize(static_cast<cudaEvent_t>(op.done_event));
  if (op.span_start) {
    std::vector<std::string> names;
    for (auto& e : *op.keep) names.push_back(e.spec.name);
    EmitDeviceSpan(names, op.span_start, err == cudaSuccess ? op.done_event : nullptr);
  }
  cudaEventDestroy(static_cast<cudaEvent_t>(op.done_event));
  Status s = err == cudaSuccess ? Status::OK() : Status::UnknownError("CUDA error: " + CudaErrorString(err));
  if (s.ok()) s = GpuStatusToError();
  for (auto& e : *op.keep) {
    timeline_.ActivityEnd(e.spec.name);   // ENQUEUE_*
    if (e.ready_event) cudaEventDestroy(static_cast<cudaEvent_t>(e.ready_event));
    {
      std::lock_guard<std::mutex> g(inline_mu_);
      inline_names_.erase(e.spec.name);
    }
    MarkDone(e.handle, s);
  }
  op.keep->clear();
  *finished = true;
  return s;
}

int Runtime::Enqueue(OpSpec spec) {
  int handle;
  {
    std::lock_guard<std::mutex> g(handle_mu_);
    handle = next_handle_++;
    handles_[handle] = Status::InProgress();
  }
  if (!initialized_.load() || loop_exited_.load()) {
    MarkDone(handle, initialized_.load() ? Status::Aborted(kShutDownError()) : Status::PreconditionError(kNotInitializedError()));
    return handle;
  }
  if (suspended_.load()) {
    MarkDone(handle, Status::PreconditionError(kSuspendError()));
    return handle;
  }
  if (spec.type >= 0 && spec.type < kStatOpTypes) stats_.enqueued[spec.type].fetch_add(1);
  if (spec.input.has_value() && spec.input->defined()) stats_.input_bytes.fetch_add(static_cast<uint64_t>(spec.input->nbytes()));
  Entry e;
  e.handle = handle;
  e.enqueued = Clock::now();
  // Work queued on the producer's stream must be finished before the payload is read.
  const at::Tensor* probe = spec.input.has_value() ? &*spec.input : (spec.output.has_value() ? &*spec.output : nullptr);
  if (probe != nullptr && probe->is_cuda()) {
    c10::cuda::CUDAGuard guard(probe->get_device());
    cudaEvent_t ev;
    cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
    cudaEventRecord(ev, c10::cuda::getCurrentCUDAStream(probe->get_device()).stream());
    e.ready_event = ev;
  }
  timeline_.ActivityStart(spec.name, std::string("ENQUEUE_") + OpTypeName(static_cast<OpType>(spec.type)));
  e.spec = std::move(spec);
  if (InlineEligible(e.spec) && TryRunInline(e)) {
    stats_.inline_issued.fetch_add(1);
    return handle;
  }
  {
    std::lock_guard<std::mutex> g(queue_mu_);
    queue_.push_back(std::move(e));
  }
  Wake();
  return handle;
}

Status Runtime::BarrierNow() {
  std::lock_guard<std::mutex> g(user_chan_mu_);
  return cp_.Barrier(kChanUser);
}

Status Runtime::AllgatherBytesNow(const std::string& mine, std::vector<std::string>* all) {
  std::lock_guard<std::mutex> g(user_chan_mu_);
  return cp_.AllgatherBytes(kChanUser, mine, all);
}

// ----------------------------------------------------------------------------------------
// background loop
// ----------------------------------------------------------------------------------------
void Runtime::DrainLocalQueue(RequestList* outgoing, std::vector<std::string>* immediate) {
  std::deque<Entry> local;
  {
    std::lock_guard<std::mutex> g(queue_mu_);
    local.swap(queue_);
  }
  for (auto& e : local) {
    const std::string name = e.spec.name;
    {
      std::lock_guard<std::mutex> g(table_mu_);
      if (table_.count(name)) {
        timeline_.ActivityEnd(name);
        MarkDone(e.handle, Status::InvalidArgument(DuplicateNameError(name)));
        if (e.ready_event) cudaEventDestroy(static_cast<cudaEvent_t>(e.ready_event));
        continue;
      }
    }
    const bool negotiate = e.spec.negotiate && !skip_negotiate_.load() && size_ > 1;
    if (negotiate) {
      Request q;
      q.rank = rank_;
      q.type = static_cast<OpType>(e.spec.type);
      q.name = name;
      q.root_rank = e.spec.root_rank;
      q.is_hierarchical = e.spec.is_hierarchical;
      q.neighbor_sig = NeighborSignature(e.spec);
      const at::Tensor* t = e.spec.input.has_value() ? &*e.spec.input : (e.spec.output.has_value() ? &*e.spec.output : nullptr);
      if (t != nullptr) {
        bool ok;
        q.dtype = ToDataType(t->scalar_type(), &ok);
        q.device = t->is_cuda() ? t->get_device() : -1;
        q.shape = t->sizes().vec();
        q.nbytes = static_cast<uint64_t>(t->numel()) * t->element_size();
      }
      outgoing->requests.push_back(std::move(q));
    } else {
      immediate->push_back(name);
    }
    std::lock_guard<std::mutex> g(table_mu_);
    table_.emplace(name, std::move(e));
  }
}

// ATen parallelises CPU arithmetic with OpenMP, and every thread that enters a parallel region gets a team of
// its own.  On the communication thread that means: per rank a second team of as many threads as the machine has
// cores, spinning between operations next to the training thread's team.  Four ranks on eight cores spent 130 ms on
// a neighbor_allreduce of 100 000 floats that way, against 1.4 ms with the combine kept on the calling thread.
// OpenMP's thread count is a per-thread setting, so this limits only the thread that calls it.
// BLUEFOG_B200_CPU_COMBINE_THREADS (default 1) is the team size of the communication thread.
void LimitIntraOpThreadsOfThisThread() {
  int n = 1;
  if (const char* v = std::getenv("BLUEFOG_B200_CPU_COMBINE_THREADS")) n = std::max(1, std::atoi(v));
  at::internal::lazy_init_num_threads();      // ATen's own first-use initialisation of this thread comes first
  using SetFn = void (*)(int);
  static SetFn set_threads = reinterpret_cast<SetFn>(dlsym(RTLD_DEFAULT, "omp_set_num_threads"));
  if (set_threads != nullptr) set_threads(n);
}

void Runtime::Loop() {
  LimitIntraOpThreadsOfThisThread();
  if (device_ >= 0) cudaSetDevice(device_);
  const bool coordinator = rank_ == 0;
  std::vector<struct pollfd> pfds;
  while (true) {
    pfds.clear();
    pfds.push_back({wake_fd_, POLLIN, 0});
    if (size_ > 1) {
      if (coordinator) {
        for (int r = 1; r < size_; ++r) pfds.push_back({cp_.fd(kChanNegotiate, r), POLLIN, 0});
      } else {
        pfds.push_back({cp_.fd(kChanNegotiate, 0), POLLIN, 0});
      }
    }
    int timeout_ms = 200;
    poll(pfds.data(), pfds.size(), timeout_ms);
    if (pfds[0].revents & POLLIN) {
      uint64_t junk;
      while (::read(wake_fd_, &junk, sizeof(junk)) > 0) {}
    }
    if (suspended_.load() && !shutdown_requested_.load()) continue;

    RequestList outgoing;
    std::vector<std::string> immediate;
    DrainLocalQueue(&outgoing, &immediate);
    // Operations that need no agreement run right away, in local order.
    for (const auto& name : immediate) {
      Response r;
      {
        std::lock_guard<std::mutex> g(table_mu_);
        r.type = static_cast<OpType>(table_[name].spec.type);
      }
      r.names = {name};
      std::lock_guard<std::mutex> ex(exec_mu_);
      ExecuteResponse(r);
    }
    if (shutdown_requested_.load() && !shutdown_sent_) {
      outgoing.shutdown = true;
      shutdown_sent_ = true;
    }
    bool fatal = false;
    if (size_ == 1) {
      if (outgoing.shutdown) break;
      continue;
    }
    if (coordinator) {
      if (!outgoing.requests.empty() || outgoing.shutdown) CoordinatorHandle(outgoing, 0);
      for (size_t i = 1; i < pfds.size(); ++i) {
        if (!(pfds[i].revents & (POLLIN | POLLHUP | POLLERR))) continue;
        const int from = static_cast<int>(i);  // pfds[i] belongs to rank i
        std::string bytes;
        Status s = cp_.RecvMsg(kChanNegotiate, from, &bytes, 30.0);
        RequestList list;
        if (!s.ok() || !RequestList::Parse(bytes, &list)) {
          BFLOG(WARNING, rank_) << "lost contact with rank " << from << ": " << s.reason() << "; shutting down";
          any_shutdown_ = true;
          continue;
        }
        CoordinatorHandle(list, from);
      }
      ResponseList responses = CoordinatorBuildResponses();
      if (any_shutdown_) responses.shutdown = true;
      if (!responses.responses.empty() || responses.shutdown) {
        const std::string bytes = responses.Serialize();
        for (int r = 1; r < size_; ++r) {
          Status s = cp_.SendMsg(kChanNegotiate, r, bytes);
          if (!s.ok()) BFLOG(DEBUG, rank_) << "could not send responses to rank " << r << ": " << s.reason();
        }
        ExecuteResponseList(responses);
        if (responses.shutdown) break;
      }
      CheckStalled();
    } else {
      if (!outgoing.requests.empty() || outgoing.shutdown) {
        Status s = cp_.SendMsg(kChanNegotiate, 0, outgoing.Serialize());
        if (!s.ok()) fatal = true;
      }
      if (!fatal && (pfds.back().revents & (POLLIN | POLLHUP | POLLERR))) {
        std::string bytes;
        Status s = cp_.RecvMsg(kChanNegotiate, 0, &bytes, 30.0);
        ResponseList list;
        if (!s.ok() || !ResponseList::Parse(bytes, &list)) {
          fatal = true;
        } else {
          ExecuteResponseList(list);
          if (list.shutdown) break;
        }
      }
      if (fatal) {
        BFLOG(DEBUG, rank_) << "lost contact with the coordinator; shutting down";
        break;
      }
    }
  }
  loop_exited_.store(true);
  FailAll(Status::Aborted(kShutDownError()));
}

void Runtime::FailAll(const Status& s) {
  std::vector<Entry> entries;
  {
    std::lock_guard<std::mutex> g(table_mu_);
    for (auto& kv : table_) entries.push_back(std::move(kv.second));
    table_.clear();
  }
  {
    std::lock_guard<std::mutex> g(queue_mu_);
    for (auto& e : queue_) entries.push_back(std::move(e));
    queue_.clear();
  }
  for (auto& e : entries) {
    timeline_.ActivityEnd(e.spec.name);
    if (e.ready_event) cudaEventDestroy(static_cast<cudaEvent_t>(e.ready_event));
    MarkDone(e.handle, s);
  }
}

// ----------------------------------------------------------------------------------------
// coordinator
// ----------------------------------------------------------------------------------------
void Runtime::CoordinatorHandle(const RequestList& list, int from_rank) {
  if (list.shutdown) any_shutdown_ = true;
  for (const auto& q : list.requests) {
    auto& pt = message_table_[q.name];
    if (pt.requests.empty()) {
      pt.requests.resize(size_);
      pt.seen.assign(size_, false);
      pt.first_seen = Clock::now();
    }
    if (pt.seen[from_rank]) continue;  // duplicate submission is rejected on the sender
    pt.requests[from_rank] = q;
    pt.seen[from_rank] = true;
    if (++pt.count == size_) ready_names_.push_back(q.name);
  }
}

Response Runtime::ConstructResponse(const std::string& name, PendingTensor& pt) {
  Response resp;
  resp.names = {name};
  const Request& first = pt.requests[0];
  resp.type = first.type;
  StrBuilder err;
  bool bad = false;
  for (int r = 1; r < size_ && !bad; ++r) {
    const Request& q = pt.requests[r];
    if (q.type != first.type) {
      err << "Mismatched operations: rank 0 requested " << OpTypeName(first.type) << " but rank " << r
          << " requested " << OpTypeName(q.type) << ".";
      bad = true;
    } else if (q.dtype != first.dtype) {
      err << "Mismatched data types: rank 0 has " << DataTypeName(first.dtype) << " but rank " << r << " has "
          << DataTypeName(q.dtype) << ".";
      bad = true;
    } else if ((q.device < 0) != (first.device < 0)) {
      err << "Mismatched devices: rank 0 holds the tensor on " << (first.device < 0 ? "CPU" : "GPU")
          << " but rank " << r << " on " << (q.device < 0 ? "CPU" : "GPU") << ".";
      bad = true;
    } else if (q.is_hierarchical != first.is_hierarchical) {
      err << "Mismatched hierarchical flag between rank 0 and rank " << r << ".";
      bad = true;
    }
  }
  const OpType t = first.type;
  if (!bad && (t == OpType::BROADCAST)) {
    for (int r = 1; r < size_ && !bad; ++r)
      if (pt.requests[r].root_rank != first.root_rank) {
        err << "Mismatched root ranks: rank 0 specified " << first.root_rank << " but rank " << r
            << " specified " << pt.requests[r].root_rank << ".";
        bad = true;
      }
  }
  if (!bad && (t == OpType::ALLREDUCE || t == OpType::BROADCAST || t == OpType::NEIGHBOR_ALLREDUCE ||
               t == OpType::WIN_CREATE)) {
    for (int r = 1; r < size_ && !bad; ++r)
      if (pt.requests[r].shape != first.shape) {
        err << "Mismatched tensor shapes between rank 0 and rank " << r << " for " << OpTypeName(t) << ".";
        bad = true;
      }
  }
  if (!bad && (t == OpType::ALLGATHER || t == OpType::NEIGHBOR_ALLGATHER)) {
    if (first.shape.empty()) {
      err << "Rank zero tried to gather a rank-zero tensor.";
      bad = true;
    }
    for (int r = 1; r < size_ && !bad; ++r) {
      const auto& sh = pt.requests[r].shape;
      if (sh.size() != first.shape.size()) {
        err << "Mismatched tensor ranks between rank 0 and rank " << r << " for " << OpTypeName(t) << ".";
        bad = true;
        break;
      }
      for (size_t d = 1; d < sh.size(); ++d)
        if (sh[d] != first.shape[d]) {
          err << "Mismatched trailing dimensions between rank 0 and rank " << r << " for " << OpTypeName(t) << ".";
          bad = true;
          break;
        }
    }
    if (!bad)
      for (int r = 0; r < size_; ++r) resp.first_dims.push_back(pt.requests[r].shape[0]);
  }
  for (int r = 0; r < size_; ++r) resp.devices.push_back(pt.requests[r].device);
  if (bad) {
    resp.type = OpType::ERROR;
    resp.error_message = err.str();
  }
  return resp;
}

ResponseList Runtime::CoordinatorBuildResponses() {
  ResponseList out;
  while (!ready_names_.empty()) {
    const std::string name = ready_names_.front();
    ready_names_.pop_front();
    auto it = message_table_.find(name);
    if (it == message_table_.end()) continue;
    PendingTensor pt = std::move(it->second);
    message_table_.erase(it);
    Response resp = ConstructResponse(name, pt);
    // Fusion: keep appending following ready tensors of the same kind while they fit.
    if (resp.type == OpType::ALLREDUCE || resp.type == OpType::NEIGHBOR_ALLREDUCE) {
      uint64_t total = pt.requests[0].nbytes;
      while (!ready_names_.empty()) {
        const std::string& next = ready_names_.front();
        auto nit = message_table_.find(next);
        if (nit == message_table_.end()) break;
        PendingTensor& np = nit->second;
        const Request& a = pt.requests[0];
        const Request& b = np.requests[0];
        bool same = b.type == a.type && b.dtype == a.dtype && (b.device < 0) == (a.device < 0) &&
                    b.is_hierarchical == a.is_hierarchical && total + b.nbytes <= static_cast<uint64_t>(fusion_threshold_);
        for (int r = 0; r < size_ && same; ++r) same = np.requests[r].neighbor_sig == pt.requests[r].neighbor_sig;
        if (!same) break;
        Response probe = ConstructResponse(next, np);
        if (probe.type == OpType::ERROR) break;
        total += b.nbytes;
        resp.names.push_back(next);
        message_table_.erase(nit);
        ready_names_.pop_front();
      }
    }
    out.responses.push_back(std::move(resp));
  }
  return out;
}

std::vector<std::string> Runtime::StalledTensors() {
  std::vector<std::string> out;
  for (auto& kv : message_table_) out.push_back(kv.first);
  return out;
}

void Runtime::CheckStalled() {
  auto now = Clock::now();
  if (std::chrono::duration<double>(now - last_stall_check_).count() < std::min(stall_warning_s_, 5.0)) return;
  last_stall_check_ = now;
  bool header = false;
  for (auto& kv : message_table_) {
    const double waited = std::chrono::duration<double>(now - kv.second.first_seen).count();
    if (waited < stall_warning_s_) continue;
    if (!header) {
      BFLOG(WARNING) << "One or more tensors were submitted to be reduced, gathered or broadcasted by a subset "
                        "of ranks and are waiting for the remainder for more than " << stall_warning_s_
                     << " seconds. This may indicate that different ranks are trying to submit different "
                        "tensors or that only a subset of ranks is submitting tensors, which will cause a deadlock.";
      header = true;
    }
    StrBuilder os;
    os << kv.first << " [missing ranks:";
    for (int r = 0; r < size_; ++r)
      if (!kv.second.seen[r]) os << " " << r;
    os << "]";
    BFLOG(WARNING) << os.str();
    kv.second.first_seen = now;  // warn again after another period
  }
}

// ----------------------------------------------------------------------------------------
// execution
// ----------------------------------------------------------------------------------------
void Runtime::ExecuteResponseList(const ResponseList& list) {
  for (const auto& r : list.responses) {
    std::lock_guard<std::mutex> ex(exec_mu_);   // callers on the fast path take the same lock
    ExecuteResponse(r);
  }
}

void Runtime::ExecuteResponse(const Response& resp) {
  std::vector<Entry> entries;
  {
    std::lock_guard<std::mutex> g(table_mu_);
    for (const auto& n : resp.names) {
      auto it = table_.find(n);
      if (it == table_.end()) continue;  // possible after a local failure
      entries.push_back(std::move(it->second));
      table_.erase(it);
    }
  }
  if (entries.empty()) return;
  stats_.responses.fetch_add(1);
  if (entries.size() > 1) stats_.fused_tensors.fetch_add(entries.size());
  if (resp.type == OpType::ERROR) {
    FinishEntries(entries, Status::PreconditionError(resp.error_message), nullptr);
    return;
  }
  ExecuteEntries(entries, resp);
}

void Runtime::FinishEntries(std::vector<Entry>& entries, const Status& s, void* done_event, void* span_start) {
  if (done_event == nullptr || !s.ok()) {
    if (done_event) cudaEventDestroy(static_cast<cudaEvent_t>(done_event));
    if (span_start) cudaEventDestroy(static_cast<cudaEvent_t>(span_start));
    for (auto& e : entries) {
      timeline_.ActivityEnd(e.spec.name);  // ENQUEUE_*
      if (e.ready_event) cudaEventDestroy(static_cast<cudaEvent_t>(e.ready_event));
      MarkDone(e.handle, s);
    }
    return;
  }
  if (tls_inline_) {
    // fast path: the caller's Wait/Poll finishes the handle, no thread hand-over
    InlineOp op;
    op.done_event = done_event;
    op.span_start = span_start;
    op.keep = std::make_shared<std::vector<Entry>>(std::move(entries));
    const int handle = (*op.keep)[0].handle;
    std::lock_guard<std::mutex> g(inline_mu_);
    inline_ops_[handle] = std::move(op);
    return;
  }
  // GPU work in flight: a finalizer thread waits for the completion event, converts a device
  // timeout into an error, and only then completes the handles.
  std::vector<int> handles;
  std::vector<std::string> names;
  std::vector<void*> ready;
  for (auto& e : entries) {
    handles.push_back(e.handle);
    names.push_back(e.spec.name);
    ready.push_back(e.ready_event);
  }
  // Keep the tensors alive until the kernels are done.
  auto keep = std::make_shared<std::vector<Entry>>(std::move(entries));
  const int device = device_;
  finalizers_.execute([this, handles, names, ready, keep, done_event, span_start, device] {
    cudaSetDevice(device);
    cudaError_t err = cudaEventSynchronize(static_cast<cudaEvent_t>(done_event));
    EmitDeviceSpan(names, span_start, err == cudaSuccess ? done_event : nullptr);
    cudaEventDestroy(static_cast<cudaEvent_t>(done_event));
    Status s = err == cudaSuccess ? Status::OK() : Status::UnknownError("CUDA error: " + CudaErrorString(err));
    if (s.ok()) s = GpuStatusToError();
    for (size_t i = 0; i < handles.size(); ++i) {
      timeline_.ActivityEnd(names[i]);
      if (ready[i]) cudaEventDestroy(static_cast<cudaEvent_t>(ready[i]));
      MarkDone(handles[i], s);
    }
    keep->clear();
  });
}

Status Runtime::TopoCheck(const OpSpec& spec) {
  // Every rank publishes who it sends to and who it receives from; the send matrix must
  // be the transpose of the receive matrix (reference: mpi_controller.cc:364-417).
  std::string mine(2 * size_, 0);
  for (int d : spec.dst_ranks)
    if (d >= 0 && d < size_) mine[d] = 1;
  for (int s : spec.src_ranks)
    if (s >= 0 && s < size_) mine[size_ + s] = 1;
  std::vector<std::string> all;
  Status s = cp_.AllgatherBytes(kChanData, mine, &all);
  if (!s.ok()) return s;
  for (int i = 0; i < size_; ++i)
    for (int j = 0; j < size_; ++j)
      if (all[i][j] != all[j][size_ + i])
        return Status::InvalidArgument(
            "Send and recv neighbors dont' match in neighbor communication: rank " + std::to_string(i) +
            (all[i][j] ? " sends to rank " : " does not send to rank ") + std::to_string(j) + " but rank " +
            std::to_string(j) + (all[j][size_ + i] ? " expects" : " does not expect") + " to receive from it.");
  return Status::OK();
}

void Runtime::ExecuteEntries(std::vector<Entry>& entries, const Response& resp) {
  const OpType type = static_cast<OpType>(entries[0].spec.type);
  for (auto& e : entries) timeline_.ActivityStart(e.spec.name, ProcActivity(type));
  auto end_proc = [&] { for (auto& e : entries) timeline_.ActivityEnd(e.spec.name); };

  if (type == OpType::BARRIER) {
    Status s = size_ > 1 ? cp_.Barrier(kChanData) : Status::OK();
    end_proc();
    FinishEntries(entries, s, nullptr);
    return;
  }
  if (type == OpType::WIN_CREATE || type == OpType::WIN_FREE || type == OpType::WIN_PUT ||
      type == OpType::WIN_GET || type == OpType::WIN_ACCUMULATE) {
    Status s = Status::OK();
    void* done = nullptr;
    for (auto& e : entries) {
      s = ExecuteWindowOp(e);
      if (!s.ok()) break;
    }
    const at::Tensor* t = entries[0].spec.input.has_value() ? &*entries[0].spec.input : nullptr;
    bool gpu = (t != nullptr && t->is_cuda());
    if (!gpu && (type == OpType::WIN_GET)) {
      at::Tensor v = windows_->SelfView(entries[0].spec.win_name);
      gpu = v.defined() && v.is_cuda();
    }
    if (s.ok() && gpu && comm_stream_ && (type == OpType::WIN_PUT || type == OpType::WIN_GET || type == OpType::WIN_ACCUMULATE)) {
      cudaEvent_t ev;
      cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
      cudaEventRecord(ev, static_cast<cudaStream_t>(comm_stream_));
      done = ev;
    }
    end_proc();
    FinishEntries(entries, s, done);
    return;
  }
  if (entries[0].spec.enable_topo_check && size_ > 1 &&
      (type == OpType::NEIGHBOR_ALLREDUCE || type == OpType::NEIGHBOR_ALLGATHER)) {
    Status s = TopoCheck(entries[0].spec);
    if (!s.ok()) {
      end_proc();
      FinishEntries(entries, s, nullptr);
      return;
    }
  }
  const at::Tensor* probe = entries[0].spec.input.has_value() ? &*entries[0].spec.input : &*entries[0].spec.output;
  Status s;
  void* done = nullptr;
  void* span_start = nullptr;
  if (probe->is_cuda()) {
    const bool traced = timeline_.Initialized() && comm_stream_ != nullptr;
    if (traced) {
      cudaEvent_t t0;
      cudaEventCreate(&t0);
      cudaEventRecord(t0, static_cast<cudaStream_t>(comm_stream_));
      span_start = t0;
    }
    s = ExecuteGpu(entries, resp);
    if (s.ok()) {
      cudaEvent_t ev;
      cudaEventCreateWithFlags(&ev, span_start ? cudaEventDefault : cudaEventDisableTiming);
      cudaEventRecord(ev, static_cast<cudaStream_t>(comm_stream_));
      done = ev;
    }
  } else {
    s = ExecuteCpu(entries, resp);
  }
  end_proc();
  FinishEntries(entries, s, done, span_start);
}

void Runtime::EmitDeviceSpan(const std::vector<std::string>& names, void* span_start, void* done_event) {
  if (span_start == nullptr) return;
  float ms = 0.f;
  if (done_event != nullptr && timeline_.Initialized() &&
      cudaEventElapsedTime(&ms, static_cast<cudaEvent_t>(span_start), static_cast<cudaEvent_t>(done_event)) == cudaSuccess) {
    const long end_us = timeline_.NowMicros();
    const long begin_us = end_us - static_cast<long>(ms * 1000.f);
    for (const auto& n : names) timeline_.CompleteSpan(n, "DEVICE", begin_us, end_us, /*lane=*/1000000 + device_);
  }
  cudaEventDestroy(static_cast<cudaEvent_t>(span_start));
}

Status Runtime::ExecuteWindowOp(Entry& e) {
  const OpType type = static_cast<OpType>(e.spec.type);
  const at::Tensor* t = e.spec.input.has_value() ? &*e.spec.input : nullptr;
  bool gpu = t != nullptr && t->is_cuda();
  if (type == OpType::WIN_GET) {
    at::Tensor v = windows_->SelfView(e.spec.win_name);
    gpu = v.defined() && v.is_cuda();
  }
  if (gpu) {
    cudaSetDevice(device_);
    if (!comm_stream_) {
      cudaStream_t st;
      int lo, hi;
      cudaDeviceGetStreamPriorityRange(&lo, &hi);
      cudaStreamCreateWithPriority(&st, cudaStreamNonBlocking, hi);
      comm_stream_ = st;
    }
    if (e.ready_event) cudaStreamWaitEvent(static_cast<cudaStream_t>(comm_stream_), static_cast<cudaEvent_t>(e.ready_event), 0);
  }
  switch (type) {
    case OpType::WIN_CREATE: return windows_->Create(e.spec, kChanData);
    case OpType::WIN_FREE: return windows_->Free(e.spec.win_name, kChanData);
    case OpType::WIN_PUT:
    case OpType::WIN_ACCUMULATE: return windows_->Put(e.spec, comm_stream_);
    case OpType::WIN_GET: return windows_->Get(e.spec, comm_stream_);
    default: return Status::InvalidArgument("not a window operation");
  }
}

// CPU data path: payloads travel over the TCP mesh, the combine is done with ATen.
Status Runtime::ExecuteCpu(std::vector<Entry>& entries, const Response& resp) {
  for (size_t idx = 0; idx < entries.size(); ++idx) {
    Entry& e = entries[idx];
    OpSpec& sp = e.spec;
    const OpType type = static_cast<OpType>(sp.type);
    timeline_.ActivityStart(sp.name, "COMMUNICATE");
    Status s = Status::OK();
    if (type == OpType::BROADCAST) {
      at::Tensor buf = *sp.output;
      if (rank_ == sp.root_rank) {
        if (sp.input.has_value() && sp.input->data_ptr() != buf.data_ptr()) buf.copy_(*sp.input);
        std::vector<SendSpec> sends;
        for (int r = 0; r < size_; ++r)
          if (r != rank_) sends.push_back({r, buf.data_ptr(), static_cast<size_t>(buf.nbytes())});
        s = cp_.Exchange(kChanData, sends, {});
      } else {
        s = cp_.Exchange(kChanData, {}, {{sp.root_rank, buf.data_ptr(), static_cast<size_t>(buf.nbytes())}});
      }
    } else if (type == OpType::ALLGATHER || type == OpType::NEIGHBOR_ALLGATHER) {
      const at::Tensor& in = *sp.input;
      at::Tensor& out = *sp.output;
      const int64_t row_bytes = in.numel() == 0 ? 0 : in.nbytes() / std::max<int64_t>(in.size(0), 1);
      std::vector<int64_t> dims(size_, in.size(0));  // negotiation skipped: equal sizes assumed
      if (resp.first_dims.size() >= (idx + 1) * static_cast<size_t>(size_))
        dims.assign(resp.first_dims.begin() + idx * size_, resp.first_dims.begin() + (idx + 1) * size_);
      std::vector<int> order;
      if (type == OpType::ALLGATHER) {
        for (int r = 0; r < size_; ++r) order.push_back(r);
      } else {
        order = sp.src_ranks;
      }
      int64_t total = 0;
      for (int r : order) total += dims[r];
      std::vector<int64_t> shape = in.sizes().vec();
      shape[0] = total;
      out.resize_(shape);
      std::vector<SendSpec> sends;
      std::vector<RecvSpec> recvs;
      const std::vector<int>& dsts = sp.dst_ranks;
      for (int d : dsts) sends.push_back({d, in.data_ptr(), static_cast<size_t>(in.nbytes())});
      char* base = static_cast<char*>(out.data_ptr());
      int64_t off = 0;
      for (int r : order) {
        const size_t nb = static_cast<size_t>(dims[r] * row_bytes);
        if (r == rank_) std::memcpy(base + off, in.data_ptr(), nb);
        else recvs.push_back({r, base + off, nb});
        off += nb;
      }
      s = cp_.Exchange(kChanData, sends, recvs);
    } else if (IsReduceOp(type)) {
      const at::Tensor& in = *sp.input;
      at::Tensor& out = *sp.output;
      // 16-bit floats are combined in fp32 (the reference does the same detour on CPU).
      const bool widen = in.scalar_type() == at::kHalf || in.scalar_type() == at::kBFloat16;
      std::vector<at::Tensor> scaled;   // per-destination scaled copies, kept alive during the exchange
      std::vector<SendSpec> sends;
      for (size_t i = 0; i < sp.dst_ranks.size(); ++i) {
        const void* ptr = in.data_ptr();
        if (sp.use_dst_weight && sp.dst_weights[i] != 1.0) {
          scaled.push_back(in.mul(sp.dst_weights[i]));
          ptr = scaled.back().data_ptr();
        }
        sends.push_back({sp.dst_ranks[i], ptr, static_cast<size_t>(in.nbytes())});
      }
      std::vector<at::Tensor> recv_bufs;
      std::vector<RecvSpec> recvs;
      for (int r : sp.src_ranks) {
        recv_bufs.push_back(at::empty_like(in));
        recvs.push_back({r, recv_bufs.back().data_ptr(), static_cast<size_t>(in.nbytes())});
      }
      s = cp_.Exchange(kChanData, sends, recvs);
      if (s.ok()) {
        timeline_.ActivityEnd(sp.name);
        timeline_.ActivityStart(sp.name, "COMPUTE_AVERAGE");
        const bool integral = at::isIntegralType(in.scalar_type(), /*includeBool=*/true);
        at::Tensor acc = widen ? in.to(at::kFloat) : in.clone();
        if (integral) {
          for (size_t j = 0; j < recv_bufs.size(); ++j) acc.add_(recv_bufs[j]);
        } else {
          if (sp.self_weight != 1.0) acc.mul_(sp.self_weight);
          for (size_t j = 0; j < recv_bufs.size(); ++j)
            acc.add_(widen ? recv_bufs[j].to(at::kFloat) : recv_bufs[j], sp.src_weights[j]);
          if (sp.post_scale != 1.0) acc.mul_(sp.post_scale);
        }
        out.resize_(in.sizes());
        out.copy_(acc);
      }
    } else {
      s = Status::InvalidArgument(std::string("unsupported CPU operation ") + OpTypeName(type));
    }
    timeline_.ActivityEnd(sp.name);
    if (!s.ok()) return s;
  }
  return Status::OK();
}

Status Runtime::GpuStatusToError() {
  if (windows_) {
    Status s = windows_->TakeDeviceError();       // a window mutex wait that ran out on the device
    if (!s.ok()) return s;
  }
  if (gpu_channel_) {
    Status s = gpu_channel_->StatusToError();
    if (!s.ok()) return s;
  }
  std::lock_guard<std::mutex> g(pair_mu_);
  for (auto& kv : pair_channels_) {
    Status s = kv.second.chan->StatusToError();
    if (!s.ok()) return s;
  }
  return Status::OK();
}

Status Runtime::EnsureCommStream() {
  cudaSetDevice(device_);
  if (!comm_stream_) {
    cudaStream_t st;
    int lo, hi;
    cudaDeviceGetStreamPriorityRange(&lo, &hi);
    BFB_CUDA_OK(cudaStreamCreateWithPriority(&st, cudaStreamNonBlocking, hi));
    comm_stream_ = st;
  }
  return Status::OK();
}

// The channel of a gossip pair lives in memory that only the two partners map; its versions advance with
// the gossips of this pair, whatever the other ranks do meanwhile.
Status Runtime::EnsurePairChannel(int peer, uint64_t need_bytes, Channel** chan) {
  Status s = EnsureCommStream();
  if (!s.ok()) return s;
  std::map<int, PairChannel>::iterator it;
  {
    std::lock_guard<std::mutex> g(pair_mu_);
    it = pair_channels_.find(peer);
  }
  const bool have = it != pair_channels_.end();
  if (have && need_bytes <= it->second.chan->half_bytes()) {
    *chan = it->second.chan.get();
    return Status::OK();
  }
  uint64_t half = have ? it->second.chan->half_bytes()
                       : static_cast<uint64_t>(EnvDouble("BLUEFOG_B200_PAIR_ARENA_BYTES", 8.0 * 1024 * 1024));
  while (half < need_bytes) half *= 2;
  if (have) {
    // both partners arrive here for the same gossip: finish the local work, then make sure the partner has
    // finished reading the old arena before it is released
    BFB_CUDA_OK(cudaStreamSynchronize(static_cast<cudaStream_t>(comm_stream_)));
    char mine = 1, theirs = 0;
    s = cp_.Exchange(kChanData, {{peer, &mine, 1}}, {{peer, &theirs, 1}});
    if (!s.ok()) return s;
  }
  std::shared_ptr<SymmBuffer> arena;
  s = AllocateIpcPair(&cp_, kChanData, peer, device_, half * 2, &arena);
  if (!s.ok()) return s;
  if (!have) {
    PairChannel pc;
    s = AllocateIpcPair(&cp_, kChanData, peer, device_, sizeof(ChannelCtrl), &pc.ctrl);
    if (!s.ok()) return s;
    pc.chan = std::make_unique<Channel>(pc.ctrl, arena, half);
    std::lock_guard<std::mutex> g(pair_mu_);
    it = pair_channels_.emplace(peer, std::move(pc)).first;
  } else {
    it->second.chan->ResetArena(arena, half);
  }
  *chan = it->second.chan.get();
  return Status::OK();
}

Status Runtime::ExecutePairGossipGpu(Entry& e) {
  OpSpec& sp = e.spec;
  if (sp.src_ranks.size() != 1) return Status::InvalidArgument("pair_gossip needs exactly one partner");
  const int peer = sp.src_ranks[0];
  const int elem = ToElem(sp.input->scalar_type());
  if (elem < 0 || elem == kI32 || elem == kI64) return Status::InvalidArgument("unsupported tensor type for pair_gossip");
  SegSpec sg;
  sg.in = sp.input->data_ptr();
  sg.nbytes = static_cast<uint64_t>(sp.input->nbytes());
  sg.numel = static_cast<uint64_t>(sp.input->numel());
  Channel* chan = nullptr;
  Status s = EnsurePairChannel(peer, std::max<uint64_t>(Channel::PaddedSize(sg.nbytes), 256), &chan);
  if (!s.ok()) return s;
  cudaStream_t stream = static_cast<cudaStream_t>(comm_stream_);
  if (e.ready_event) cudaStreamWaitEvent(stream, static_cast<cudaEvent_t>(e.ready_event), 0);
  timeline_.ActivityStart(sp.name, "COMMUNICATE");
  at::Tensor& out = *sp.output;
  if (out.sizes() != sp.input->sizes()) {
    c10::cuda::CUDAStreamGuard g(c10::cuda::getStreamFromExternal(stream, device_));
    out.resize_(sp.input->sizes());
  }
  sg.out = out.data_ptr();
  Round round;
  s = chan->Publish({sg}, nullptr, /*n_readers=*/1, stream, &round);
  if (s.ok())
    s = chan->PullCombine(round, {sg}, elem, sp.self_weight, {1 - chan->rank()}, {sp.src_weights.empty() ? 0.5 : sp.src_weights[0]},
                          false, 1.0, stream);
  timeline_.ActivityEnd(sp.name);
  return s;
}

Status Runtime::EnsureGpuChannel(uint64_t need_bytes) {
  Status cs = EnsureCommStream();
  if (!cs.ok()) return cs;
  const bool have = gpu_channel_ != nullptr;
  if (have && need_bytes <= gpu_channel_->half_bytes()) return Status::OK();
  // (Re)allocation is collective: payload sizes agree on every rank, so all ranks get here
  // for the same operation.
  uint64_t half = have ? gpu_channel_->half_bytes() : static_cast<uint64_t>(EnvDouble("BLUEFOG_B200_ARENA_BYTES", 32.0 * 1024 * 1024));
  while (half < need_bytes) half *= 2;
  if (have) {
    BFB_CUDA_OK(cudaStreamSynchronize(static_cast<cudaStream_t>(comm_stream_)));
    Status s = cp_.Barrier(kChanData);  // no peer still reads the old arena
    if (!s.ok()) return s;
  }
  std::shared_ptr<SymmBuffer> arena;
  Status s = AllocateIpc(&cp_, kChanData, device_, half * 2, &arena);
  if (!s.ok()) return s;
  if (!have) {
    s = AllocateIpc(&cp_, kChanData, device_, sizeof(ChannelCtrl), &gpu_ctrl_);
    if (!s.ok()) return s;
    gpu_channel_ = std::make_unique<Channel>(gpu_ctrl_, arena, half);
  } else {
    gpu_channel_->ResetArena(arena, half);
  }
  return Status::OK();
}

// GPU data path: publish into the symmetric arena, then pull from the peers' arenas.
Status Runtime::ExecuteGpu(std::vector<Entry>& entries, const Response& resp) {
  const OpType type = static_cast<OpType>(entries[0].spec.type);
  if (type == OpType::PAIR_GOSSIP) {
    Status ps = Status::OK();
    for (auto& e : entries) {
      ps = ExecutePairGossipGpu(e);
      if (!ps.ok()) break;
    }
    return ps;
  }
  OpSpec& first = entries[0].spec;
  std::vector<SegSpec> segs;
  for (auto& e : entries) {
    SegSpec sg;
    const at::Tensor* in = e.spec.input.has_value() ? &*e.spec.input : nullptr;
    sg.in = in ? in->data_ptr() : nullptr;
    sg.nbytes = in ? static_cast<uint64_t>(in->nbytes()) : 0;
    sg.numel = in ? static_cast<uint64_t>(in->numel()) : 0;
    if (type == OpType::BROADCAST) {
      at::Tensor& buf = *e.spec.output;
      sg.in = buf.data_ptr();
      sg.nbytes = static_cast<uint64_t>(buf.nbytes());
      sg.numel = static_cast<uint64_t>(buf.numel());
      if (rank_ != e.spec.root_rank) { sg.in = nullptr; }
    }
    segs.push_back(sg);
  }
  // Arena demand must be identical on all ranks: use the largest contribution for gathers.
  uint64_t need = 0;
  if (type == OpType::ALLGATHER || type == OpType::NEIGHBOR_ALLGATHER) {
    const at::Tensor& in = *first.input;
    const int64_t row_bytes = in.size(0) > 0 ? in.nbytes() / in.size(0) : 0;
    int64_t max_dim = in.size(0);
    for (int r = 0; r < size_ && !resp.first_dims.empty(); ++r) max_dim = std::max(max_dim, resp.first_dims[r]);
    need = Channel::PaddedSize(static_cast<uint64_t>(max_dim * row_bytes));
  } else if (type == OpType::BROADCAST) {
    for (auto& e : entries) need += Channel::PaddedSize(static_cast<uint64_t>(e.spec.output->nbytes()));
  } else {
    need = Channel::RequiredBytes(segs);
  }
  Status s = EnsureGpuChannel(std::max<uint64_t>(need, 256));
  if (!s.ok()) return s;
  cudaStream_t stream = static_cast<cudaStream_t>(comm_stream_);
  for (auto& e : entries)
    if (e.ready_event) cudaStreamWaitEvent(stream, static_cast<cudaEvent_t>(e.ready_event), 0);
  for (auto& e : entries) timeline_.ActivityStart(e.spec.name, "COMMUNICATE");
  auto end_act = [&] { for (auto& e : entries) timeline_.ActivityEnd(e.spec.name); };

  Round round;
  if (type == OpType::BROADCAST) {
    const bool root = rank_ == first.root_rank;
    std::vector<SegSpec> pub;
    if (root) pub = segs;
    s = gpu_channel_->Publish(pub, nullptr, root ? size_ - 1 : 0, stream, &round);
    if (s.ok() && !root) {
      // The root's round layout is the same deterministic packing of the same sizes.
      std::vector<Channel::CopySpec> copies;
      uint64_t off = 0;
      for (auto& e : entries) {
        const uint64_t nb = static_cast<uint64_t>(e.spec.output->nbytes());
        copies.push_back({first.root_rank, off, nb, e.spec.output->data_ptr()});
        off += Channel::PaddedSize(nb);
      }
      s = gpu_channel_->PullGather(round, {first.root_rank}, copies, stream);
    }
    end_act();
    return s;
  }
  if (type == OpType::ALLGATHER || type == OpType::NEIGHBOR_ALLGATHER) {
    const at::Tensor& in = *first.input;
    at::Tensor& out = *first.output;
    const int64_t row_bytes = in.size(0) > 0 ? in.nbytes() / in.size(0) : 0;
    std::vector<int64_t> dims(size_, in.size(0));
    if (!resp.first_dims.empty()) dims.assign(resp.first_dims.begin(), resp.first_dims.begin() + size_);
    std::vector<int> order;
    if (type == OpType::ALLGATHER) for (int r = 0; r < size_; ++r) order.push_back(r);
    else order = first.src_ranks;
    int64_t total = 0;
    for (int r : order) total += dims[r];
    std::vector<int64_t> shape = in.sizes().vec();
    shape[0] = total;
    {
      // Allocation happens on the scheduling thread: make the allocator use the comm stream.
      c10::cuda::CUDAStreamGuard g(c10::cuda::getStreamFromExternal(stream, device_));
      out.resize_(shape);
    }
    s = gpu_channel_->Publish(segs, nullptr, static_cast<int>(first.dst_ranks.size()), stream, &round);
    if (s.ok()) {
      std::vector<int> srcs;
      std::vector<Channel::CopySpec> copies;
      char* base = static_cast<char*>(out.data_ptr());
      int64_t off = 0;
      for (int r : order) {
        const uint64_t nb = static_cast<uint64_t>(dims[r] * row_bytes);
        if (r != rank_) srcs.push_back(r);
        if (nb > 0) copies.push_back({r, 0, nb, base + off});
        off += static_cast<int64_t>(nb);
      }
      s = gpu_channel_->PullGather(round, srcs, copies, stream);
    }
    end_act();
    return s;
  }
  if (IsReduceOp(type)) {
    const int elem = ToElem(first.input->scalar_type());
    if (elem < 0) {
      end_act();
      return Status::InvalidArgument("unsupported tensor type for a GPU reduction");
    }
    static const uint64_t two_shot_bytes = static_cast<uint64_t>(EnvDouble("BLUEFOG_B200_TWO_SHOT_BYTES", 1024.0 * 1024.0));
    if (type == OpType::ALLREDUCE && entries.size() == 1 && size_ > 2 &&
        static_cast<int>(first.src_ranks.size()) == size_ - 1 && segs[0].nbytes >= two_shot_bytes) {
      // Two-shot allreduce for large tensors: every rank reduces one slice out of all peers'
      // published tensors (reduce-scatter), publishes its reduced slice, and then gathers the
      // other slices.  Each rank moves 2*(N-1)/N of the tensor over NVLink instead of (N-1) times it.
      const bool integral = elem == kI32 || elem == kI64;
      const uint64_t esize = static_cast<uint64_t>(ElemSize(elem));
      const uint64_t numel = segs[0].numel;
      uint64_t per = (numel + size_ - 1) / size_;
      per = (per + 63) & ~uint64_t(63);
      auto start_of = [&](int r) { return std::min<uint64_t>(numel, static_cast<uint64_t>(r) * per); };
      auto len_of = [&](int r) { return std::min<uint64_t>(numel, start_of(r) + per) - start_of(r); };
      at::Tensor temp;
      {
        c10::cuda::CUDAStreamGuard g(c10::cuda::getStreamFromExternal(stream, device_));
        temp = at::empty({static_cast<int64_t>(per)}, first.input->options());
        at::Tensor& out = *first.output;
        if (out.sizes() != first.input->sizes()) out.resize_(first.input->sizes());
      }
      s = gpu_channel_->Publish(segs, nullptr, size_ - 1, stream, &round);
      if (s.ok()) {
        SegSpec mine;
        mine.out = temp.data_ptr();
        mine.numel = len_of(rank_);
        mine.elem_offset = start_of(rank_);
        std::vector<double> ones(first.src_ranks.size(), 1.0);
        s = gpu_channel_->PullCombine(round, {mine}, elem, 1.0, first.src_ranks, ones, false,
                                      integral ? 1.0 : first.post_scale, stream);
      }
      Round round2;
      if (s.ok()) {
        SegSpec pub;
        pub.in = temp.data_ptr();
        pub.nbytes = len_of(rank_) * esize;
        pub.numel = len_of(rank_);
        s = gpu_channel_->Publish({pub}, nullptr, size_ - 1, stream, &round2);
      }
      if (s.ok()) {
        std::vector<Channel::CopySpec> copies;
        char* base = static_cast<char*>(first.output->data_ptr());
        for (int r = 0; r < size_; ++r)
          if (len_of(r) > 0) copies.push_back({r, 0, len_of(r) * esize, base + start_of(r) * esize});
        s = gpu_channel_->PullGather(round2, first.src_ranks, copies, stream);
      }
      end_act();
      return s;
    }
    // The weights a sender attaches to its destinations always travel with the version (ones when it attaches
    // none) and the readers always apply them: whether destination weighting is "on" is the sender's decision
    // alone (any weight != 1), which a reader cannot know, and it may differ from rank to rank and step to step.
    std::vector<double> dstw(size_, 1.0);
    if (first.dst_weights.size() == first.dst_ranks.size())
      for (size_t i = 0; i < first.dst_ranks.size(); ++i) dstw[first.dst_ranks[i]] = first.dst_weights[i];
    // A tensor in registered symmetric memory is published in place: no copy into the arena, neighbors pull it from
    // where it is, and the operation ends with a wait for those neighbors (the tensor is the caller's to overwrite
    // again only when nobody reads it any more).  One tensor per operation, not the output of the same call.
    RegisteredLoc reg;
    const bool in_place = type == OpType::NEIGHBOR_ALLREDUCE && entries.size() == 1 && !first.is_hierarchical &&
                          first.output->data_ptr() != segs[0].in && FindRegistered(segs[0].in, segs[0].nbytes, &reg);
    s = gpu_channel_->Publish(segs, dstw.data(), static_cast<int>(first.dst_ranks.size()), stream, &round,
                              in_place ? reg.key : 0);
    if (s.ok()) {
      for (size_t i = 0; i < entries.size(); ++i) {
        at::Tensor& out = *entries[i].spec.output;
        if (out.sizes() != entries[i].spec.input->sizes()) {
          c10::cuda::CUDAStreamGuard g(c10::cuda::getStreamFromExternal(stream, device_));
          out.resize_(entries[i].spec.input->sizes());
        }
        segs[i].out = out.data_ptr();
      }
      const bool integral = elem == kI32 || elem == kI64;
      std::vector<double> w = first.src_weights;
      if (integral) w.assign(first.src_ranks.size(), 1.0);
      s = gpu_channel_->PullCombine(round, segs, elem, integral ? 1.0 : first.self_weight, first.src_ranks, w,
                                    /*use_dst_weight=*/!integral, integral ? 1.0 : first.post_scale, stream,
                                    in_place ? &reg : nullptr);
      if (s.ok() && in_place) s = gpu_channel_->WaitReaders(round, stream);
    }
    end_act();
    return s;
  }
  end_act();
  return Status::InvalidArgument(std::string("unsupported GPU operation ") + OpTypeName(type));
}

}  // namespace bfb
