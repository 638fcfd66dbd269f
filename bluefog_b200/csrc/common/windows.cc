#include "windows.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

#include <chrono>
#include <cstring>
#include <thread>

#include "../cuda/symm_mem.h"
#include "../cuda/window_kernels.h"
#include "logging.h"
#include "runtime.h"

namespace bfb {

namespace {

struct HostHeader {
  std::atomic<int> mutex[kMaxWorld];  // mutex[s]: guards slot of source s on this rank
};

constexpr size_t kHostHeaderBytes = (sizeof(HostHeader) + 255) & ~size_t(255);

int ToElemType(at::ScalarType t) {
  switch (t) {
    case at::kFloat: return kF32;
    case at::kDouble: return kF64;
    case at::kInt: return kI32;
    case at::kLong: return kI64;
    case at::kBFloat16: return kBF16;
    case at::kHalf: return kF16;
    default: return -1;
  }
}

}  // namespace

ShmSegment::~ShmSegment() {
  if (base) munmap(base, bytes);
  if (created) shm_unlink(name.c_str());
}

static Status OpenShm(const std::string& name, size_t bytes, bool create, std::shared_ptr<ShmSegment>* out) {
  auto seg = std::make_shared<ShmSegment>();
  seg->name = name;
  seg->bytes = bytes;
  int fd = -1;
  if (create) {
    shm_unlink(name.c_str());
    fd = shm_open(name.c_str(), O_CREAT | O_EXCL | O_RDWR, 0600);
    if (fd < 0) return Status::UnknownError("shm_open(create) failed for " + name + ": " + std::strerror(errno));
    seg->created = true;
    if (ftruncate(fd, static_cast<off_t>(bytes)) != 0) {
      ::close(fd);
      return Status::UnknownError("ftruncate failed for " + name + ": " + std::strerror(errno));
    }
  } else {
    fd = shm_open(name.c_str(), O_RDWR, 0600);
    if (fd < 0) return Status::UnknownError("shm_open failed for " + name + ": " + std::strerror(errno));
  }
  void* p = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  ::close(fd);
  if (p == MAP_FAILED) return Status::UnknownError("mmap failed for " + name + ": " + std::strerror(errno));
  seg->base = p;
  if (create) std::memset(p, 0, bytes);
  *out = seg;
  return Status::OK();
}

size_t Window::data_offset() const { return kHostHeaderBytes; }

unsigned char* Window::data_base(int rank) const {
  if (on_gpu) return static_cast<unsigned char*>(dev->ptrs[rank]);
  return static_cast<unsigned char*>(shm[rank]->base) + kHostHeaderBytes;
}
unsigned char* Window::self_ptr(int rank) const { return data_base(rank) + sizeof(WinHeader); }
unsigned char* Window::slot_ptr(int rank, int k) const {
  return data_base(rank) + sizeof(WinHeader) + padded * static_cast<size_t>(1 + k);
}
namespace {
const unsigned char kGuardPattern[Window::kGuardBytes] = {0xB1, 0xFE, 0x06, 0x20, 0xB2, 0x00, 0x5A, 0xA5,
                                                          0xC3, 0x3C, 0x96, 0x69, 0x0F, 0xF0, 0x77, 0x88};
}

void Window::WriteGuards(int rank) const {
  for (int k = -1; k < num_slots; ++k) {
    unsigned char* g = (k < 0 ? self_ptr(rank) : slot_ptr(rank, k)) + padded - kGuardBytes;
    if (on_gpu) cudaMemcpy(g, kGuardPattern, kGuardBytes, cudaMemcpyHostToDevice);
    else std::memcpy(g, kGuardPattern, kGuardBytes);
  }
}

int Window::DamagedGuards(int rank) const {
  int damaged = 0;
  for (int k = -1; k < num_slots; ++k) {
    const unsigned char* g = (k < 0 ? self_ptr(rank) : slot_ptr(rank, k)) + padded - kGuardBytes;
    unsigned char seen[kGuardBytes];
    if (on_gpu) {
      if (cudaMemcpy(seen, g, kGuardBytes, cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    } else {
      std::memcpy(seen, g, kGuardBytes);
    }
    if (std::memcmp(seen, kGuardPattern, kGuardBytes) != 0) ++damaged;
  }
  return damaged;
}

std::atomic<int>* Window::mutex_word(int owner, int source) const {
  return &static_cast<HostHeader*>(shm[owner]->base)->mutex[source];
}

WindowManager::~WindowManager() {
  std::lock_guard<std::mutex> g(mu_);
  windows_.clear();
}

std::shared_ptr<Window> WindowManager::Find(const std::string& name) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = windows_.find(name);
  return it == windows_.end() ? nullptr : it->second;
}

std::vector<std::string> WindowManager::Names() {
  std::lock_guard<std::mutex> g(mu_);
  std::vector<std::string> out;
  for (auto& kv : windows_) out.push_back(kv.first);
  return out;
}

size_t WindowManager::Count() {
  std::lock_guard<std::mutex> g(mu_);
  return windows_.size();
}

at::Tensor WindowManager::SelfView(const std::string& name) {
  auto w = Find(name);
  return w ? w->self_view : at::Tensor();
}

Status WindowManager::Create(const OpSpec& spec, int channel) {
  if (Find(spec.win_name)) return Status::InvalidArgument("Window " + spec.win_name + " already exists.");
  if (!spec.input.has_value()) return Status::InvalidArgument("win_create needs a tensor");
  const at::Tensor& t = *spec.input;
  auto w = std::make_shared<Window>();
  w->name = spec.win_name;
  w->id = next_id_++;
  w->on_gpu = t.is_cuda();
  w->device = t.is_cuda() ? t.get_device() : -1;
  w->dtype = t.scalar_type();
  w->shape = t.sizes().vec();
  w->numel = static_cast<uint64_t>(t.numel());
  w->nbytes = w->numel * t.element_size();
  w->padded = (w->nbytes + Window::kGuardBytes + 255) & ~uint64_t(255);     // room for the guard words behind the tensor
  w->num_slots = spec.num_slots;
  w->in_neighbors = spec.in_neighbors;
  if (static_cast<int>(w->in_neighbors.size()) > w->num_slots)
    return Status::InvalidArgument("win_create: more in-neighbors than slots");
  if (size_ > kMaxWorld) return Status::InvalidArgument("windows support at most 64 ranks");
  const size_t data_bytes = sizeof(WinHeader) + w->padded * static_cast<size_t>(1 + w->num_slots);
  const size_t shm_bytes = kHostHeaderBytes + (w->on_gpu ? 0 : data_bytes);
  w->shm.resize(size_);
  auto shm_name = [&](int r) {
    return "/bfb200_" + job_tag_ + "_" + std::to_string(w->id) + "_" + std::to_string(r);
  };
  Status s = OpenShm(shm_name(rank_), shm_bytes, /*create=*/true, &w->shm[rank_]);
  if (!s.ok()) return s;
  if (w->on_gpu) {
    s = AllocateIpc(cp_, channel, w->device, data_bytes + 512, &w->dev);     // + block counters and lock states
    if (!s.ok()) return s;
    w->block_counter = reinterpret_cast<unsigned int*>(static_cast<unsigned char*>(w->dev->local()) + data_bytes);
  }
  s = cp_->Barrier(channel);   // every rank has created its segment
  if (!s.ok()) return s;
  for (int r = 0; r < size_; ++r) {
    if (r == rank_) continue;
    s = OpenShm(shm_name(r), shm_bytes, /*create=*/false, &w->shm[r]);
    if (!s.ok()) return s;
  }
  // Initialise my own block: self = tensor; slots = tensor (or zero); p[self] = 1.
  auto opts = at::TensorOptions().dtype(w->dtype);
  std::shared_ptr<Window> keep = w;
  if (w->on_gpu) {
    c10::cuda::CUDAGuard guard(w->device);
    opts = opts.device(at::kCUDA, w->device);
    w->self_view = at::from_blob(w->self_ptr(rank_), w->shape, [keep](void*) {}, opts);
    w->self_view.copy_(t);
    for (int k = 0; k < w->num_slots; ++k) {
      at::Tensor slot = at::from_blob(w->slot_ptr(rank_, k), w->shape, opts);
      if (spec.zero_init) slot.zero_(); else slot.copy_(t);
    }
    double one = 1.0;
    WinHeader* h = reinterpret_cast<WinHeader*>(w->data_base(rank_));
    cudaMemcpy(&h->p[rank_], &one, sizeof(double), cudaMemcpyHostToDevice);
    w->WriteGuards(rank_);
    cudaDeviceSynchronize();
  } else {
    w->self_view = at::from_blob(w->self_ptr(rank_), w->shape, [keep](void*) {}, opts);
    w->self_view.copy_(t);
    for (int k = 0; k < w->num_slots; ++k) {
      at::Tensor slot = at::from_blob(w->slot_ptr(rank_, k), w->shape, opts);
      if (spec.zero_init) slot.zero_(); else slot.copy_(t);
    }
    reinterpret_cast<WinHeader*>(w->data_base(rank_))->p[rank_] = 1.0;
    w->WriteGuards(rank_);
  }
  s = cp_->Barrier(channel);   // every rank has mapped and initialised
  if (!s.ok()) return s;
  // The names can go now: every rank holds its mappings.
  shm_unlink(shm_name(rank_).c_str());
  w->shm[rank_]->created = false;
  std::lock_guard<std::mutex> g(mu_);
  windows_[w->name] = w;
  return Status::OK();
}

Status WindowManager::FreeOne(std::shared_ptr<Window> w) {
  // self_view's deleter holds the last reference to the memory if the user still uses the tensor.
  w->self_view = at::Tensor();
  return Status::OK();
}

Status WindowManager::Free(const std::string& name, int channel) {
  std::vector<std::shared_ptr<Window>> victims;
  {
    std::lock_guard<std::mutex> g(mu_);
    if (name.empty()) {
      for (auto& kv : windows_) victims.push_back(kv.second);
      windows_.clear();
    } else {
      auto it = windows_.find(name);
      if (it == windows_.end()) return Status::InvalidArgument("Window " + name + " does not exist.");
      victims.push_back(it->second);
      windows_.erase(it);
    }
  }
  for (auto& w : victims)
    if (w->on_gpu) {
      c10::cuda::CUDAGuard guard(w->device);
      cudaDeviceSynchronize();
    }
  // Nobody may unmap while a peer could still be writing into it.
  Status s = cp_->Barrier(channel);
  // every writer is done: the guard words behind the regions of my blocks must be as win_create left them
  std::string overrun;
  for (auto& w : victims) {
    c10::cuda::OptionalCUDAGuard guard;
    if (w->on_gpu) guard.set_index(w->device);
    const int damaged = w->DamagedGuards(rank_);
    if (damaged != 0)
      overrun += (overrun.empty() ? "" : ", ") + w->name + " (" + (damaged < 0 ? std::string("unreadable") : std::to_string(damaged)) + ")";
  }
  for (auto& w : victims) FreeOne(w);
  if (s.ok() && !overrun.empty())
    return Status::UnknownError("window memory was written past the end of a tensor on rank " + std::to_string(rank_) +
                                ": " + overrun + " region(s) with a damaged guard");
  return s;
}

static Status SpinLock(std::atomic<int>* word, double timeout_s) {
  auto t0 = std::chrono::steady_clock::now();
  for (;;) {
    int expected = 0;
    if (word->compare_exchange_strong(expected, 1, std::memory_order_acquire)) return Status::OK();
    std::this_thread::sleep_for(std::chrono::microseconds(5));
    if (std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > timeout_s)
      return Status::Aborted("timed out acquiring a window mutex");
  }
}

static WinLockState* LockStateOf(const Window& w, bool user) {
  return reinterpret_cast<WinLockState*>(reinterpret_cast<unsigned char*>(w.block_counter) + (user ? 192 : 128));
}

Status WindowManager::DeviceLock(Window& w, const std::vector<int>& ranks, bool for_self, bool acquire, bool user,
                                 void* stream) {
  if (ranks.empty()) return Status::OK();
  if (dev_status_host_ == nullptr) {
    if (cudaHostAlloc(&dev_status_host_, sizeof(CommStatus), cudaHostAllocMapped) != cudaSuccess)
      return Status::UnknownError("cannot allocate the pinned status block of the window mutexes");
    std::memset(dev_status_host_, 0, sizeof(CommStatus));
    if (cudaHostGetDevicePointer(&dev_status_dev_, dev_status_host_, 0) != cudaSuccess)
      return Status::UnknownError("cannot map the status block of the window mutexes");
  }
  std::vector<int> sorted(ranks);
  std::sort(sorted.begin(), sorted.end());                     // one global order of acquisition: no cycles
  sorted.erase(std::unique(sorted.begin(), sorted.end()), sorted.end());
  size_t begin = 0;
  while (begin < sorted.size()) {
    const size_t end = std::min(sorted.size(), begin + static_cast<size_t>(kMaxWinPeers));
    WinLockParams p;
    std::memset(&p, 0, sizeof(p));
    p.acquire = acquire ? 1 : 0;
    p.n = static_cast<int>(end - begin);
    p.my_rank = rank_;
    p.timeout_ns = static_cast<unsigned long long>(mutex_timeout_s * 1e9);
    for (size_t i = begin; i < end; ++i) {
      const int r = sorted[i];
      if (r < 0 || r >= size_) return Status::InvalidArgument("invalid rank in mutex list");
      p.header[i - begin] = reinterpret_cast<WinHeader*>(w.data_base(for_self ? rank_ : r));
      p.index[i - begin] = for_self ? r : rank_;
      p.owner[i - begin] = for_self ? rank_ : r;
    }
    p.state = LockStateOf(w, user);
    p.status = static_cast<CommStatus*>(dev_status_dev_);
    cudaError_t e = LaunchWinLock(p, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return Status::UnknownError("window mutex launch failed: " + CudaErrorString(e));
    begin = end;
  }
  return Status::OK();
}

Status WindowManager::TakeDeviceError() {
  if (dev_status_host_ == nullptr) return Status::OK();
  volatile CommStatus* st = static_cast<volatile CommStatus*>(dev_status_host_);
  if (st->error == kCommOk) return Status::OK();
  const unsigned peer = st->peer;
  st->error = kCommOk;
  return Status::Aborted("timed out acquiring a window mutex on rank " + std::to_string(peer) +
                         " (held for longer than BLUEFOG_B200_MUTEX_TIMEOUT_SECONDS); the operation was skipped");
}

Status WindowManager::MutexAcquire(const std::string& name, const std::vector<int>& ranks, bool for_self) {
  auto w = Find(name);
  if (!w) return Status::InvalidArgument("Window " + name + " does not exist.");
  if (w->on_gpu) {
    // an explicit win_mutex: the caller's host code runs under it, so wait until the kernel has taken the words
    c10::cuda::CUDAGuard guard(w->device);
    cudaStream_t st = c10::cuda::getCurrentCUDAStream(w->device).stream();
    Status s = DeviceLock(*w, ranks, for_self, /*acquire=*/true, /*user=*/true, st);
    if (!s.ok()) return s;
    if (cudaStreamSynchronize(st) != cudaSuccess) return Status::UnknownError("CUDA error while taking a window mutex");
    return TakeDeviceError();
  }
  for (int r : ranks) {
    if (r < 0 || r >= size_) return Status::InvalidArgument("invalid rank in mutex list");
    Status s = for_self ? SpinLock(w->mutex_word(rank_, r), mutex_timeout_s)
                        : SpinLock(w->mutex_word(r, rank_), mutex_timeout_s);
    if (!s.ok()) return s;
  }
  return Status::OK();
}

Status WindowManager::MutexRelease(const std::string& name, const std::vector<int>& ranks, bool for_self) {
  auto w = Find(name);
  if (!w) return Status::InvalidArgument("Window " + name + " does not exist.");
  if (w->on_gpu) {
    c10::cuda::CUDAGuard guard(w->device);
    cudaStream_t st = c10::cuda::getCurrentCUDAStream(w->device).stream();
    return DeviceLock(*w, ranks, for_self, /*acquire=*/false, /*user=*/true, st);
  }
  for (int r : ranks) {
    if (r < 0 || r >= size_) continue;
    auto* word = for_self ? w->mutex_word(rank_, r) : w->mutex_word(r, rank_);
    word->store(0, std::memory_order_release);
  }
  return Status::OK();
}

Status WindowManager::Versions(const std::string& name, std::vector<int64_t>* versions) {
  auto w = Find(name);
  if (!w) return Status::InvalidArgument("Window " + name + " does not exist.");
  versions->assign(size_, 0);
  WinHeader* h = reinterpret_cast<WinHeader*>(w->data_base(rank_));
  if (w->on_gpu) {
    std::vector<unsigned long long> tmp(kMaxWorld);
    c10::cuda::CUDAGuard guard(w->device);
    cudaMemcpy(tmp.data(), h->version, sizeof(unsigned long long) * kMaxWorld, cudaMemcpyDeviceToHost);
    for (int r = 0; r < size_; ++r) (*versions)[r] = static_cast<int64_t>(tmp[r]);
  } else {
    for (int r = 0; r < size_; ++r)
      (*versions)[r] = static_cast<int64_t>(reinterpret_cast<std::atomic<unsigned long long>*>(&h->version[r])->load());
  }
  return Status::OK();
}

Status WindowManager::GetAssociatedP(const std::string& name, double* p) {
  auto w = Find(name);
  if (!w) return Status::InvalidArgument("Window " + name + " does not exist.");
  WinHeader* h = reinterpret_cast<WinHeader*>(w->data_base(rank_));
  if (w->on_gpu) {
    c10::cuda::CUDAGuard guard(w->device);
    cudaMemcpy(p, &h->p[rank_], sizeof(double), cudaMemcpyDeviceToHost);
  } else {
    *p = *reinterpret_cast<volatile double*>(&h->p[rank_]);
  }
  return Status::OK();
}

Status WindowManager::SetAssociatedP(const std::string& name, double p) {
  auto w = Find(name);
  if (!w) return Status::InvalidArgument("Window " + name + " does not exist.");
  WinHeader* h = reinterpret_cast<WinHeader*>(w->data_base(rank_));
  if (w->on_gpu) {
    c10::cuda::CUDAGuard guard(w->device);
    cudaMemcpy(&h->p[rank_], &p, sizeof(double), cudaMemcpyHostToDevice);
  } else {
    *reinterpret_cast<volatile double*>(&h->p[rank_]) = p;
  }
  return Status::OK();
}

// put / accumulate -----------------------------------------------------------------------
Status WindowManager::Put(const OpSpec& spec, void* stream) {
  auto w = Find(spec.win_name);
  if (!w) return Status::InvalidArgument("Window " + spec.win_name + " does not exist.");
  if (!spec.input.has_value()) return Status::InvalidArgument("win_put needs a tensor");
  at::Tensor t = *spec.input;
  if (static_cast<uint64_t>(t.numel()) != w->numel || t.scalar_type() != w->dtype)
    return Status::InvalidArgument("win_put: tensor does not match the window " + spec.win_name);
  if (t.is_cuda() != w->on_gpu) return Status::InvalidArgument("win_put: tensor and window live on different device types");
  if (spec.dst_ranks.size() != spec.slot_index.size() || spec.dst_ranks.size() != spec.dst_weights.size())
    return Status::InvalidArgument("win_put: inconsistent destination lists");
  const bool with_p = with_p_.load();
  const bool host_mutex = spec.require_mutex && !w->on_gpu;
  const bool dev_mutex = spec.require_mutex && w->on_gpu;
  if (host_mutex) {
    Status s = MutexAcquire(spec.win_name, spec.dst_ranks, /*for_self=*/false);
    if (!s.ok()) return s;
  }
  Status result = Status::OK();
  if (w->on_gpu) {
    c10::cuda::CUDAGuard guard(w->device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dev_mutex) {
      Status s = DeviceLock(*w, spec.dst_ranks, /*for_self=*/false, /*acquire=*/true, /*user=*/false, st);
      if (!s.ok()) return s;
    }
    size_t begin = 0;
    const size_t n = spec.dst_ranks.size();
    do {
      const size_t end = std::min(n, begin + static_cast<size_t>(kMaxWinPeers));
      WinPutParams p;
      std::memset(&p, 0, sizeof(p));
      p.src = t.data_ptr();
      p.self_scale_target = (end == n) ? t.data_ptr() : nullptr;
      p.numel = w->numel;
      p.elem_type = ToElemType(w->dtype);
      if (p.elem_type < 0) { result = Status::InvalidArgument("win_put: unsupported dtype"); break; }
      p.accumulate = spec.accumulate ? 1 : 0;
      p.n_dst = static_cast<int>(end - begin);
      p.my_rank = rank_;
      p.with_p = with_p ? 1 : 0;
      p.self_weight = (end == n) ? spec.self_weight : 1.0;
      for (size_t i = begin; i < end; ++i) {
        const int d = spec.dst_ranks[i];
        p.weight[i - begin] = spec.dst_weights[i];
        p.dst_slot[i - begin] = w->slot_ptr(d, spec.slot_index[i]);
        p.dst_header[i - begin] = reinterpret_cast<WinHeader*>(w->data_base(d));
      }
      p.my_header = reinterpret_cast<WinHeader*>(w->data_base(rank_));
      p.block_counter = w->block_counter;
      p.lock_state = dev_mutex ? LockStateOf(*w, false) : nullptr;
      cudaError_t e = LaunchWinPut(p, st);
      if (e != cudaSuccess) { result = Status::UnknownError("win_put launch failed: " + CudaErrorString(e)); break; }
      begin = end;
    } while (begin < n);
    if (dev_mutex) DeviceLock(*w, spec.dst_ranks, /*for_self=*/false, /*acquire=*/false, /*user=*/false, st);
  } else {
    auto opts = at::TensorOptions().dtype(w->dtype);
    WinHeader* mine = reinterpret_cast<WinHeader*>(w->data_base(rank_));
    for (size_t i = 0; i < spec.dst_ranks.size(); ++i) {
      const int d = spec.dst_ranks[i];
      const double wgt = spec.dst_weights[i];
      at::Tensor slot = at::from_blob(w->slot_ptr(d, spec.slot_index[i]), t.sizes(), opts);
      if (spec.accumulate) slot.add_(t, wgt);
      else if (wgt == 1.0) slot.copy_(t);
      else slot.copy_(t.mul(wgt));
      WinHeader* h = reinterpret_cast<WinHeader*>(w->data_base(d));
      if (with_p) {
        auto* slot_p = reinterpret_cast<std::atomic<double>*>(&h->p[rank_]);
        const double v = *reinterpret_cast<volatile double*>(&mine->p[rank_]) * wgt;
        if (spec.accumulate) {
          double cur = slot_p->load();
          while (!slot_p->compare_exchange_weak(cur, cur + v)) {}
        } else {
          slot_p->store(v);
        }
      }
      reinterpret_cast<std::atomic<unsigned long long>*>(&h->version[rank_])->fetch_add(1, std::memory_order_release);
    }
    if (spec.self_weight != 1.0) t.mul_(spec.self_weight);
    if (with_p && spec.self_weight != 1.0) mine->p[rank_] *= spec.self_weight;
  }
  if (host_mutex) MutexRelease(spec.win_name, spec.dst_ranks, /*for_self=*/false);
  return result;
}

// get --------------------------------------------------------------------------------------
Status WindowManager::Get(const OpSpec& spec, void* stream) {
  auto w = Find(spec.win_name);
  if (!w) return Status::InvalidArgument("Window " + spec.win_name + " does not exist.");
  if (spec.src_ranks.size() != spec.slot_index.size() || spec.src_ranks.size() != spec.src_weights.size())
    return Status::InvalidArgument("win_get: inconsistent source lists");
  const bool host_mutex = spec.require_mutex && !w->on_gpu;
  const bool dev_mutex = spec.require_mutex && w->on_gpu;
  if (host_mutex) {
    Status s = MutexAcquire(spec.win_name, spec.src_ranks, /*for_self=*/false);
    if (!s.ok()) return s;
  }
  Status result = Status::OK();
  if (w->on_gpu) {
    c10::cuda::CUDAGuard guard(w->device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dev_mutex) {
      Status s = DeviceLock(*w, spec.src_ranks, /*for_self=*/false, /*acquire=*/true, /*user=*/false, st);
      if (!s.ok()) return s;
    }
    WinGetParams p;
    std::memset(&p, 0, sizeof(p));
    p.numel = w->numel;
    p.elem_type = ToElemType(w->dtype);
    p.n_src = static_cast<int>(spec.src_ranks.size());
    if (p.n_src > kMaxWinPeers || p.elem_type < 0) return Status::InvalidArgument("win_get: unsupported arguments");
    for (int i = 0; i < p.n_src; ++i) {
      p.weight[i] = spec.src_weights[i];
      p.src_self[i] = w->self_ptr(spec.src_ranks[i]);
      p.local_slot[i] = w->slot_ptr(rank_, spec.slot_index[i]);
      p.src_rank[i] = spec.src_ranks[i];
    }
    p.my_header = reinterpret_cast<WinHeader*>(w->data_base(rank_));
    p.block_counter = w->block_counter;
    p.lock_state = dev_mutex ? LockStateOf(*w, false) : nullptr;
    cudaError_t e = LaunchWinGet(p, st);
    if (e != cudaSuccess) result = Status::UnknownError("win_get launch failed: " + CudaErrorString(e));
    if (dev_mutex) DeviceLock(*w, spec.src_ranks, /*for_self=*/false, /*acquire=*/false, /*user=*/false, st);
  } else {
    auto opts = at::TensorOptions().dtype(w->dtype);
    WinHeader* mine = reinterpret_cast<WinHeader*>(w->data_base(rank_));
    for (size_t i = 0; i < spec.src_ranks.size(); ++i) {
      const int s = spec.src_ranks[i];
      at::Tensor remote = at::from_blob(w->self_ptr(s), w->shape, opts);
      at::Tensor slot = at::from_blob(w->slot_ptr(rank_, spec.slot_index[i]), w->shape, opts);
      if (spec.src_weights[i] == 1.0) slot.copy_(remote); else slot.copy_(remote.mul(spec.src_weights[i]));
      reinterpret_cast<std::atomic<unsigned long long>*>(&mine->version[s])->fetch_add(1);
    }
  }
  if (host_mutex) MutexRelease(spec.win_name, spec.src_ranks, /*for_self=*/false);
  return result;
}

// update -----------------------------------------------------------------------------------
Status WindowManager::Update(const std::string& name, at::Tensor out, double self_weight,
                             const std::vector<int>& src_ranks, const std::vector<double>& src_weights,
                             bool reset, bool require_mutex, void* stream) {
  auto w = Find(name);
  if (!w) return Status::InvalidArgument("Window " + name + " does not exist.");
  if (src_ranks.size() != src_weights.size()) return Status::InvalidArgument("win_update: inconsistent weights");
  std::vector<int> slots;
  for (int s : src_ranks) {
    auto it = std::find(w->in_neighbors.begin(), w->in_neighbors.end(), s);
    if (it == w->in_neighbors.end())
      return Status::InvalidArgument("win_update: rank " + std::to_string(s) + " is not an in-neighbor of window " + name);
    slots.push_back(static_cast<int>(it - w->in_neighbors.begin()));
  }
  const bool with_p = with_p_.load();
  const bool host_mutex = require_mutex && !w->on_gpu;
  // GPU windows: the read-and-clear of win_update(reset) is atomic against concurrent accumulates by itself; the
  // mutex is still taken when asked for, as three stream-ordered launches
  const bool dev_mutex = require_mutex && w->on_gpu;
  if (host_mutex) {
    Status s = MutexAcquire(name, src_ranks, /*for_self=*/true);
    if (!s.ok()) return s;
  }
  Status result = Status::OK();
  if (w->on_gpu) {
    c10::cuda::CUDAGuard guard(w->device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dev_mutex) {
      Status s = DeviceLock(*w, src_ranks, /*for_self=*/true, /*acquire=*/true, /*user=*/false, st);
      if (!s.ok()) return s;
    }
    WinUpdateParams p;
    std::memset(&p, 0, sizeof(p));
    p.self = w->self_ptr(rank_);
    p.out = out.defined() ? out.data_ptr() : p.self;
    p.numel = w->numel;
    p.elem_type = ToElemType(w->dtype);
    p.n_src = static_cast<int>(src_ranks.size());
    p.reset = reset ? 1 : 0;
    p.with_p = with_p ? 1 : 0;
    p.my_rank = rank_;
    p.self_weight = self_weight;
    if (p.n_src > kMaxWinPeers || p.elem_type < 0) return Status::InvalidArgument("win_update: unsupported arguments");
    for (int i = 0; i < p.n_src; ++i) {
      p.weight[i] = src_weights[i];
      p.slot[i] = w->slot_ptr(rank_, slots[i]);
      p.src_rank[i] = src_ranks[i];
    }
    p.my_header = reinterpret_cast<WinHeader*>(w->data_base(rank_));
    p.block_counter = w->block_counter + 8;
    p.lock_state = dev_mutex ? LockStateOf(*w, false) : nullptr;
    cudaError_t e = LaunchWinUpdate(p, st);
    if (e != cudaSuccess) result = Status::UnknownError("win_update launch failed: " + CudaErrorString(e));
    if (dev_mutex) DeviceLock(*w, src_ranks, /*for_self=*/true, /*acquire=*/false, /*user=*/false, st);
  } else {
    auto opts = at::TensorOptions().dtype(w->dtype);
    WinHeader* h = reinterpret_cast<WinHeader*>(w->data_base(rank_));
    at::Tensor self_t = w->self_view;
    at::Tensor acc = self_t.mul(self_weight);
    double pv = h->p[rank_] * self_weight;
    for (size_t i = 0; i < src_ranks.size(); ++i) {
      at::Tensor slot = at::from_blob(w->slot_ptr(rank_, slots[i]), w->shape, opts);
      acc.add_(slot, src_weights[i]);
      if (reset) slot.zero_();
      if (with_p) {
        pv += *reinterpret_cast<volatile double*>(&h->p[src_ranks[i]]) * src_weights[i];
        if (reset) h->p[src_ranks[i]] = 0.0;
      }
    }
    if (out.defined() && out.data_ptr() != self_t.data_ptr()) out.copy_(acc); else self_t.copy_(acc);
    if (with_p) h->p[rank_] = pv;
    for (int r = 0; r < size_; ++r)
      reinterpret_cast<std::atomic<unsigned long long>*>(&h->version[r])->store(0);
  }
  if (host_mutex) MutexRelease(name, src_ranks, /*for_self=*/true);
  return result;
}

}  // namespace bfb
