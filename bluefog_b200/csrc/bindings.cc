// Python bindings of the native runtime (module bluefog_b200._C).
// Role of bluefog/torch/mpi_ops.cc:572-690 and mpi_win_ops.cc:663-728 in the reference,
// with one generic enqueue entry instead of one symbol per tensor type.
#include <torch/extension.h>

#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <pybind11/stl.h>

#include <map>
#include <mutex>

#include "common/logging.h"
#include "common/runtime.h"
#include "common/windows.h"
#include "cuda/bn_kernels.h"
#include "cuda/bucket.h"
#include "cuda/combine_noalloc.h"
#include "cuda/ce_kernels.h"
#include "cuda/conv_tcgen05.h"
#include "cuda/embed_kernels.h"
#include "cuda/gemm_tcgen05.h"
#include "cuda/gpu_channel.h"
#include "cuda/ln_kernels.h"
#include "cuda/pool_kernels.h"
#include "cuda/stem_kernels.h"
#include "cuda/symm_mem.h"
#include "cuda/window_kernels.h"

namespace py = pybind11;
using namespace bfb;

namespace {

int ElemOf(const at::Tensor& t) {
  switch (t.scalar_type()) {
    case at::kFloat: return kF32;
    case at::kDouble: return kF64;
    case at::kHalf: return kF16;
    case at::kBFloat16: return kBF16;
    case at::kInt: return kI32;
    case at::kLong: return kI64;
    default: throw std::invalid_argument("unsupported tensor type for this kernel");
  }
}

cudaStream_t CurrentStream(int device) { return c10::cuda::getCurrentCUDAStream(device).stream(); }

void* PtrOrNull(const c10::optional<at::Tensor>& t) { return t.has_value() && t->defined() ? t->data_ptr() : nullptr; }

// ---- single-process world of channels: every "rank" is a set of buffers on one GPU ----------
class LocalWorld {
 public:
  LocalWorld(int world, int64_t half_bytes, int device) : world_(world), device_(device) {
    std::vector<std::shared_ptr<SymmBuffer>> ctrl, arena;
    ThrowIfError(AllocateLocal(world, device, sizeof(ChannelCtrl), &ctrl));
    ThrowIfError(AllocateLocal(world, device, static_cast<size_t>(half_bytes) * 2, &arena));
    for (int r = 0; r < world; ++r) chans_.push_back(std::make_unique<Channel>(ctrl[r], arena[r], half_bytes));
  }
  void set_timeout_ms(double ms) { for (auto& c : chans_) c->set_timeout_ms(ms); }
  int publish(int rank, std::vector<at::Tensor> tensors, c10::optional<std::vector<double>> dst_weight, int n_readers) {
    c10::cuda::CUDAGuard g(device_);
    std::vector<SegSpec> segs;
    for (auto& t : tensors) segs.push_back({t.data_ptr(), nullptr, static_cast<uint64_t>(t.nbytes()), static_cast<uint64_t>(t.numel())});
    Round round;
    ThrowIfError(chans_[rank]->Publish(segs, dst_weight ? dst_weight->data() : nullptr, n_readers, CurrentStream(device_), &round));
    rounds_.push_back(round);
    return static_cast<int>(rounds_.size()) - 1;
  }
  void combine(int rank, int round_id, std::vector<at::Tensor> outs, double self_w, std::vector<int> src_ranks,
               std::vector<double> src_w, bool use_dst_weight, double post_scale) {
    c10::cuda::CUDAGuard g(device_);
    std::vector<SegSpec> segs;
    for (auto& t : outs) segs.push_back({nullptr, t.data_ptr(), static_cast<uint64_t>(t.nbytes()), static_cast<uint64_t>(t.numel())});
    ThrowIfError(chans_[rank]->PullCombine(rounds_[round_id], segs, ElemOf(outs[0]), self_w, src_ranks, src_w,
                                           use_dst_weight, post_scale, CurrentStream(device_)));
  }
  void gather(int rank, int round_id, std::vector<int> src_ranks, std::vector<int> copy_src, std::vector<int64_t> arena_off,
              std::vector<at::Tensor> outs) {
    c10::cuda::CUDAGuard g(device_);
    std::vector<Channel::CopySpec> copies;
    for (size_t i = 0; i < outs.size(); ++i)
      copies.push_back({copy_src[i], static_cast<uint64_t>(arena_off[i]), static_cast<uint64_t>(outs[i].nbytes()), outs[i].data_ptr()});
    ThrowIfError(chans_[rank]->PullGather(rounds_[round_id], src_ranks, copies, CurrentStream(device_)));
  }
  // Registered tensors: one buffer of `nbytes` per rank, every rank's registry knows all of them.  Returns the
  // ranks' buffers as uint8 tensors.
  std::vector<at::Tensor> alloc_symmetric(int64_t nbytes) {
    c10::cuda::CUDAGuard g(device_);
    std::vector<std::shared_ptr<SymmBuffer>> bufs;
    ThrowIfError(AllocateLocal(world_, device_, static_cast<size_t>((nbytes + 255) & ~int64_t(255)), &bufs));
    if (regs_.empty()) regs_.resize(world_);
    std::vector<at::Tensor> out;
    for (int r = 0; r < world_; ++r) {
      regs_[r].Add(bufs[r]);
      std::shared_ptr<SymmBuffer> keep = bufs[r];
      out.push_back(at::from_blob(bufs[r]->local(), {nbytes}, [keep](void*) {},
                                  at::TensorOptions().dtype(at::kByte).device(at::kCUDA, device_)));
    }
    return out;
  }
  // Publishes `x` (a tensor inside rank's registered buffer) in place; a tensor elsewhere is copied into the arena.
  int publish_in_place(int rank, at::Tensor x, c10::optional<std::vector<double>> dst_weight, int n_readers) {
    c10::cuda::CUDAGuard g(device_);
    RegisteredLoc reg;
    const bool found = !regs_.empty() && regs_[rank].Find(x.data_ptr(), static_cast<uint64_t>(x.nbytes()), &reg);
    std::vector<SegSpec> segs{{x.data_ptr(), nullptr, static_cast<uint64_t>(x.nbytes()), static_cast<uint64_t>(x.numel())}};
    Round round;
    ThrowIfError(chans_[rank]->Publish(segs, dst_weight ? dst_weight->data() : nullptr, n_readers, CurrentStream(device_), &round,
                                       found ? reg.key : 0));
    rounds_.push_back(round);
    return static_cast<int>(rounds_.size()) - 1;
  }
  // The pull of a rank that published `x` with publish_in_place.
  void combine_in_place(int rank, int round_id, at::Tensor x, at::Tensor out, double self_w, std::vector<int> src_ranks,
                        std::vector<double> src_w, bool use_dst_weight, double post_scale) {
    c10::cuda::CUDAGuard g(device_);
    RegisteredLoc reg;
    const bool found = !regs_.empty() && regs_[rank].Find(x.data_ptr(), static_cast<uint64_t>(x.nbytes()), &reg);
    std::vector<SegSpec> segs{{nullptr, out.data_ptr(), static_cast<uint64_t>(out.nbytes()), static_cast<uint64_t>(out.numel())}};
    ThrowIfError(chans_[rank]->PullCombine(rounds_[round_id], segs, ElemOf(out), self_w, src_ranks, src_w, use_dst_weight,
                                           post_scale, CurrentStream(device_), found ? &reg : nullptr));
  }
  // Launch only after the pulls of every reader have been launched: ranks of this world share one GPU.
  void wait_readers(int rank, int round_id) {
    c10::cuda::CUDAGuard g(device_);
    ThrowIfError(chans_[rank]->WaitReaders(rounds_[round_id], CurrentStream(device_)));
  }
  // Rounds published by different ranks in the same position share version and layout.
  std::vector<int64_t> round_offsets(int round_id) {
    return std::vector<int64_t>(rounds_[round_id].offsets.begin(), rounds_[round_id].offsets.end());
  }
  py::tuple status(int rank) {
    CommStatus s = chans_[rank]->ReadStatus();
    return py::make_tuple(s.error, s.peer, s.want, s.seen);
  }
  void clear_status(int rank) { chans_[rank]->ClearStatus(); }

 private:
  int world_, device_;
  std::vector<std::unique_ptr<Channel>> chans_;
  std::vector<Round> rounds_;
  std::vector<SymmRegistry> regs_;       // per rank
};

std::unique_ptr<Channel> MakeIpcChannel(size_t half_bytes) {
  Runtime& rt = Runtime::Get();
  if (!rt.initialized()) throw std::invalid_argument(kNotInitializedError());
  std::shared_ptr<SymmBuffer> ctrl, arena;
  ThrowIfError(AllocateIpc(&rt.control_plane(), kChanUser, rt.device(), sizeof(ChannelCtrl), &ctrl));
  ThrowIfError(AllocateIpc(&rt.control_plane(), kChanUser, rt.device(), half_bytes * 2, &arena));
  rt.KeepUntilShutdown(ctrl);    // peers' kernels read these: they stay mapped until the barrier in Shutdown
  rt.KeepUntilShutdown(arena);
  return std::make_unique<Channel>(ctrl, arena, half_bytes);
}

int PubElem(const std::string& dtype) {
  if (dtype == "float32") return kF32;
  if (dtype == "bfloat16") return kBF16;
  throw std::invalid_argument("published dtype must be float32 or bfloat16");
}

// One device word per process that the GEMM kernel sets when a bounded wait expired.
at::Tensor& GemmStatusWord(const at::Tensor& like) {
  static at::Tensor status;
  if (!status.defined()) status = at::zeros({1}, like.options().dtype(at::kInt));
  return status;
}

// ---- single-process world of windows: every "rank" is a block [WinHeader | self | one slot per source rank] on
// one GPU; the per-rank kernels are launched one after the other (tests and micro-benchmarks of the window kernels)
class LocalWindows {
 public:
  LocalWindows(int world, int64_t numel, at::ScalarType dtype, int device)
      : world_(world), numel_(numel), dtype_(dtype), device_(device) {
    TORCH_CHECK(world >= 1 && world <= kMaxWorld && numel > 0, "LocalWindows: bad geometry");
    c10::cuda::CUDAGuard g(device);
    const int64_t esize = static_cast<int64_t>(c10::elementSize(dtype));
    region_ = (numel * esize + 255) / 256 * 256;
    auto opts = at::TensorOptions().device(at::kCUDA, device).dtype(at::kByte);
    for (int r = 0; r < world; ++r) {
      mem_.push_back(at::zeros({static_cast<int64_t>(sizeof(WinHeader)) + region_ * (world + 1)}, opts));
      scratch_.push_back(at::zeros({256}, opts));
    }
    for (int r = 0; r < world; ++r) header(r);   // touch
    std::vector<double> one(1, 1.0);
    for (int r = 0; r < world; ++r) set_p(r, r, 1.0);
  }
  WinHeader* header(int r) { return reinterpret_cast<WinHeader*>(mem_[r].data_ptr()); }
  unsigned char* self_ptr(int r) { return static_cast<unsigned char*>(mem_[r].data_ptr()) + sizeof(WinHeader); }
  unsigned char* slot_ptr(int r, int src) { return self_ptr(r) + region_ * (1 + src); }
  unsigned int* counter(int r) { return reinterpret_cast<unsigned int*>(scratch_[r].data_ptr()); }
  WinLockState* lock_state_ptr(int r) { return reinterpret_cast<WinLockState*>(static_cast<unsigned char*>(scratch_[r].data_ptr()) + 64); }
  at::Tensor view(unsigned char* p) {
    return at::from_blob(p, {numel_}, at::TensorOptions().device(at::kCUDA, device_).dtype(dtype_));
  }
  at::Tensor self_tensor(int r) { return view(self_ptr(r)); }
  at::Tensor slot_tensor(int r, int src) { return view(slot_ptr(r, src)); }
  void put(int rank, at::Tensor src, std::vector<int> dst, std::vector<double> w, double self_weight, bool accumulate,
           bool with_p, bool guarded) {
    c10::cuda::CUDAGuard g(device_);
    WinPutParams p;
    std::memset(&p, 0, sizeof(p));
    p.src = src.data_ptr();
    p.self_scale_target = src.data_ptr();
    p.numel = static_cast<unsigned long long>(numel_);
    p.elem_type = ElemOf(src);
    p.accumulate = accumulate ? 1 : 0;
    p.n_dst = static_cast<int>(dst.size());
    p.my_rank = rank;
    p.with_p = with_p ? 1 : 0;
    p.self_weight = self_weight;
    for (size_t i = 0; i < dst.size(); ++i) {
      p.weight[i] = w[i];
      p.dst_slot[i] = slot_ptr(dst[i], rank);
      p.dst_header[i] = header(dst[i]);
    }
    p.my_header = header(rank);
    p.block_counter = counter(rank);
    p.lock_state = guarded ? lock_state_ptr(rank) : nullptr;
    cudaError_t e = LaunchWinPut(p, CurrentStream(device_));
    TORCH_CHECK(e == cudaSuccess, "win_put launch failed: ", cudaGetErrorString(e));
  }
  void get(int rank, std::vector<int> srcs, std::vector<double> w) {
    c10::cuda::CUDAGuard g(device_);
    WinGetParams p;
    std::memset(&p, 0, sizeof(p));
    p.numel = static_cast<unsigned long long>(numel_);
    p.elem_type = ElemOf(self_tensor(rank));
    p.n_src = static_cast<int>(srcs.size());
    for (size_t i = 0; i < srcs.size(); ++i) {
      p.weight[i] = w[i];
      p.src_self[i] = self_ptr(srcs[i]);
      p.local_slot[i] = slot_ptr(rank, srcs[i]);
      p.src_rank[i] = srcs[i];
    }
    p.my_header = header(rank);
    p.block_counter = counter(rank);
    cudaError_t e = LaunchWinGet(p, CurrentStream(device_));
    TORCH_CHECK(e == cudaSuccess, "win_get launch failed: ", cudaGetErrorString(e));
  }
  void update(int rank, std::vector<int> srcs, std::vector<double> w, double self_weight, bool reset, bool with_p) {
    c10::cuda::CUDAGuard g(device_);
    WinUpdateParams p;
    std::memset(&p, 0, sizeof(p));
    p.self = self_ptr(rank);
    p.out = self_ptr(rank);
    p.numel = static_cast<unsigned long long>(numel_);
    p.elem_type = ElemOf(self_tensor(rank));
    p.n_src = static_cast<int>(srcs.size());
    p.reset = reset ? 1 : 0;
    p.with_p = with_p ? 1 : 0;
    p.my_rank = rank;
    p.self_weight = self_weight;
    for (size_t i = 0; i < srcs.size(); ++i) {
      p.weight[i] = w[i];
      p.slot[i] = slot_ptr(rank, srcs[i]);
      p.src_rank[i] = srcs[i];
    }
    p.my_header = header(rank);
    p.block_counter = counter(rank);
    cudaError_t e = LaunchWinUpdate(p, CurrentStream(device_));
    TORCH_CHECK(e == cudaSuccess, "win_update launch failed: ", cudaGetErrorString(e));
  }
  // takes or frees lock[index[i]] on rank owners[i], as `rank`
  void lock(int rank, std::vector<int> owners, std::vector<int> index, bool acquire, double timeout_ms) {
    c10::cuda::CUDAGuard g(device_);
    WinLockParams p;
    std::memset(&p, 0, sizeof(p));
    p.acquire = acquire ? 1 : 0;
    p.n = static_cast<int>(owners.size());
    p.my_rank = rank;
    p.timeout_ns = static_cast<unsigned long long>(timeout_ms * 1e6);
    for (size_t i = 0; i < owners.size(); ++i) {
      p.header[i] = header(owners[i]);
      p.index[i] = index[i];
      p.owner[i] = owners[i];
    }
    p.state = lock_state_ptr(rank);
    cudaError_t e = LaunchWinLock(p, CurrentStream(device_));
    TORCH_CHECK(e == cudaSuccess, "win_lock launch failed: ", cudaGetErrorString(e));
  }
  std::vector<int64_t> lock_state(int rank) {
    at::Tensor host = scratch_[rank].cpu();
    const WinLockState* s = reinterpret_cast<const WinLockState*>(static_cast<const unsigned char*>(host.data_ptr()) + 64);
    return {static_cast<int64_t>(s->failed), static_cast<int64_t>(s->failed_rank), static_cast<int64_t>(s->held)};
  }
  std::vector<int64_t> versions(int rank) {
    at::Tensor host = mem_[rank].slice(0, 0, sizeof(WinHeader)).cpu();
    const WinHeader* h = reinterpret_cast<const WinHeader*>(host.data_ptr());
    std::vector<int64_t> out(world_);
    for (int r = 0; r < world_; ++r) out[r] = static_cast<int64_t>(h->version[r]);
    return out;
  }
  std::vector<double> p_values(int rank) {
    at::Tensor host = mem_[rank].slice(0, 0, sizeof(WinHeader)).cpu();
    const WinHeader* h = reinterpret_cast<const WinHeader*>(host.data_ptr());
    return std::vector<double>(h->p, h->p + world_);
  }
  void set_p(int rank, int index, double v) {
    c10::cuda::CUDAGuard g(device_);
    cudaMemcpy(&header(rank)->p[index], &v, sizeof(double), cudaMemcpyHostToDevice);
  }

 private:
  int world_;
  int64_t numel_;
  at::ScalarType dtype_;
  int device_;
  int64_t region_ = 0;
  std::vector<at::Tensor> mem_, scratch_;
};

// channels_last [N, C, H, W] -> the [n, h, w, c] view the convolution kernels address
ConvView MakeConvView(const at::Tensor& t, bool stem_view) {
  const int N = static_cast<int>(t.size(0)), C = static_cast<int>(t.size(1)), H = static_cast<int>(t.size(2)),
            W = static_cast<int>(t.size(3));
  if (stem_view) {
    TORCH_CHECK(C == 16 && W > 3, "the stem view needs a 16-channel image wider than 3 pixels");
    return ConvView{t.data_ptr(), N, H, W - 3, 64, 16, (long long)W * 16, (long long)H * W * 16};
  }
  return ConvView{t.data_ptr(), N, H, W, C, C, (long long)W * C, (long long)H * W * C};
}

// Zero-initialised scratch of the split-K filter gradients, one per (device, stream): fp32 partial sums and
// tile counters.  The kernel leaves both zero, so they are cleared only when they are (re)allocated.
struct WgradScratch {
  at::Tensor sums, counters;
};
WgradScratch& WgradScratchFor(const at::Tensor& like, cudaStream_t stream, int64_t floats) {
  static std::mutex mu;
  static std::map<std::pair<int, cudaStream_t>, WgradScratch> all;
  std::lock_guard<std::mutex> lk(mu);
  WgradScratch& sc = all[{like.get_device(), stream}];
  if (!sc.sums.defined() || sc.sums.numel() < floats) {
    const int64_t want = std::max<int64_t>(floats, int64_t(1) << 23);
    sc.sums = at::zeros({want}, like.options().dtype(at::kFloat));
  }
  if (!sc.counters.defined()) sc.counters = at::zeros({4096}, like.options().dtype(at::kInt));
  return sc;
}

struct PyBucketArgs : BucketStepArgs {
  c10::optional<at::Tensor> t_master, t_grad, t_state1, t_state2, t_state3, t_shadow;
  // int64 CUDA tensors: per-parameter gradient addresses, first element and length of each parameter
  c10::optional<at::Tensor> t_grad_ptrs, t_seg_start, t_seg_numel;
  bool grad_table_bf16 = false;
};

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "bluefog_b200 native runtime";

  py::class_<OpSpec>(m, "OpSpec")
      .def(py::init<>())
      .def_readwrite("type", &OpSpec::type)
      .def_readwrite("name", &OpSpec::name)
      .def_readwrite("input", &OpSpec::input)
      .def_readwrite("output", &OpSpec::output)
      .def_readwrite("root_rank", &OpSpec::root_rank)
      .def_readwrite("self_weight", &OpSpec::self_weight)
      .def_readwrite("post_scale", &OpSpec::post_scale)
      .def_readwrite("src_ranks", &OpSpec::src_ranks)
      .def_readwrite("src_weights", &OpSpec::src_weights)
      .def_readwrite("dst_ranks", &OpSpec::dst_ranks)
      .def_readwrite("dst_weights", &OpSpec::dst_weights)
      .def_readwrite("use_dst_weight", &OpSpec::use_dst_weight)
      .def_readwrite("enable_topo_check", &OpSpec::enable_topo_check)
      .def_readwrite("is_hierarchical", &OpSpec::is_hierarchical)
      .def_readwrite("negotiate", &OpSpec::negotiate)
      .def_readwrite("win_name", &OpSpec::win_name)
      .def_readwrite("require_mutex", &OpSpec::require_mutex)
      .def_readwrite("zero_init", &OpSpec::zero_init)
      .def_readwrite("accumulate", &OpSpec::accumulate)
      .def_readwrite("slot_index", &OpSpec::slot_index)
      .def_readwrite("num_slots", &OpSpec::num_slots)
      .def_readwrite("in_neighbors", &OpSpec::in_neighbors);

  // ---- lifecycle ---------------------------------------------------------------------------
  m.def("listen", [](const std::string& addr) {
    int port = 0;
    ThrowIfError(Runtime::Get().Listen(addr, &port));
    return port;
  });
  m.def("init", [](int rank, int size, int local_rank, int local_size, std::vector<std::string> endpoints, int device) {
    py::gil_scoped_release nogil;
    ThrowIfError(Runtime::Get().Init(rank, size, local_rank, local_size, endpoints, device));
  });
  m.def("shutdown", [] {
    py::gil_scoped_release nogil;
    Runtime::Get().Shutdown();
  });
  m.def("is_initialized", [] { return Runtime::Get().initialized(); });
  m.def("rank", [] { return Runtime::Get().rank(); });
  m.def("size", [] { return Runtime::Get().size(); });
  m.def("local_rank", [] { return Runtime::Get().local_rank(); });
  m.def("local_size", [] { return Runtime::Get().local_size(); });
  // Collective: `nbytes` of this rank's device memory, mapped into every rank (see Runtime::SymmetricAlloc); a uint8
  // tensor that Python views as the dtype and shape it wants.
  m.def("symmetric_alloc", [](int64_t nbytes) {
    Runtime& rt = Runtime::Get();
    std::shared_ptr<SymmBuffer> buf;
    {
      py::gil_scoped_release nogil;
      ThrowIfError(rt.SymmetricAlloc(static_cast<size_t>(nbytes), &buf));
    }
    std::shared_ptr<SymmBuffer> keep = buf;
    return at::from_blob(buf->local(), {nbytes}, [keep](void*) {},
                         at::TensorOptions().dtype(at::kByte).device(at::kCUDA, rt.device()));
  });
  m.def("is_symmetric", [](at::Tensor t) {
    RegisteredLoc loc;
    return t.is_cuda() && Runtime::Get().FindRegistered(t.data_ptr(), static_cast<uint64_t>(t.nbytes()), &loc);
  });
  // Counters of this rank's runtime since init, plus the kernel launches of this library (see Runtime::StatsSnapshot).
  m.def("runtime_stats", [] {
    py::dict d;
    for (const auto& kv : Runtime::Get().StatsSnapshot()) d[py::str(kv.first)] = kv.second;
    d["kernel_launches"] = KernelLaunchCount();
    return d;
  });
  m.def("set_skip_negotiate_stage", [](bool v) { Runtime::Get().set_skip_negotiate(v); });
  m.def("get_skip_negotiate_stage", [] { return Runtime::Get().skip_negotiate(); });
  m.def("suspend", [] { Runtime::Get().Suspend(); });
  m.def("resume", [] { Runtime::Get().Resume(); });
  m.def("fusion_threshold", [] { return Runtime::Get().fusion_threshold(); });
  m.def("set_fusion_threshold", [](int64_t v) { Runtime::Get().set_fusion_threshold(v); });
  m.def("set_stall_warning_seconds", [](double s) { Runtime::Get().set_stall_warning_seconds(s); });
  m.def("kernel_launch_count", [] { return KernelLaunchCount(); });
  // control words of the allocation-free combine's static scratch on the current device:
  // (block_counter, calls_done, [done of each source])
  m.def("noalloc_scratch_words", [](int n_src) {
    unsigned int block_counter = 0;
    unsigned long long calls_done = 0;
    std::vector<unsigned long long> done(static_cast<size_t>(n_src > 0 ? n_src : 0));
    cudaError_t e = bfb::NoAllocScratchRead(n_src, &block_counter, &calls_done, done.data());
    if (e != cudaSuccess) throw std::runtime_error(std::string("noalloc_scratch_words: ") + cudaGetErrorString(e));
    return py::make_tuple(block_counter, calls_done, done);
  });

  // ---- operations --------------------------------------------------------------------------
  m.def("enqueue", [](OpSpec spec) {
    py::gil_scoped_release nogil;   // a GPU collective may be issued right here, on the calling thread
    return Runtime::Get().Enqueue(std::move(spec));
  });
  m.def("poll", [](int h) { return Runtime::Get().Poll(h); });
  m.def("wait", [](int h) {
    Status s;
    {
      py::gil_scoped_release nogil;
      s = Runtime::Get().Wait(h);
    }
    ThrowIfError(s);
  });
  m.def("release", [](int h) { Runtime::Get().Release(h); });
  m.def("barrier_now", [] {
    py::gil_scoped_release nogil;
    ThrowIfError(Runtime::Get().BarrierNow());
  });
  m.def("allgather_bytes", [](py::bytes mine) {
    std::string in = mine;
    std::vector<std::string> all;
    {
      py::gil_scoped_release nogil;
      ThrowIfError(Runtime::Get().AllgatherBytesNow(in, &all));
    }
    std::vector<py::bytes> out;
    for (auto& s : all) out.emplace_back(s);
    return out;
  });

  // ---- timeline / logging ------------------------------------------------------------------
  m.def("timeline_initialized", [] { return Runtime::Get().timeline().Initialized(); });
  m.def("timeline_start", [](const std::string& file) { return Runtime::Get().timeline().Initialize(file, Runtime::Get().size()); });
  m.def("timeline_stop", [] { Runtime::Get().timeline().Shutdown(); });
  m.def("timeline_start_activity", [](const std::string& tensor, const std::string& activity) {
    auto& tl = Runtime::Get().timeline();
    if (!tl.Initialized()) return false;
    tl.ActivityStart(tensor, activity);
    return true;
  });
  m.def("timeline_end_activity", [](const std::string& tensor) {
    auto& tl = Runtime::Get().timeline();
    if (!tl.Initialized()) return false;
    tl.ActivityEnd(tensor);
    return true;
  });
  m.def("timeline_span", [](const std::string& tensor, const std::string& activity, long b, long e, long lane) {
    Runtime::Get().timeline().CompleteSpan(tensor, activity, b, e, lane);
  });
  m.def("timeline_now_us", [] { return Runtime::Get().timeline().NowMicros(); });
  m.def("log", [](int level, const std::string& msg, int rank) {
    if (level >= static_cast<int>(MinLogLevelFromEnv())) LogMessage("python", 0, static_cast<LogLevel>(level), rank) << msg;
  });
  m.def("log_level", [] { return static_cast<int>(MinLogLevelFromEnv()); });

  // ---- windows -----------------------------------------------------------------------------
  m.def("win_self_view", [](const std::string& name) { return Runtime::Get().windows()->SelfView(name); });
  m.def("win_update", [](const std::string& name, c10::optional<at::Tensor> out, double self_weight, std::vector<int> src_ranks,
                         std::vector<double> src_weights, bool reset, bool require_mutex) {
    Runtime& rt = Runtime::Get();
    at::Tensor view = rt.windows()->SelfView(name);
    void* stream = nullptr;
    if (view.defined() && view.is_cuda()) stream = CurrentStream(view.get_device());
    at::Tensor o = out.has_value() ? *out : at::Tensor();
    Status s;
    {
      py::gil_scoped_release nogil;
      rt.timeline().ActivityStart(name, "WIN_SYNC_COMPUTE_AVERAGE");
      s = rt.windows()->Update(name, o, self_weight, src_ranks, src_weights, reset, require_mutex, stream);
      rt.timeline().ActivityEnd(name);
    }
    ThrowIfError(s);
  });
  m.def("win_mutex_acquire", [](const std::string& name, std::vector<int> ranks, bool for_self) {
    py::gil_scoped_release nogil;
    ThrowIfError(Runtime::Get().windows()->MutexAcquire(name, ranks, for_self));
  });
  m.def("win_mutex_release", [](const std::string& name, std::vector<int> ranks, bool for_self) {
    ThrowIfError(Runtime::Get().windows()->MutexRelease(name, ranks, for_self));
  });
  m.def("win_versions", [](const std::string& name) {
    std::vector<int64_t> v;
    ThrowIfError(Runtime::Get().windows()->Versions(name, &v));
    return v;
  });
  m.def("win_get_p", [](const std::string& name) {
    double p = 0;
    ThrowIfError(Runtime::Get().windows()->GetAssociatedP(name, &p));
    return p;
  });
  m.def("win_set_p", [](const std::string& name, double p) { ThrowIfError(Runtime::Get().windows()->SetAssociatedP(name, p)); });
  m.def("win_set_with_p", [](bool v) { Runtime::Get().windows()->set_with_associated_p(v); });
  m.def("win_get_with_p", [] { return Runtime::Get().windows()->with_associated_p(); });
  m.def("win_names", [] { return Runtime::Get().windows() ? Runtime::Get().windows()->Names() : std::vector<std::string>(); });
  m.def("win_count", [] { return Runtime::Get().windows() ? Runtime::Get().windows()->Count() : size_t(0); });

  // ---- kernels on explicit buffers -----------------------------------------------------------
  m.def("scale_", [](at::Tensor t, double s) {
    TORCH_CHECK(t.is_cuda() && t.is_contiguous(), "scale_ needs a contiguous CUDA tensor");
    c10::cuda::CUDAGuard g(t.get_device());
    cudaError_t e = LaunchScale(t.data_ptr(), static_cast<unsigned long long>(t.numel()), s, ElemOf(t), CurrentStream(t.get_device()));
    TORCH_CHECK(e == cudaSuccess, "scale kernel launch failed: ", cudaGetErrorString(e));
  });

  // ---- fused BatchNorm (+ReLU, +residual), NHWC bf16 -----------------------------------------
  m.def("bn_supported", [](at::Tensor x) {
    return x.is_cuda() && x.dim() == 4 && x.scalar_type() == at::kBFloat16 &&
           x.is_contiguous(at::MemoryFormat::ChannelsLast) &&
           BnShapeSupported(x.numel() / std::max<int64_t>(x.size(1), 1), static_cast<int>(x.size(1)));
  });
  // zeroed fp32 words a BatchNorm pass over C channels wants for its one-launch form (accumulator copies + barrier)
  m.def("bn_workspace_floats", [](int C) { return BnSumCopies(C) * 2 * C + 16; });
  m.def("bn_forward", [](at::Tensor x, c10::optional<at::Tensor> residual, at::Tensor gamma, at::Tensor beta,
                         c10::optional<at::Tensor> running_mean, c10::optional<at::Tensor> running_var, double eps,
                         double momentum, bool relu, c10::optional<at::Tensor> zeroed_sums, bool stats_ready) {
    // stats_ready: zeroed_sums already holds sum(x) and sum(x^2) per channel (written by the kernel that produced
    // x), so the statistics pass over x is skipped
    TORCH_CHECK(!stats_ready || (zeroed_sums.has_value() && zeroed_sums->defined()), "stats_ready needs the sums");
    TORCH_CHECK(x.is_cuda() && x.dim() == 4 && x.scalar_type() == at::kBFloat16 &&
                x.is_contiguous(at::MemoryFormat::ChannelsLast), "bn_forward expects a bf16 NHWC (channels_last) CUDA tensor");
    const int C = static_cast<int>(x.size(1));
    const long long R = x.numel() / C;
    TORCH_CHECK(BnShapeSupported(R, C), "bn_forward: unsupported channel count ", C);
    TORCH_CHECK(gamma.numel() == C && beta.numel() == C && gamma.scalar_type() == beta.scalar_type(), "bad affine parameters");
    const bool pbf16 = gamma.scalar_type() == at::kBFloat16;
    TORCH_CHECK(pbf16 || gamma.scalar_type() == at::kFloat, "affine parameters must be bf16 or fp32");
    c10::cuda::CUDAGuard g(x.get_device());
    at::Tensor y = at::empty_like(x);
    auto fopts = x.options().dtype(at::kFloat);
    // 2*C floats that must be zero on entry; callers may hand in a slice of a workspace that they
    // clear once per step instead of paying one memset per layer
    at::Tensor sums;
    if (zeroed_sums.has_value() && zeroed_sums->defined()) {
      TORCH_CHECK(zeroed_sums->is_cuda() && zeroed_sums->scalar_type() == at::kFloat && zeroed_sums->is_contiguous() &&
                  zeroed_sums->numel() >= 2 * C, "zeroed_sums must be a contiguous fp32 CUDA tensor of 2*C elements");
      sums = *zeroed_sums;
    } else {
      sums = at::zeros({BnSumCopies(C) * 2 * C + 16}, fopts);
    }
    // room for several sets of accumulators and one more word lets the pass run as a single cooperative launch
    const int copies = static_cast<int>(std::min<int64_t>(BnSumCopies(C), (sums.numel() - 1) / (2 * C)));
    at::Tensor& status = GemmStatusWord(x);
    at::Tensor save_mean = at::empty({C}, fopts), save_rstd = at::empty({C}, fopts);
    const void* res = nullptr;
    if (residual.has_value() && residual->defined()) {
      TORCH_CHECK(residual->sizes() == x.sizes() && residual->scalar_type() == at::kBFloat16 &&
                  residual->is_contiguous(at::MemoryFormat::ChannelsLast), "residual must match x (bf16, channels_last)");
      res = residual->data_ptr();
    }
    float* rm = nullptr;
    float* rv = nullptr;
    if (running_mean.has_value() && running_mean->defined()) {
      TORCH_CHECK(running_mean->scalar_type() == at::kFloat && running_var->scalar_type() == at::kFloat, "running statistics must be fp32");
      rm = running_mean->data_ptr<float>();
      rv = running_var->data_ptr<float>();
    }
    at::Tensor mask = relu ? at::empty({static_cast<int64_t>(R) * (C / 8)}, x.options().dtype(at::kByte)) : at::Tensor();
    cudaError_t e = LaunchBnForward(x.data_ptr(), res, y.data_ptr(), relu ? mask.data_ptr() : nullptr,
                                    sums.data_ptr<float>(), gamma.data_ptr(), beta.data_ptr(),
                                    rm, rv, save_mean.data_ptr<float>(), save_rstd.data_ptr<float>(), R, C,
                                    static_cast<float>(eps), static_cast<float>(momentum), relu ? 1 : 0, pbf16 ? 1 : 0,
                                    CurrentStream(x.get_device()), stats_ready ? 1 : 0, copies,
                                    reinterpret_cast<unsigned int*>(status.data_ptr<int>()));
    TORCH_CHECK(e == cudaSuccess, "bn_forward launch failed: ", cudaGetErrorString(e));
    return std::make_tuple(y, save_mean, save_rstd, mask);
  }, py::arg("x"), py::arg("residual"), py::arg("gamma"), py::arg("beta"), py::arg("running_mean"),
     py::arg("running_var"), py::arg("eps"), py::arg("momentum"), py::arg("relu"), py::arg("zeroed_sums") = py::none(),
     py::arg("stats_ready") = false);
  m.def("bn_backward", [](at::Tensor dy, c10::optional<at::Tensor> mask, at::Tensor x, at::Tensor save_mean, at::Tensor save_rstd,
                          at::Tensor gamma, bool relu, bool want_dres, c10::optional<at::Tensor> zeroed_sums,
                          c10::optional<at::Tensor> dy2) {
    // dy2: a second addend of the incoming gradient; the kernels use dy + dy2 without a pass that adds them
    const void* dy2_ptr = nullptr;
    if (dy2.has_value() && dy2->defined()) {
      TORCH_CHECK(dy2->is_cuda() && dy2->scalar_type() == at::kBFloat16 && dy2->sizes() == dy.sizes() &&
                  dy2->is_contiguous(at::MemoryFormat::ChannelsLast), "dy2 must match dy (bf16, channels_last)");
      dy2_ptr = dy2->data_ptr();
    }
    TORCH_CHECK(dy.is_cuda() && dy.scalar_type() == at::kBFloat16 && dy.is_contiguous(at::MemoryFormat::ChannelsLast) &&
                dy.sizes() == x.sizes(), "bn_backward expects a bf16 NHWC gradient of the shape of x");
    const int C = static_cast<int>(x.size(1));
    const long long R = x.numel() / C;
    const bool pbf16 = gamma.scalar_type() == at::kBFloat16;
    c10::cuda::CUDAGuard g(x.get_device());
    at::Tensor dx = at::empty_like(x);
    at::Tensor dres = want_dres ? at::empty_like(x) : at::Tensor();
    at::Tensor sums = (zeroed_sums.has_value() && zeroed_sums->defined())
                          ? *zeroed_sums : at::zeros({BnSumCopies(C) * 2 * C + 16}, x.options().dtype(at::kFloat));
    TORCH_CHECK(sums.is_cuda() && sums.scalar_type() == at::kFloat && sums.is_contiguous() && sums.numel() >= 2 * C,
                "zeroed_sums must be a contiguous fp32 CUDA tensor of 2*C elements");
    const int copies = static_cast<int>(std::min<int64_t>(BnSumCopies(C), (sums.numel() - 1) / (2 * C)));
    at::Tensor& status = GemmStatusWord(x);
    at::Tensor dgamma = at::empty_like(gamma), dbeta = at::empty_like(gamma);
    const void* mptr = nullptr;
    if (relu) {
      TORCH_CHECK(mask.has_value() && mask->defined() && mask->scalar_type() == at::kByte &&
                  mask->numel() == R * (C / 8), "bn_backward needs the ReLU bit mask of the forward pass");
      mptr = mask->data_ptr();
    }
    cudaError_t e = LaunchBnBackward(dy.data_ptr(), dy2_ptr, mptr, x.data_ptr(), dx.data_ptr(),
                                     want_dres ? dres.data_ptr() : nullptr, sums.data_ptr<float>(),
                                     save_mean.data_ptr<float>(), save_rstd.data_ptr<float>(), gamma.data_ptr(),
                                     dgamma.data_ptr(), dbeta.data_ptr(), R, C, relu ? 1 : 0, pbf16 ? 1 : 0,
                                     CurrentStream(x.get_device()), copies,
                                     reinterpret_cast<unsigned int*>(status.data_ptr<int>()));
    TORCH_CHECK(e == cudaSuccess, "bn_backward launch failed: ", cudaGetErrorString(e));
    return std::make_tuple(dx, dres, dgamma, dbeta);
  }, py::arg("dy"), py::arg("mask"), py::arg("x"), py::arg("save_mean"), py::arg("save_rstd"), py::arg("gamma"),
     py::arg("relu"), py::arg("want_dres"), py::arg("zeroed_sums") = py::none(), py::arg("dy2") = py::none());

  // ---- LayerNorm over the last dimension, bf16 ------------------------------------------------
  m.def("ln_supported", [](at::Tensor x) {
    return x.is_cuda() && x.dim() >= 1 && x.scalar_type() == at::kBFloat16 && x.is_contiguous() && x.numel() > 0 &&
           LnShapeSupported(x.numel() / x.size(-1), static_cast<int>(x.size(-1)));
  });
  m.def("ln_forward", [](at::Tensor x, at::Tensor gamma, at::Tensor beta, double eps) {
    TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.is_contiguous() && x.dim() >= 1 && x.numel() > 0,
                "ln_forward expects a contiguous bf16 CUDA tensor");
    const int C = static_cast<int>(x.size(-1));
    const long long R = x.numel() / C;
    TORCH_CHECK(LnShapeSupported(R, C), "ln_forward: unsupported row length ", C);
    const bool pbf16 = gamma.scalar_type() == at::kBFloat16;
    TORCH_CHECK(gamma.is_cuda() && beta.is_cuda() && gamma.numel() == C && beta.numel() == C &&
                gamma.scalar_type() == beta.scalar_type() && (pbf16 || gamma.scalar_type() == at::kFloat) &&
                gamma.is_contiguous() && beta.is_contiguous(), "ln_forward: weight/bias must be C fp32 or bf16 values");
    at::Tensor y = at::empty_like(x);
    at::Tensor mean = at::empty({static_cast<int64_t>(R)}, x.options().dtype(at::kFloat));
    at::Tensor rstd = at::empty({static_cast<int64_t>(R)}, x.options().dtype(at::kFloat));
    cudaError_t e = LaunchLnForward(x.data_ptr(), gamma.data_ptr(), beta.data_ptr(), y.data_ptr(), mean.data_ptr<float>(),
                                    rstd.data_ptr<float>(), R, C, static_cast<float>(eps), pbf16 ? 1 : 0,
                                    CurrentStream(x.get_device()));
    TORCH_CHECK(e == cudaSuccess, "ln_forward launch failed: ", cudaGetErrorString(e));
    return std::make_tuple(y, mean, rstd);
  });
  // addend (optional, same shape as x): dx = LN'(dy) + addend, and a third row of the sums holds the fp32 column sums of dx.
  m.def("ln_backward", [](at::Tensor dy, at::Tensor x, at::Tensor gamma, at::Tensor mean, at::Tensor rstd,
                          c10::optional<at::Tensor> addend) {
    TORCH_CHECK(dy.is_cuda() && dy.scalar_type() == at::kBFloat16 && dy.is_contiguous() && dy.sizes() == x.sizes() &&
                x.scalar_type() == at::kBFloat16 && x.is_contiguous(), "ln_backward expects contiguous bf16 dy and x");
    const int C = static_cast<int>(x.size(-1));
    const long long R = x.numel() / C;
    TORCH_CHECK(LnShapeSupported(R, C) && mean.numel() == R && rstd.numel() == R && mean.scalar_type() == at::kFloat &&
                rstd.scalar_type() == at::kFloat, "ln_backward: statistics do not match x");
    const bool extra = addend.has_value() && addend->defined();
    if (extra)
      TORCH_CHECK(addend->is_cuda() && addend->scalar_type() == at::kBFloat16 && addend->is_contiguous() &&
                  addend->sizes() == x.sizes(), "ln_backward: the second gradient term has to be contiguous bf16 of x's shape");
    const bool pbf16 = gamma.scalar_type() == at::kBFloat16;
    c10::cuda::CUDAGuard g(x.get_device());
    at::Tensor dx = at::empty_like(x);
    at::Tensor sums = at::zeros({extra ? 3 : 2, static_cast<int64_t>(C)}, x.options().dtype(at::kFloat));
    float* sp = sums.data_ptr<float>();
    cudaStream_t stream = CurrentStream(x.get_device());
    cudaError_t e = LaunchLnBackward(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), mean.data_ptr<float>(),
                                     rstd.data_ptr<float>(), dx.data_ptr(), sp, sp + C, R, C, pbf16 ? 1 : 0, stream,
                                     extra ? addend->data_ptr() : nullptr, extra ? sp + 2 * C : nullptr);
    if (extra && e == cudaErrorNotSupported) {
      (void)cudaGetLastError();
      e = LaunchLnBackward(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), mean.data_ptr<float>(), rstd.data_ptr<float>(),
                           dx.data_ptr(), sp, sp + C, R, C, pbf16 ? 1 : 0, stream);
      TORCH_CHECK(e == cudaSuccess, "ln_backward launch failed: ", cudaGetErrorString(e));
      dx.add_(*addend);
      e = LaunchColumnSum(dx.data_ptr(), sp + 2 * C, R, C, stream);
    }
    TORCH_CHECK(e == cudaSuccess, "ln_backward launch failed: ", cudaGetErrorString(e));
    // rows of sums: dgamma, dbeta(, column sums of dx); one tensor so that a caller converts them in one pass
    return std::make_tuple(dx, sums);
  }, py::arg("dy"), py::arg("x"), py::arg("gamma"), py::arg("mean"), py::arg("rstd"), py::arg("addend") = py::none());

  // ---- token + position embedding (GPT-2) ------------------------------------------------------
  m.def("embed_forward", [](at::Tensor idx, at::Tensor wte, at::Tensor wpe) {
    TORCH_CHECK(idx.is_cuda() && idx.scalar_type() == at::kLong && idx.dim() == 2 && idx.is_contiguous(),
                "embed_forward: idx has to be a contiguous int64 CUDA matrix [batch, positions]");
    TORCH_CHECK(wte.is_cuda() && wpe.is_cuda() && wte.scalar_type() == at::kBFloat16 && wpe.scalar_type() == at::kBFloat16 &&
                wte.dim() == 2 && wpe.dim() == 2 && wte.is_contiguous() && wpe.is_contiguous() && wte.size(1) == wpe.size(1) &&
                wte.size(1) % 8 == 0 && idx.size(1) <= wpe.size(0) && idx.numel() > 0,
                "embed_forward: bf16 tables [V, C] and [P, C] with C % 8 == 0 and at most P positions");
    c10::cuda::CUDAGuard g(idx.get_device());
    const int C = static_cast<int>(wte.size(1));
    at::Tensor out = at::empty({idx.size(0), idx.size(1), wte.size(1)}, wte.options());
    at::Tensor bad = at::zeros({1}, idx.options().dtype(at::kInt));
    cudaError_t e = LaunchEmbedForward(reinterpret_cast<const long long*>(idx.data_ptr<int64_t>()), wte.data_ptr(), wpe.data_ptr(), out.data_ptr(), idx.numel(), static_cast<int>(idx.size(1)),
                                       C, wte.size(0), bad.data_ptr<int>(), CurrentStream(idx.get_device()));
    TORCH_CHECK(e == cudaSuccess, "embed_forward launch failed: ", cudaGetErrorString(e));
    return std::make_tuple(out, bad);
  });
  // slot: int32 [V] filled with INT_MAX, acc: fp32 [N, C] zeros; both come back in that state
  m.def("embed_backward", [](at::Tensor idx, at::Tensor dx, int64_t vocab, at::Tensor slot, at::Tensor acc) {
    TORCH_CHECK(idx.is_cuda() && idx.scalar_type() == at::kLong && idx.dim() == 2 && idx.is_contiguous() && dx.is_cuda() &&
                dx.scalar_type() == at::kBFloat16 && dx.is_contiguous() && dx.dim() == 3 && dx.size(0) == idx.size(0) &&
                dx.size(1) == idx.size(1) && dx.size(2) % 8 == 0, "embed_backward: dx has to be contiguous bf16 [batch, positions, C]");
    TORCH_CHECK(slot.is_cuda() && slot.scalar_type() == at::kInt && slot.numel() >= vocab && acc.is_cuda() &&
                acc.scalar_type() == at::kFloat && acc.numel() >= dx.numel() && slot.is_contiguous() && acc.is_contiguous(),
                "embed_backward: scratch buffers too small");
    c10::cuda::CUDAGuard g(idx.get_device());
    const int C = static_cast<int>(dx.size(2));
    at::Tensor d_wte = at::empty({vocab, dx.size(2)}, dx.options());
    at::Tensor d_wpe = at::empty({idx.size(1), dx.size(2)}, dx.options());
    cudaError_t e = LaunchEmbedBackward(reinterpret_cast<const long long*>(idx.data_ptr<int64_t>()), dx.data_ptr(), d_wte.data_ptr(),
                                        d_wpe.data_ptr(), slot.data_ptr<int>(), acc.data_ptr<float>(), idx.numel(),
                                        static_cast<int>(idx.size(1)), C, vocab, CurrentStream(idx.get_device()));
    TORCH_CHECK(e == cudaSuccess, "embed_backward launch failed: ", cudaGetErrorString(e));
    return std::make_tuple(d_wte, d_wpe);
  });

  m.def("column_sum", [](at::Tensor x) {
    TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.scalar_type() == at::kBFloat16 && x.is_contiguous() &&
                x.size(1) % 8 == 0 && x.numel() > 0, "column_sum expects a contiguous bf16 CUDA matrix with C % 8 == 0");
    c10::cuda::CUDAGuard g(x.get_device());
    at::Tensor out = at::zeros({x.size(1)}, x.options().dtype(at::kFloat));
    cudaError_t e = LaunchColumnSum(x.data_ptr(), out.data_ptr<float>(), x.size(0), static_cast<int>(x.size(1)),
                                    CurrentStream(x.get_device()));
    TORCH_CHECK(e == cudaSuccess, "column_sum launch failed: ", cudaGetErrorString(e));
    return out;
  });

  // ---- space-to-depth input of the ResNet stem -------------------------------------------------
  m.def("s2d_stem_input", [](at::Tensor x) {
    TORCH_CHECK(x.is_cuda() && x.dim() == 4 && x.size(1) == 3 && x.size(2) % 2 == 0 && x.size(3) % 2 == 0 &&
                (x.scalar_type() == at::kFloat || x.scalar_type() == at::kBFloat16),
                "s2d_stem_input expects a [N, 3, H, W] fp32 or bf16 CUDA tensor with even H and W");
    c10::cuda::CUDAGuard g(x.get_device());
    const int N = static_cast<int>(x.size(0)), H = static_cast<int>(x.size(2)), W = static_cast<int>(x.size(3));
    at::Tensor out = at::empty({N, 16, (H + 6) / 2, (W + 6) / 2},
                               x.options().dtype(at::kBFloat16).memory_format(at::MemoryFormat::ChannelsLast));
    cudaError_t e = LaunchS2dStemInput(x.data_ptr(), x.scalar_type() == at::kBFloat16 ? 1 : 0, out.data_ptr(), N, H, W,
                                       x.stride(0), x.stride(1), x.stride(2), x.stride(3), CurrentStream(x.get_device()));
    TORCH_CHECK(e == cudaSuccess, "s2d_stem_input launch failed: ", cudaGetErrorString(e));
    return out;
  });

  // ---- mean cross-entropy of bf16 logits ------------------------------------------------------
  m.def("cross_entropy_forward", [](at::Tensor logits, at::Tensor target) {
    TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.scalar_type() == at::kBFloat16 && logits.is_contiguous() &&
                logits.size(1) % 8 == 0 && logits.size(0) > 0, "cross_entropy_forward expects contiguous bf16 logits [R, C], C % 8 == 0");
    TORCH_CHECK(target.is_cuda() && target.scalar_type() == at::kLong && target.is_contiguous() &&
                target.numel() == logits.size(0), "cross_entropy_forward expects int64 targets [R]");
    c10::cuda::CUDAGuard g(logits.get_device());
    at::Tensor lse = at::empty({logits.size(0)}, logits.options().dtype(at::kFloat));
    at::Tensor loss = at::zeros({}, logits.options().dtype(at::kFloat));
    cudaError_t e = LaunchCrossEntropyForward(logits.data_ptr(), reinterpret_cast<const long long*>(target.data_ptr<int64_t>()),
                                              lse.data_ptr<float>(), loss.data_ptr<float>(), logits.size(0),
                                              static_cast<int>(logits.size(1)), CurrentStream(logits.get_device()));
    TORCH_CHECK(e == cudaSuccess, "cross_entropy_forward launch failed: ", cudaGetErrorString(e));
    return std::make_tuple(loss, lse);
  });
  m.def("cross_entropy_backward", [](at::Tensor logits, at::Tensor target, at::Tensor lse, at::Tensor grad_out) {
    TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.scalar_type() == at::kBFloat16 && logits.is_contiguous() &&
                logits.size(1) % 8 == 0, "cross_entropy_backward expects contiguous bf16 logits [R, C], C % 8 == 0");
    TORCH_CHECK(grad_out.is_cuda() && grad_out.scalar_type() == at::kFloat && grad_out.numel() == 1 &&
                lse.scalar_type() == at::kFloat && lse.numel() == logits.size(0) && target.scalar_type() == at::kLong &&
                target.numel() == logits.size(0), "cross_entropy_backward: mismatched arguments");
    c10::cuda::CUDAGuard g(logits.get_device());
    at::Tensor dx = at::empty_like(logits);
    cudaError_t e = LaunchCrossEntropyBackward(logits.data_ptr(), reinterpret_cast<const long long*>(target.data_ptr<int64_t>()),
                                               lse.data_ptr<float>(), grad_out.data_ptr<float>(), dx.data_ptr(),
                                               logits.size(0), static_cast<int>(logits.size(1)),
                                               CurrentStream(logits.get_device()));
    TORCH_CHECK(e == cudaSuccess, "cross_entropy_backward launch failed: ", cudaGetErrorString(e));
    return dx;
  });

  // ---- 3x3/2 max pooling, NHWC bf16 ---------------------------------------------------------
  m.def("maxpool3x3s2_forward", [](at::Tensor x) {
    TORCH_CHECK(x.is_cuda() && x.dim() == 4 && x.scalar_type() == at::kBFloat16 &&
                x.is_contiguous(at::MemoryFormat::ChannelsLast) && x.size(1) % 8 == 0,
                "maxpool3x3s2_forward expects a bf16 NHWC CUDA tensor with C % 8 == 0");
    const int N = x.size(0), C = x.size(1), H = x.size(2), W = x.size(3);
    const int Ho = (H - 1) / 2 + 1, Wo = (W - 1) / 2 + 1;
    c10::cuda::CUDAGuard g(x.get_device());
    at::Tensor y = at::empty({N, C, Ho, Wo}, x.options().memory_format(at::MemoryFormat::ChannelsLast));
    at::Tensor idx = at::empty({N, C, Ho, Wo}, x.options().dtype(at::kByte).memory_format(at::MemoryFormat::ChannelsLast));
    cudaError_t e = LaunchMaxPool3x3s2Forward(x.data_ptr(), y.data_ptr(), idx.data_ptr(), N, H, W, C, CurrentStream(x.get_device()));
    TORCH_CHECK(e == cudaSuccess, "maxpool forward launch failed: ", cudaGetErrorString(e));
    return std::make_tuple(y, idx);
  });
  m.def("maxpool3x3s2_backward", [](at::Tensor dy, at::Tensor idx, int64_t H, int64_t W) {
    TORCH_CHECK(dy.is_cuda() && dy.scalar_type() == at::kBFloat16 && dy.is_contiguous(at::MemoryFormat::ChannelsLast),
                "maxpool3x3s2_backward expects a bf16 NHWC gradient");
    const int N = dy.size(0), C = dy.size(1);
    c10::cuda::CUDAGuard g(dy.get_device());
    at::Tensor dx = at::empty({N, C, H, W}, dy.options().memory_format(at::MemoryFormat::ChannelsLast));
    cudaError_t e = LaunchMaxPool3x3s2Backward(dy.data_ptr(), idx.data_ptr(), dx.data_ptr(), N, static_cast<int>(H),
                                               static_cast<int>(W), C, CurrentStream(dy.get_device()));
    TORCH_CHECK(e == cudaSuccess, "maxpool backward launch failed: ", cudaGetErrorString(e));
    return dx;
  });

  // ---- tcgen05 GEMM -------------------------------------------------------------------------
  m.def("gemm_supported", [] { return GemmSupported(); });
  // col_stats (optional, >= 2*N zero-initialised or running fp32 values): receives the column sums and sums of
  // squares of the rounded output, added by the GEMM epilogue (needs N % 8 == 0, no bias, act == 0)
  m.def("gemm_bf16_nt", [](at::Tensor a, at::Tensor w, c10::optional<at::Tensor> bias, int act,
                           c10::optional<at::Tensor> col_stats, c10::optional<at::Tensor> addend) {
    TORCH_CHECK(a.is_cuda() && w.is_cuda() && a.dim() == 2 && w.dim() == 2, "gemm_bf16_nt expects 2-D CUDA tensors");
    TORCH_CHECK(a.scalar_type() == at::kBFloat16 && w.scalar_type() == at::kBFloat16, "gemm_bf16_nt expects bf16");
    TORCH_CHECK(a.is_contiguous() && w.is_contiguous(), "gemm_bf16_nt expects contiguous tensors");
    TORCH_CHECK(a.size(1) == w.size(1), "inner dimensions differ");
    TORCH_CHECK(a.size(1) % 8 == 0, "K must be a multiple of 8");
    c10::cuda::CUDAGuard g(a.get_device());
    at::Tensor& status = GemmStatusWord(a);
    at::Tensor out = at::empty({a.size(0), w.size(0)}, a.options());
    const void* bptr = nullptr;
    if (bias.has_value() && bias->defined()) {
      TORCH_CHECK(bias->scalar_type() == at::kBFloat16 && bias->is_contiguous() && bias->numel() == w.size(0), "bias must be bf16 [N]");
      bptr = bias->data_ptr();
    }
    float* stats = nullptr;
    if (col_stats.has_value() && col_stats->defined()) {
      TORCH_CHECK(col_stats->is_cuda() && col_stats->scalar_type() == at::kFloat && col_stats->is_contiguous() &&
                  col_stats->numel() >= 2 * w.size(0) && w.size(0) % 8 == 0 && bptr == nullptr && act == 0 &&
                  (reinterpret_cast<uintptr_t>(col_stats->data_ptr()) & 15) == 0,
                  "col_stats needs 2*N 16-byte aligned fp32 values, N % 8 == 0, no bias and no activation");
      stats = col_stats->data_ptr<float>();
    }
    const void* add = nullptr;
    if (addend.has_value() && addend->defined()) {
      // out = a w^T + bias + addend, the addend read in the epilogue
      TORCH_CHECK(addend->is_cuda() && addend->scalar_type() == at::kBFloat16 && addend->is_contiguous() &&
                  addend->dim() == 2 && addend->size(0) == a.size(0) && addend->size(1) == w.size(0) && w.size(0) % 8 == 0 &&
                  act == 0 && stats == nullptr, "addend must be a contiguous bf16 [M, N] matrix, N % 8 == 0, no activation");
      add = addend->data_ptr();
    }
    cudaError_t e = LaunchGemmBf16NT(a.data_ptr(), w.data_ptr(), out.data_ptr(), bptr, static_cast<int>(a.size(0)),
                                     static_cast<int>(w.size(0)), static_cast<int>(a.size(1)), act,
                                     reinterpret_cast<unsigned int*>(status.data_ptr()), CurrentStream(a.get_device()),
                                     nullptr, stats, add);
    TORCH_CHECK(e == cudaSuccess, "gemm_bf16_nt launch failed: ", cudaGetErrorString(e));
    return out;
  }, py::arg("a"), py::arg("w"), py::arg("bias") = py::none(), py::arg("act") = 0, py::arg("col_stats") = py::none(),
     py::arg("addend") = py::none());

  // ---- tcgen05 implicit-GEMM 3x3 convolution (stride 1, pad 1), NHWC bf16 ---------------------
  m.def("conv3x3_supported", [](int64_t n, int64_t h, int64_t w, int64_t cin, int64_t cout) {
    return Conv3x3Supported(static_cast<int>(n), static_cast<int>(h), static_cast<int>(w), static_cast<int>(cin),
                            static_cast<int>(cout));
  });
  m.def("conv3x3_nhwc", [](at::Tensor x, at::Tensor w, bool flip_taps, int filter_mode) {
    TORCH_CHECK(x.is_cuda() && w.is_cuda() && x.dim() == 4 && w.dim() == 4 && x.scalar_type() == at::kBFloat16 &&
                w.scalar_type() == at::kBFloat16, "conv3x3_nhwc expects 4-D bf16 CUDA tensors");
    TORCH_CHECK(x.is_contiguous(at::MemoryFormat::ChannelsLast) && w.is_contiguous(at::MemoryFormat::ChannelsLast),
                "conv3x3_nhwc expects channels_last input and filter");
    // filter_mode 0: w = [Cout, Cin, 3, 3]; 1: w = [Cin, Cout, 3, 3], i.e. the forward filter of an input gradient
    const int red_dim = filter_mode == 0 ? 1 : 0, out_dim = filter_mode == 0 ? 0 : 1;
    TORCH_CHECK(w.size(2) == 3 && w.size(3) == 3 && w.size(red_dim) == x.size(1), "conv3x3_nhwc: filter does not match the input");
    const int N = static_cast<int>(x.size(0)), Cin = static_cast<int>(x.size(1)), H = static_cast<int>(x.size(2)),
              W = static_cast<int>(x.size(3)), Cout = static_cast<int>(w.size(out_dim));
    TORCH_CHECK(Conv3x3Supported(N, H, W, Cin, Cout), "conv3x3_nhwc: unsupported shape");
    c10::cuda::CUDAGuard g(x.get_device());
    at::Tensor& status = GemmStatusWord(x);
    at::Tensor y = at::empty({N, Cout, H, W}, x.options().memory_format(at::MemoryFormat::ChannelsLast));
    cudaError_t e = LaunchConv3x3Nhwc(x.data_ptr(), w.data_ptr(), y.data_ptr(), N, H, W, Cin, Cout, flip_taps ? 1 : 0,
                                      filter_mode, reinterpret_cast<unsigned int*>(status.data_ptr()),
                                      CurrentStream(x.get_device()));
    TORCH_CHECK(e == cudaSuccess, "conv3x3_nhwc launch failed: ", cudaGetErrorString(e));
    return y;
  }, py::arg("x"), py::arg("w"), py::arg("flip_taps") = false, py::arg("filter_mode") = 0);

  // ---- general implicit-GEMM convolution (taps, strides) and its filter gradient ---------------
  // x: bf16 channels_last [N, C, H, W].  stem_view: x has 16 channels and every position reads the 64 consecutive
  // values of four neighbouring pixels (reduction channels = 64, usable width = W - 3).
  // w: contiguous bf16 memory [Cout, w_taps, Cred] (filter_mode 0) or [Cred, w_taps, Cout] (filter_mode 1).
  // y: bf16 channels_last [N, Cout, Hy, Wy], written at (a*out_stride + out_ph, b*out_stride + out_pw) for the
  // grid of output positions a < Ho, b < Wo; positions of y outside that lattice are left as they are.
  m.def("conv_igemm", [](at::Tensor x, at::Tensor w, at::Tensor y, int64_t Ho, int64_t Wo, std::vector<int> dh,
                         std::vector<int> dw, std::vector<int> wt, int64_t w_taps, int64_t in_stride, int64_t filter_mode,
                         int64_t out_stride, int64_t out_ph, int64_t out_pw, bool stem_view) {
    TORCH_CHECK(x.is_cuda() && w.is_cuda() && y.is_cuda() && x.dim() == 4 && y.dim() == 4 &&
                x.scalar_type() == at::kBFloat16 && w.scalar_type() == at::kBFloat16 && y.scalar_type() == at::kBFloat16,
                "conv_igemm expects bf16 CUDA tensors");
    TORCH_CHECK(x.is_contiguous(at::MemoryFormat::ChannelsLast) && y.is_contiguous(at::MemoryFormat::ChannelsLast),
                "conv_igemm expects channels_last activations");
    TORCH_CHECK(dh.size() == dw.size() && dh.size() == wt.size() && !dh.empty() && dh.size() <= size_t(kConvMaxTaps),
                "conv_igemm: between 1 and 16 taps");
    ConvProblem p{};
    p.x = MakeConvView(x, stem_view);
    const int64_t Cout = y.size(1);
    TORCH_CHECK(w.numel() == Cout * w_taps * p.x.c && y.size(0) == x.size(0), "conv_igemm: filter or output does not match");
    p.w = w.data_ptr();
    p.filter_mode = static_cast<int>(filter_mode);
    p.w_taps = static_cast<int>(w_taps);
    p.y = y.data_ptr();
    p.Hy = static_cast<int>(y.size(2)); p.Wy = static_cast<int>(y.size(3)); p.Cout = static_cast<int>(Cout);
    p.Ho = static_cast<int>(Ho); p.Wo = static_cast<int>(Wo);
    p.out_stride = static_cast<int>(out_stride); p.out_ph = static_cast<int>(out_ph); p.out_pw = static_cast<int>(out_pw);
    p.in_stride = static_cast<int>(in_stride);
    p.taps.T = static_cast<int>(dh.size());
    for (int i = 0; i < p.taps.T; ++i) { p.taps.dh[i] = dh[i]; p.taps.dw[i] = dw[i]; p.taps.wt[i] = wt[i]; }
    TORCH_CHECK((Ho - 1) * out_stride + out_ph < y.size(2) && (Wo - 1) * out_stride + out_pw < y.size(3),
                "conv_igemm: the output lattice leaves y");
    TORCH_CHECK(ConvIgemmSupported(p), "conv_igemm: unsupported shape");
    c10::cuda::CUDAGuard g(x.get_device());
    at::Tensor& status = GemmStatusWord(x);
    cudaError_t e = LaunchConvIgemm(p, reinterpret_cast<unsigned int*>(status.data_ptr()), CurrentStream(x.get_device()));
    TORCH_CHECK(e == cudaSuccess, "conv_igemm launch failed: ", cudaGetErrorString(e));
    return y;
  }, py::arg("x"), py::arg("w"), py::arg("y"), py::arg("Ho"), py::arg("Wo"), py::arg("dh"), py::arg("dw"), py::arg("wt"),
     py::arg("w_taps"), py::arg("in_stride") = 1, py::arg("filter_mode") = 0, py::arg("out_stride") = 1,
     py::arg("out_ph") = 0, py::arg("out_pw") = 0, py::arg("stem_view") = false);
  m.def("conv_igemm_supported", [](int64_t n, int64_t ho, int64_t wo, int64_t cred, int64_t cout, int64_t in_stride) {
    int bw, bh, bn;
    return GemmSupported() && cred >= 64 && cred % 64 == 0 && cout >= 8 && cout % 8 == 0 &&
           ConvPatch(static_cast<int>(n), static_cast<int>(ho), static_cast<int>(wo), false, &bw, &bh, &bn) &&
           bw * in_stride <= 256 && bh * in_stride <= 256;
  });
  // dw[Cout, w_taps, Cred] (bf16) = sum over positions of dy (x) shifted x, see conv_tcgen05.h
  m.def("conv_wgrad", [](at::Tensor dy, at::Tensor x, std::vector<int> dh, std::vector<int> dw, std::vector<int> wt,
                         int64_t w_taps, int64_t in_stride, bool stem_view) {
    TORCH_CHECK(dy.is_cuda() && x.is_cuda() && dy.dim() == 4 && x.dim() == 4 && dy.scalar_type() == at::kBFloat16 &&
                x.scalar_type() == at::kBFloat16, "conv_wgrad expects 4-D bf16 CUDA tensors");
    TORCH_CHECK(x.is_contiguous(at::MemoryFormat::ChannelsLast) && dy.is_contiguous(at::MemoryFormat::ChannelsLast),
                "conv_wgrad expects channels_last tensors");
    TORCH_CHECK(dh.size() == dw.size() && dh.size() == wt.size() && !dh.empty() && dh.size() <= size_t(kConvMaxTaps),
                "conv_wgrad: between 1 and 16 taps");
    WgradProblem p{};
    p.dy = MakeConvView(dy, false);
    p.x = MakeConvView(x, stem_view);
    p.in_stride = static_cast<int>(in_stride);
    p.taps.T = static_cast<int>(dh.size());
    for (int i = 0; i < p.taps.T; ++i) { p.taps.dh[i] = dh[i]; p.taps.dw[i] = dw[i]; p.taps.wt[i] = wt[i]; }
    p.w_taps = static_cast<int>(w_taps);
    TORCH_CHECK(ConvWgradSupported(p), "conv_wgrad: unsupported shape");
    c10::cuda::CUDAGuard g(x.get_device());
    cudaStream_t stream = CurrentStream(x.get_device());
    at::Tensor out = at::empty({dy.size(1), w_taps, static_cast<int64_t>(p.x.c)}, x.options());
    WgradScratch& sc = WgradScratchFor(x, stream, out.numel());
    p.dw = out.data_ptr();
    p.workspace = sc.sums.data_ptr<float>();
    p.workspace_floats = sc.sums.numel();
    p.counters = reinterpret_cast<unsigned int*>(sc.counters.data_ptr());
    p.n_counters = static_cast<int>(sc.counters.numel());
    at::Tensor& status = GemmStatusWord(x);
    cudaError_t e = LaunchConvWgrad(p, reinterpret_cast<unsigned int*>(status.data_ptr()), stream);
    TORCH_CHECK(e == cudaSuccess, "conv_wgrad launch failed: ", cudaGetErrorString(e));
    return out;
  }, py::arg("dy"), py::arg("x"), py::arg("dh"), py::arg("dw"), py::arg("wt"), py::arg("w_taps"), py::arg("in_stride") = 1,
     py::arg("stem_view") = false);
  m.def("conv_wgrad_supported", [](int64_t n, int64_t ho, int64_t wo, int64_t cin, int64_t cout, int64_t in_stride) {
    int bw, bh, bn;
    return GemmSupported() && cin >= 64 && cin % 64 == 0 && cout >= 8 && cout % 8 == 0 &&
           ConvPatch(static_cast<int>(n), static_cast<int>(ho), static_cast<int>(wo), true, &bw, &bh, &bn) &&
           bw * in_stride <= 256 && bh * in_stride <= 256;
  });

  // ---- global average pooling, NHWC bf16 ----------------------------------------------------
  m.def("avgpool_forward", [](at::Tensor x) {
    TORCH_CHECK(x.is_cuda() && x.dim() == 4 && x.scalar_type() == at::kBFloat16 &&
                x.is_contiguous(at::MemoryFormat::ChannelsLast) && x.size(1) % 8 == 0,
                "avgpool_forward expects a bf16 NHWC CUDA tensor with C % 8 == 0");
    c10::cuda::CUDAGuard g(x.get_device());
    at::Tensor y = at::empty({x.size(0), x.size(1)}, x.options());
    cudaError_t e = LaunchAvgPoolForward(x.data_ptr(), y.data_ptr(), static_cast<int>(x.size(0)),
                                         static_cast<int>(x.size(2) * x.size(3)), static_cast<int>(x.size(1)),
                                         CurrentStream(x.get_device()));
    TORCH_CHECK(e == cudaSuccess, "avgpool forward launch failed: ", cudaGetErrorString(e));
    return y;
  });
  m.def("avgpool_backward", [](at::Tensor dy, int64_t H, int64_t W) {
    TORCH_CHECK(dy.is_cuda() && dy.dim() == 2 && dy.scalar_type() == at::kBFloat16 && dy.is_contiguous() && dy.size(1) % 8 == 0,
                "avgpool_backward expects a contiguous bf16 [N, C] gradient with C % 8 == 0");
    c10::cuda::CUDAGuard g(dy.get_device());
    at::Tensor dx = at::empty({dy.size(0), dy.size(1), H, W}, dy.options().memory_format(at::MemoryFormat::ChannelsLast));
    cudaError_t e = LaunchAvgPoolBackward(dy.data_ptr(), dx.data_ptr(), static_cast<int>(dy.size(0)), static_cast<int>(H * W),
                                          static_cast<int>(dy.size(1)), CurrentStream(dy.get_device()));
    TORCH_CHECK(e == cudaSuccess, "avgpool backward launch failed: ", cudaGetErrorString(e));
    return dx;
  });

  m.def("gemm_bf16_nn", [](at::Tensor a, at::Tensor b, c10::optional<at::Tensor> addend) {
    TORCH_CHECK(a.is_cuda() && b.is_cuda() && a.dim() == 2 && b.dim() == 2 && a.scalar_type() == at::kBFloat16 &&
                b.scalar_type() == at::kBFloat16 && a.is_contiguous() && b.is_contiguous() && a.size(1) == b.size(0),
                "gemm_bf16_nn expects contiguous bf16 CUDA matrices [M,K] and [K,N]");
    const void* add = nullptr;
    if (addend.has_value() && addend->defined()) {
      TORCH_CHECK(addend->is_cuda() && addend->scalar_type() == at::kBFloat16 && addend->is_contiguous() && addend->dim() == 2 &&
                  addend->size(0) == a.size(0) && addend->size(1) == b.size(1), "addend must be a contiguous bf16 [M,N] matrix");
      add = addend->data_ptr();
    }
    c10::cuda::CUDAGuard g(a.get_device());
    at::Tensor& status = GemmStatusWord(a);
    at::Tensor out = at::empty({a.size(0), b.size(1)}, a.options());
    cudaError_t e = LaunchGemmBf16NN(a.data_ptr(), b.data_ptr(), out.data_ptr(), static_cast<int>(a.size(0)),
                                     static_cast<int>(b.size(1)), static_cast<int>(a.size(1)),
                                     reinterpret_cast<unsigned int*>(status.data_ptr()), CurrentStream(a.get_device()),
                                     nullptr, add);
    TORCH_CHECK(e == cudaSuccess, "gemm_bf16_nn launch failed: ", cudaGetErrorString(e));
    return out;
  }, py::arg("a"), py::arg("b"), py::arg("addend") = py::none());

  // act(a w^T + bias) with the tanh GELU, returning the activated matrix and the pre-activation (kept for backward)
  m.def("gemm_bf16_nt_gelu", [](at::Tensor a, at::Tensor w, c10::optional<at::Tensor> bias) {
    TORCH_CHECK(a.is_cuda() && w.is_cuda() && a.dim() == 2 && w.dim() == 2 && a.scalar_type() == at::kBFloat16 &&
                w.scalar_type() == at::kBFloat16 && a.is_contiguous() && w.is_contiguous() && a.size(1) == w.size(1) &&
                a.size(1) % 8 == 0 && w.size(0) % 8 == 0, "gemm_bf16_nt_gelu expects contiguous bf16 [M,K], [N,K] with K, N % 8 == 0");
    c10::cuda::CUDAGuard g(a.get_device());
    at::Tensor& status = GemmStatusWord(a);
    at::Tensor out = at::empty({a.size(0), w.size(0)}, a.options());
    at::Tensor pre = at::empty({a.size(0), w.size(0)}, a.options());
    const void* bptr = nullptr;
    if (bias.has_value() && bias->defined()) {
      TORCH_CHECK(bias->scalar_type() == at::kBFloat16 && bias->is_contiguous() && bias->numel() == w.size(0), "bias must be bf16 [N]");
      bptr = bias->data_ptr();
    }
    cudaError_t e = LaunchGemmBf16NT(a.data_ptr(), w.data_ptr(), out.data_ptr(), bptr, static_cast<int>(a.size(0)),
                                     static_cast<int>(w.size(0)), static_cast<int>(a.size(1)), kActGeluTanh,
                                     reinterpret_cast<unsigned int*>(status.data_ptr()), CurrentStream(a.get_device()),
                                     pre.data_ptr());
    TORCH_CHECK(e == cudaSuccess, "gemm_bf16_nt_gelu launch failed: ", cudaGetErrorString(e));
    return std::make_tuple(out, pre);
  }, py::arg("a"), py::arg("w"), py::arg("bias") = py::none());
  // (a b) * GELU'(preact): the input gradient through a GELU whose pre-activation was kept
  m.def("gemm_bf16_nn_gelu_grad", [](at::Tensor a, at::Tensor b, at::Tensor preact) {
    TORCH_CHECK(a.is_cuda() && b.is_cuda() && a.dim() == 2 && b.dim() == 2 && a.scalar_type() == at::kBFloat16 &&
                b.scalar_type() == at::kBFloat16 && a.is_contiguous() && b.is_contiguous() && a.size(1) == b.size(0),
                "gemm_bf16_nn_gelu_grad expects contiguous bf16 CUDA matrices [M,K] and [K,N]");
    TORCH_CHECK(preact.is_cuda() && preact.scalar_type() == at::kBFloat16 && preact.is_contiguous() && preact.dim() == 2 &&
                preact.size(0) == a.size(0) && preact.size(1) == b.size(1), "preact must be bf16 [M,N]");
    c10::cuda::CUDAGuard g(a.get_device());
    at::Tensor& status = GemmStatusWord(a);
    at::Tensor out = at::empty({a.size(0), b.size(1)}, a.options());
    cudaError_t e = LaunchGemmBf16NN(a.data_ptr(), b.data_ptr(), out.data_ptr(), static_cast<int>(a.size(0)),
                                     static_cast<int>(b.size(1)), static_cast<int>(a.size(1)),
                                     reinterpret_cast<unsigned int*>(status.data_ptr()), CurrentStream(a.get_device()),
                                     preact.data_ptr());
    TORCH_CHECK(e == cudaSuccess, "gemm_bf16_nn_gelu_grad launch failed: ", cudaGetErrorString(e));
    return out;
  });

  m.def("gemm_bf16_tn", [](at::Tensor a, at::Tensor b) {
    TORCH_CHECK(a.is_cuda() && b.is_cuda() && a.dim() == 2 && b.dim() == 2 && a.scalar_type() == at::kBFloat16 &&
                b.scalar_type() == at::kBFloat16 && a.is_contiguous() && b.is_contiguous() && a.size(0) == b.size(0),
                "gemm_bf16_tn expects contiguous bf16 CUDA matrices [K,M] and [K,N]");
    c10::cuda::CUDAGuard g(a.get_device());
    at::Tensor& status = GemmStatusWord(a);
    at::Tensor out = at::empty({a.size(1), b.size(1)}, a.options());
    cudaError_t e = LaunchGemmBf16TN(a.data_ptr(), b.data_ptr(), out.data_ptr(), static_cast<int>(a.size(1)),
                                     static_cast<int>(b.size(1)), static_cast<int>(a.size(0)),
                                     reinterpret_cast<unsigned int*>(status.data_ptr()), CurrentStream(a.get_device()));
    TORCH_CHECK(e == cudaSuccess, "gemm_bf16_tn launch failed: ", cudaGetErrorString(e));
    return out;
  }, py::arg("a"), py::arg("b"));

  m.def("gemm_status", [] {
    at::Tensor probe = at::empty({0}, at::TensorOptions().device(at::kCUDA));
    return GemmStatusWord(probe).item<int>();
  });

  py::class_<LocalWindows>(m, "LocalWindows")
      .def(py::init([](int world, int64_t numel, py::object dtype, int device) {
             return std::make_unique<LocalWindows>(world, numel, torch::python::detail::py_object_to_dtype(dtype), device);
           }), py::arg("world"), py::arg("numel"), py::arg("dtype"), py::arg("device") = 0)
      .def("self_tensor", &LocalWindows::self_tensor)
      .def("slot_tensor", &LocalWindows::slot_tensor)
      .def("put", &LocalWindows::put, py::arg("rank"), py::arg("src"), py::arg("dst"), py::arg("weights"),
           py::arg("self_weight") = 1.0, py::arg("accumulate") = false, py::arg("with_p") = false, py::arg("guarded") = false)
      .def("get", &LocalWindows::get)
      .def("update", &LocalWindows::update, py::arg("rank"), py::arg("srcs"), py::arg("weights"), py::arg("self_weight") = 1.0,
           py::arg("reset") = false, py::arg("with_p") = false)
      .def("lock", &LocalWindows::lock, py::arg("rank"), py::arg("owners"), py::arg("index"), py::arg("acquire"),
           py::arg("timeout_ms") = 1000.0)
      .def("lock_state", &LocalWindows::lock_state)
      .def("versions", &LocalWindows::versions)
      .def("p_values", &LocalWindows::p_values)
      .def("set_p", &LocalWindows::set_p);

  py::class_<LocalWorld>(m, "LocalWorld")
      .def(py::init<int, int64_t, int>(), py::arg("world"), py::arg("half_bytes"), py::arg("device") = 0)
      .def("set_timeout_ms", &LocalWorld::set_timeout_ms)
      .def("publish", &LocalWorld::publish, py::arg("rank"), py::arg("tensors"), py::arg("dst_weight") = py::none(), py::arg("n_readers") = 0)
      .def("combine", &LocalWorld::combine)
      .def("gather", &LocalWorld::gather)
      .def("alloc_symmetric", &LocalWorld::alloc_symmetric)
      .def("publish_in_place", &LocalWorld::publish_in_place, py::arg("rank"), py::arg("x"), py::arg("dst_weight") = py::none(),
           py::arg("n_readers") = 0)
      .def("combine_in_place", &LocalWorld::combine_in_place)
      .def("wait_readers", &LocalWorld::wait_readers)
      .def("round_offsets", &LocalWorld::round_offsets)
      .def("status", &LocalWorld::status)
      .def("clear_status", &LocalWorld::clear_status);

  py::class_<PyBucketArgs>(m, "BucketStepArgs")
      .def(py::init<>())
      .def_readwrite("mode", &PyBucketArgs::mode)
      .def_readwrite("opt", &PyBucketArgs::opt)
      .def_readwrite("nesterov", &PyBucketArgs::nesterov)
      .def_readwrite("adamw", &PyBucketArgs::adamw)
      .def_readwrite("amsgrad", &PyBucketArgs::amsgrad)
      .def_readwrite("first_step", &PyBucketArgs::first_step)
      .def_readwrite("maximize", &PyBucketArgs::maximize)
      .def_readwrite("lr", &PyBucketArgs::lr)
      .def_readwrite("momentum", &PyBucketArgs::momentum)
      .def_readwrite("dampening", &PyBucketArgs::dampening)
      .def_readwrite("weight_decay", &PyBucketArgs::weight_decay)
      .def_readwrite("beta1", &PyBucketArgs::beta1)
      .def_readwrite("beta2", &PyBucketArgs::beta2)
      .def_readwrite("eps", &PyBucketArgs::eps)
      .def_readwrite("bias1", &PyBucketArgs::bias1)
      .def_readwrite("bias2", &PyBucketArgs::bias2)
      .def_readwrite("grad_scale", &PyBucketArgs::grad_scale)
      .def_readwrite("self_weight", &PyBucketArgs::self_weight)
      .def_readwrite("post_scale", &PyBucketArgs::post_scale)
      .def_readwrite("src_ranks", &PyBucketArgs::src_ranks)
      .def_readwrite("src_weights", &PyBucketArgs::src_weights)
      .def_readwrite("n_readers", &PyBucketArgs::n_readers)
      .def_readwrite("dst_weights", &PyBucketArgs::dst_weights)
      .def_readwrite("read_dst_weights", &PyBucketArgs::read_dst_weights)
      .def_readwrite("master", &PyBucketArgs::t_master)
      .def_readwrite("grad", &PyBucketArgs::t_grad)
      .def_readwrite("state1", &PyBucketArgs::t_state1)
      .def_readwrite("state2", &PyBucketArgs::t_state2)
      .def_readwrite("state3", &PyBucketArgs::t_state3)
      .def_readwrite("shadow", &PyBucketArgs::t_shadow)
      .def_readwrite("grad_ptrs", &PyBucketArgs::t_grad_ptrs)
      .def_readwrite("seg_start", &PyBucketArgs::t_seg_start)
      .def_readwrite("seg_numel", &PyBucketArgs::t_seg_numel)
      .def_readwrite("grad_table_bf16", &PyBucketArgs::grad_table_bf16);

  py::class_<Bucket>(m, "Bucket")
      .def_static("create", [](int64_t numel, const std::string& pub_dtype) {
        const int pe = PubElem(pub_dtype);
        return std::make_unique<Bucket>(MakeIpcChannel(Bucket::PubBytes(numel, pe)), static_cast<uint64_t>(numel), pe);
      })
      .def_static("create_local", [](int world, int64_t numel, const std::string& pub_dtype, int device) {
        const int pe = PubElem(pub_dtype);
        const size_t half = Bucket::PubBytes(numel, pe);
        std::vector<std::shared_ptr<SymmBuffer>> ctrl, arena;
        ThrowIfError(AllocateLocal(world, device, sizeof(ChannelCtrl), &ctrl));
        ThrowIfError(AllocateLocal(world, device, half * 2, &arena));
        std::vector<std::unique_ptr<Bucket>> out;
        for (int r = 0; r < world; ++r)
          out.push_back(std::make_unique<Bucket>(std::make_unique<Channel>(ctrl[r], arena[r], half), static_cast<uint64_t>(numel), pe));
        return out;
      }, py::arg("world"), py::arg("numel"), py::arg("pub_dtype"), py::arg("device") = 0)
      .def("numel", &Bucket::numel)
      .def("versions_published", &Bucket::versions_published)
      .def("set_timeout_ms", [](Bucket& b, double ms) { b.channel()->set_timeout_ms(ms); })
      .def("status", [](Bucket& b) {
        CommStatus s = b.channel()->ReadStatus();
        return py::make_tuple(s.error, s.peer, s.want, s.seen);
      })
      .def("check", [](Bucket& b) { ThrowIfError(b.channel()->StatusToError()); })
      .def("step", [](Bucket& b, PyBucketArgs& a, int64_t stream) {
        auto check = [&](const c10::optional<at::Tensor>& t, const char* what) {
          if (t.has_value() && t->defined()) {
            TORCH_CHECK(t->is_cuda() && t->is_contiguous(), what, " must be a contiguous CUDA tensor");
            TORCH_CHECK(static_cast<uint64_t>(t->numel()) >= b.numel(), what, " is smaller than the bucket");
          }
        };
        check(a.t_master, "master"); check(a.t_grad, "grad"); check(a.t_state1, "state1");
        check(a.t_state2, "state2"); check(a.t_state3, "state3"); check(a.t_shadow, "shadow");
        if (a.t_master.has_value() && a.t_master->defined()) TORCH_CHECK(a.t_master->scalar_type() == at::kFloat, "master must be float32");
        a.BucketStepArgs::master = PtrOrNull(a.t_master);
        a.BucketStepArgs::grad = PtrOrNull(a.t_grad);
        a.BucketStepArgs::state1 = PtrOrNull(a.t_state1);
        a.BucketStepArgs::state2 = PtrOrNull(a.t_state2);
        a.BucketStepArgs::state3 = PtrOrNull(a.t_state3);
        a.BucketStepArgs::shadow = PtrOrNull(a.t_shadow);
        if (a.t_grad.has_value() && a.t_grad->defined()) {
          TORCH_CHECK(a.t_grad->scalar_type() == at::kFloat || a.t_grad->scalar_type() == at::kBFloat16, "grad must be float32 or bfloat16");
          a.grad_elem = a.t_grad->scalar_type() == at::kBFloat16 ? kBF16 : kF32;
        }
        if (a.t_shadow.has_value() && a.t_shadow->defined()) TORCH_CHECK(a.t_shadow->scalar_type() == at::kBFloat16, "shadow must be bfloat16");
        a.BucketStepArgs::grad_ptrs = nullptr;
        a.BucketStepArgs::n_seg = 0;
        if (a.t_grad_ptrs.has_value() && a.t_grad_ptrs->defined()) {
          TORCH_CHECK(!(a.t_grad.has_value() && a.t_grad->defined()), "give either a flat gradient or a gradient table");
          TORCH_CHECK(a.t_seg_start.has_value() && a.t_seg_numel.has_value(), "gradient table needs seg_start and seg_numel");
          for (const at::Tensor* t : {&*a.t_grad_ptrs, &*a.t_seg_start, &*a.t_seg_numel})
            TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kLong && t->is_contiguous() &&
                        t->numel() == a.t_grad_ptrs->numel(), "gradient table tensors must be int64 CUDA tensors of equal length");
          a.BucketStepArgs::grad_ptrs = reinterpret_cast<const void* const*>(a.t_grad_ptrs->data_ptr());
          a.BucketStepArgs::seg_start = reinterpret_cast<const unsigned long long*>(a.t_seg_start->data_ptr());
          a.BucketStepArgs::seg_numel = reinterpret_cast<const unsigned long long*>(a.t_seg_numel->data_ptr());
          a.BucketStepArgs::n_seg = static_cast<int>(a.t_grad_ptrs->numel());
          a.grad_elem = a.grad_table_bf16 ? kBF16 : kF32;
        }
        int device = b.channel()->arena()->device;
        c10::cuda::CUDAGuard g(device);
        cudaStream_t st = stream == 0 ? CurrentStream(device) : reinterpret_cast<cudaStream_t>(stream);
        ThrowIfError(b.Step(a, st));
      }, py::arg("args"), py::arg("stream") = 0);
}
