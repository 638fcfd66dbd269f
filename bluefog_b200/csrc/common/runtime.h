// The per-process runtime: operation queue, background scheduling thread, negotiation
// with the coordinator (rank 0), fusion planning, handle table, and the CPU and GPU data
// paths of every collective.
//
// Roles covered (reference files in parentheses): global state (common/global_state.h),
// tensor queue + fusion buffer manager (common/tensor_queue.{h,cc}), background loop,
// negotiation, response construction and validation, stall detection, coordinated
// shutdown and the enqueue API (common/operations.cc:101-1185, 1404-1836), handle manager
// (torch/handle_manager.cc), MPI controller CPU path (common/mpi_controller.cc) and NCCL
// controller GPU path (common/nccl_controller.cc).  The design differs: negotiation is
// event driven over TCP instead of a fixed-period MPI gather/bcast, the GPU path launches
// peer-memory kernels on one high-priority stream and orders work with CUDA events
// instead of host polling, and there is no fusion buffer copy-out: fused tensors are
// published together and combined straight into their outputs.
#pragma once
#include <torch/extension.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <deque>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "control_plane.h"
#include "status.h"
#include "thread_pool.h"
#include "timeline.h"
#include "wire.h"

namespace bfb {

class Channel;
class WindowManager;
struct SymmBuffer;
struct RegisteredLoc;
class SymmRegistry;

// Everything one operation needs; filled by the Python layer after argument validation.
struct OpSpec {
  int type = 0;            // OpType
  std::string name;        // already prefixed, e.g. "neighbor.allreduce.fc1.weight"
  c10::optional<at::Tensor> input;
  c10::optional<at::Tensor> output;
  int root_rank = -1;
  double self_weight = 1.0;
  double post_scale = 1.0;
  std::vector<int> src_ranks;        // ranks whose payload this rank reads
  std::vector<double> src_weights;   // one per src rank
  std::vector<int> dst_ranks;        // ranks that read this rank's payload
  std::vector<double> dst_weights;   // one per dst rank (only used when use_dst_weight)
  bool use_dst_weight = false;
  bool enable_topo_check = false;
  bool is_hierarchical = false;
  bool negotiate = true;             // false for one-sided window transfers
  // window operations
  std::string win_name;
  bool require_mutex = false;
  bool zero_init = false;
  bool accumulate = false;
  std::vector<int> slot_index;       // put/accumulate: my slot at each dst; get: local slot per src
  int num_slots = 0;                 // win_create: slots to allocate (max in-degree over ranks)
  std::vector<int> in_neighbors;     // win_create: in-neighbors of this rank (slot order)
};

class Runtime {
 public:
  static Runtime& Get();

  // -- lifecycle -------------------------------------------------------------------
  Status Listen(const std::string& bind_addr, int* port);
  Status Init(int rank, int size, int local_rank, int local_size, const std::vector<std::string>& endpoints,
              int device);
  void Shutdown();
  bool initialized() const { return initialized_.load(); }
  int rank() const { return rank_; }
  int size() const { return size_; }
  int local_rank() const { return local_rank_; }
  int local_size() const { return local_size_; }
  int device() const { return device_; }
  // Peer-mapped memory that other ranks' kernels may read (bucket arenas and their control blocks): kept mapped
  // until Shutdown has met every other rank at a barrier, whatever the owner object's lifetime.
  void KeepUntilShutdown(std::shared_ptr<void> memory);
  // Collective (every rank, same size): device memory of this rank that is mapped into every rank's address space.
  // A tensor placed in it is published in place by neighbor_allreduce - neighbors pull it from where it is instead
  // of from a copy in the channel arena.  The memory stays allocated until Shutdown.
  Status SymmetricAlloc(size_t bytes, std::shared_ptr<SymmBuffer>* out);
  bool FindRegistered(const void* p, uint64_t nbytes, RegisteredLoc* loc);
  void Suspend() { suspended_.store(true); }
  void Resume() {
    suspended_.store(false);
    Wake();
  }
  void set_skip_negotiate(bool v) { skip_negotiate_.store(v); }
  bool skip_negotiate() const { return skip_negotiate_.load(); }

  // -- operations -------------------------------------------------------------------
  // Returns a handle; the spec's tensors are kept alive until the handle is released.
  int Enqueue(OpSpec spec);
  bool Poll(int handle);
  Status Wait(int handle);   // blocks, then releases the handle
  void Release(int handle);
  // Control-plane barrier on the calling thread (used when negotiation is skipped).
  Status BarrierNow();
  // Collective byte exchange on the calling thread (bootstrap helpers for Python).
  Status AllgatherBytesNow(const std::string& mine, std::vector<std::string>* all);

  // Counters of this rank since init (monotonic; read without stopping anything): operations enqueued per type,
  // payload bytes of their inputs, operations issued on the calling thread, responses executed by the background
  // loop and the tensors fused into them, operations that ended in an error.
  std::map<std::string, uint64_t> StatsSnapshot() const;

  Timeline& timeline() { return timeline_; }
  ControlPlane& control_plane() { return cp_; }
  WindowManager* windows() { return windows_.get(); }
  int64_t fusion_threshold() const { return fusion_threshold_; }
  void set_fusion_threshold(int64_t v) { fusion_threshold_ = v; }
  double cycle_time_ms() const { return cycle_time_ms_; }
  // GPU channel used by the generic collectives (created on first GPU op).
  Channel* gpu_channel() { return gpu_channel_.get(); }
  void* comm_stream() const { return comm_stream_; }
  // Test hooks for failure detection on the host.
  void set_stall_warning_seconds(double s) { stall_warning_s_ = s; }
  std::vector<std::string> StalledTensors();   // rank 0: names waiting for some rank

 private:
  Runtime() = default;
  struct Entry {
    OpSpec spec;
    int handle = -1;
    void* ready_event = nullptr;   // cudaEvent_t recorded on the producer stream at enqueue time
    std::chrono::steady_clock::time_point enqueued;
  };
  struct PendingTensor {           // coordinator-side bookkeeping
    std::vector<Request> requests; // by rank
    std::vector<bool> seen;
    int count = 0;
    std::chrono::steady_clock::time_point first_seen;
  };

  void Loop();
  void Wake();
  void DrainLocalQueue(RequestList* outgoing, std::vector<std::string>* immediate);
  void CoordinatorHandle(const RequestList& list, int from_rank);
  ResponseList CoordinatorBuildResponses();
  Response ConstructResponse(const std::string& name, PendingTensor& pt);
  void ExecuteResponseList(const ResponseList& list);
  void ExecuteResponse(const Response& resp);
  void ExecuteEntries(std::vector<Entry>& entries, const Response& resp);
  Status ExecuteCpu(std::vector<Entry>& entries, const Response& resp);
  Status ExecuteGpu(std::vector<Entry>& entries, const Response& resp);
  Status ExecuteWindowOp(Entry& e);
  Status TopoCheck(const OpSpec& spec);
  Status EnsureGpuChannel(uint64_t need_bytes);
  Status EnsureCommStream();
  // pair_gossip on GPUs: a two-rank channel per partner, set up by the two ranks alone
  Status EnsurePairChannel(int peer, uint64_t need_bytes, Channel** chan);
  Status ExecutePairGossipGpu(Entry& e);
  void FinishEntries(std::vector<Entry>& entries, const Status& s, void* done_event, void* span_start = nullptr);
  // With the timeline on, the device time between span_start and done_event becomes a "DEVICE" span of
  // every tensor of the operation (drawn on its own lane, ending at the moment completion was observed).
  void EmitDeviceSpan(const std::vector<std::string>& names, void* span_start, void* done_event);
  // Fast path: a GPU collective that needs no negotiation and finds nothing queued is issued on the
  // calling thread; its handle completes when the caller waits for (or polls) the completion event.
  bool InlineEligible(const OpSpec& spec) const;
  bool TryRunInline(Entry& e);
  Status CompleteInline(int handle, bool block, bool* finished);
  void FailAll(const Status& s);
  void MarkDone(int handle, const Status& s);
  void CheckStalled();

  // identity
  int rank_ = 0, size_ = 1, local_rank_ = 0, local_size_ = 1, device_ = -1;
  std::atomic<bool> initialized_{false};
  std::atomic<bool> shutdown_requested_{false};
  std::atomic<bool> loop_exited_{false};
  std::atomic<bool> suspended_{false};
  std::atomic<bool> skip_negotiate_{false};
  bool shutdown_sent_ = false;

  ControlPlane cp_;
  std::thread thread_;
  int wake_fd_ = -1;

  // local queue (user threads -> background thread)
  std::mutex queue_mu_;
  std::deque<Entry> queue_;
  std::unordered_map<std::string, Entry> table_;   // entries waiting for a response, by name
  std::mutex table_mu_;

  // handles
  std::mutex handle_mu_;
  std::condition_variable handle_cv_;
  std::unordered_map<int, Status> handles_;
  int next_handle_ = 0;

  // operations issued on the caller's thread and not yet waited for
  struct InlineOp {
    void* done_event = nullptr;                       // cudaEvent_t
    void* span_start = nullptr;                       // cudaEvent_t, only with the timeline on
    std::shared_ptr<std::vector<Entry>> keep;         // tensors stay alive until the kernels are done
  };
  std::mutex exec_mu_;                                // one executor at a time: background loop or a caller
  std::mutex inline_mu_;
  std::mutex keep_mu_;
  std::vector<std::shared_ptr<void>> keep_until_shutdown_;
  static constexpr int kStatOpTypes = 16;
  struct Stats {
    std::atomic<uint64_t> enqueued[kStatOpTypes];
    std::atomic<uint64_t> input_bytes{0}, inline_issued{0}, responses{0}, fused_tensors{0}, errors{0};
    Stats() { for (auto& e : enqueued) e.store(0); }
  };
  Stats stats_;
  std::mutex reg_mu_;
  std::unique_ptr<SymmRegistry> registered_;          // buffers of SymmetricAlloc, in allocation order
  std::unordered_map<int, InlineOp> inline_ops_;      // by handle
  std::unordered_map<std::string, int> inline_names_; // names in flight on the fast path
  bool inline_enabled_ = true;
  static thread_local bool tls_inline_;               // FinishEntries is running for the fast path

  // coordinator state (rank 0)
  std::map<std::string, PendingTensor> message_table_;
  std::deque<std::string> ready_names_;
  bool any_shutdown_ = false;
  std::chrono::steady_clock::time_point last_stall_check_;
  double stall_warning_s_ = 60.0;

  // knobs
  int64_t fusion_threshold_ = 8 * 1024 * 1024;
  double cycle_time_ms_ = 0.5;

  Timeline timeline_;
  ThreadPool finalizers_;
  std::unique_ptr<WindowManager> windows_;

  // GPU path
  std::unique_ptr<Channel> gpu_channel_;
  std::shared_ptr<SymmBuffer> gpu_ctrl_;
  struct PairChannel {
    std::shared_ptr<SymmBuffer> ctrl;
    std::unique_ptr<Channel> chan;
  };
  std::map<int, PairChannel> pair_channels_;   // by partner rank
  std::mutex pair_mu_;                         // guards the map's structure (completion threads walk it)
  // First error recorded by a kernel of any channel (device-side wait limits), or OK.
  Status GpuStatusToError();
  void* comm_stream_ = nullptr;   // cudaStream_t
  std::mutex user_chan_mu_;
};

uint64_t NeighborSignature(const OpSpec& spec);
DataType ToDataType(at::ScalarType t, bool* ok);

}  // namespace bfb
