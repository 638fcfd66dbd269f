// Chrome-tracing ("chrome://tracing" / Perfetto JSON array) timeline writer.
//
// Public behaviour follows the reference (bluefog/common/timeline.h:37-122,
// timeline.cc:45-141): one file per rank named <prefix><rank>.json, each tensor is
// modelled as a trace "process" (pid) with process_name/process_sort_index metadata,
// host threads are "tid"s, activities are B/E pairs.  The implementation is our own:
// producers append fixed records to a double-buffered vector under a short mutex and a
// writer thread swaps and drains it, so no event is ever dropped or spun on, and
// activities may nest (a depth counter per tensor instead of a two-state machine).
// Device-side spans measured with CUDA events are added with CompleteSpan().
#pragma once
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <fstream>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

namespace bfb {

class Timeline {
 public:
  Timeline() = default;
  ~Timeline();
  // Opens the file and starts the writer thread. Returns false if the file cannot be opened.
  bool Initialize(const std::string& file_name, int world_size);
  bool Initialized() const { return initialized_.load(std::memory_order_acquire); }
  void Shutdown();

  void ActivityStart(const std::string& tensor_name, const std::string& activity, long tid = -1);
  void ActivityEnd(const std::string& tensor_name, long tid = -1);
  void ActivityStartAll(const std::vector<std::string>& names, const std::string& activity);
  void ActivityEndAll(const std::vector<std::string>& names);
  // A finished span with explicit timestamps (microseconds since Initialize), e.g. a kernel
  // timed with CUDA events.  lane selects the "tid" row it is drawn on.
  void CompleteSpan(const std::string& tensor_name, const std::string& activity, long ts_begin_us,
                    long ts_end_us, long lane);
  long NowMicros() const;
  // Number of activities currently open for a tensor (0 = top level).
  int Depth(const std::string& tensor_name);

 private:
  struct Record {
    std::string tensor;
    std::string op;
    char phase;
    long tid;
    long ts;
  };
  void Push(Record&& r);
  void WriterLoop();
  void WriteRecord(const Record& r);
  static long ThisThreadId();

  std::atomic<bool> initialized_{false};
  std::chrono::steady_clock::time_point start_;
  std::mutex state_mu_;
  std::unordered_map<std::string, int> depth_;

  std::mutex q_mu_;
  std::condition_variable q_cv_;
  std::vector<Record> pending_;
  bool stop_ = false;
  std::thread writer_;

  // writer-thread only
  std::ofstream file_;
  std::unordered_map<std::string, int> tensor_pid_;
  std::unordered_map<long, int> tid_index_;
};

}  // namespace bfb
