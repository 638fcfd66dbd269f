#include "timeline.h"

#include <functional>

#include "logging.h"

namespace bfb {

Timeline::~Timeline() { Shutdown(); }

bool Timeline::Initialize(const std::string& file_name, int /*world_size*/) {
  if (Initialized()) return true;
  file_.open(file_name, std::ios::out | std::ios::trunc);
  if (!file_.good()) {
    BFLOG(ERROR) << "Error opening the timeline file " << file_name << ", will not write a timeline.";
    return false;
  }
  file_ << "[\n";
  start_ = std::chrono::steady_clock::now();
  stop_ = false;
  writer_ = std::thread([this] { WriterLoop(); });
  initialized_.store(true, std::memory_order_release);
  return true;
}

void Timeline::Shutdown() {
  if (!Initialized()) return;
  initialized_.store(false, std::memory_order_release);
  {
    std::lock_guard<std::mutex> g(q_mu_);
    stop_ = true;
  }
  q_cv_.notify_all();
  if (writer_.joinable()) writer_.join();
  file_.flush();
  file_.close();
  tensor_pid_.clear();
  tid_index_.clear();
  depth_.clear();
}

long Timeline::NowMicros() const {
  return static_cast<long>(std::chrono::duration_cast<std::chrono::microseconds>(
                               std::chrono::steady_clock::now() - start_)
                               .count());
}

long Timeline::ThisThreadId() {
  return static_cast<long>(std::hash<std::thread::id>()(std::this_thread::get_id()) & 0x7fffffff);
}

void Timeline::Push(Record&& r) {
  {
    std::lock_guard<std::mutex> g(q_mu_);
    pending_.push_back(std::move(r));
  }
  q_cv_.notify_one();
}

void Timeline::ActivityStart(const std::string& tensor_name, const std::string& activity, long tid) {
  if (!Initialized()) return;
  {
    std::lock_guard<std::mutex> g(state_mu_);
    depth_[tensor_name] += 1;
  }
  Push(Record{tensor_name, activity, 'B', tid < 0 ? ThisThreadId() : tid, NowMicros()});
}

void Timeline::ActivityEnd(const std::string& tensor_name, long tid) {
  if (!Initialized()) return;
  {
    std::lock_guard<std::mutex> g(state_mu_);
    auto it = depth_.find(tensor_name);
    if (it == depth_.end() || it->second <= 0) return;  // unmatched end: ignore
    it->second -= 1;
  }
  Push(Record{tensor_name, "", 'E', tid < 0 ? ThisThreadId() : tid, NowMicros()});
}

void Timeline::ActivityStartAll(const std::vector<std::string>& names, const std::string& activity) {
  for (const auto& n : names) ActivityStart(n, activity);
}

void Timeline::ActivityEndAll(const std::vector<std::string>& names) {
  for (const auto& n : names) ActivityEnd(n);
}

void Timeline::CompleteSpan(const std::string& tensor_name, const std::string& activity,
                            long ts_begin_us, long ts_end_us, long lane) {
  if (!Initialized()) return;
  Push(Record{tensor_name, activity, 'B', lane, ts_begin_us});
  Push(Record{tensor_name, "", 'E', lane, ts_end_us < ts_begin_us ? ts_begin_us : ts_end_us});
}

int Timeline::Depth(const std::string& tensor_name) {
  std::lock_guard<std::mutex> g(state_mu_);
  auto it = depth_.find(tensor_name);
  return it == depth_.end() ? 0 : it->second;
}

static std::string JsonEscape(const std::string& s) {
  std::string out;
  out.reserve(s.size());
  for (char c : s) {
    if (c == '"' || c == '\\') {
      out.push_back('\\');
      out.push_back(c);
    } else if (static_cast<unsigned char>(c) < 0x20) {
      out.push_back(' ');
    } else {
      out.push_back(c);
    }
  }
  return out;
}

void Timeline::WriteRecord(const Record& r) {
  int& tid = tid_index_[r.tid];
  if (tid == 0) tid = static_cast<int>(tid_index_.size());
  int& pid = tensor_pid_[r.tensor];
  StrBuilder out;  // numbers are formatted without iostream facets
  if (pid == 0) {
    pid = static_cast<int>(tensor_pid_.size());
    out << "{\"name\": \"process_name\", \"ph\": \"M\", \"pid\": " << pid << ", \"tid\": " << tid
        << ", \"args\": {\"name\": \"" << JsonEscape(r.tensor) << "\"}},\n";
    out << "{\"name\": \"process_sort_index\", \"ph\": \"M\", \"pid\": " << pid << ", \"tid\": " << tid
        << ", \"args\": {\"sort_index\": " << pid << "}},\n";
  }
  out << "{\"ph\": \"" << r.phase << "\"";
  if (r.phase != 'E') out << ", \"name\": \"" << JsonEscape(r.op) << "\"";
  out << ", \"ts\": " << r.ts << ", \"pid\": " << pid << ", \"tid\": " << tid << "},\n";
  file_.write(out.str().data(), static_cast<std::streamsize>(out.str().size()));
}

void Timeline::WriterLoop() {
  std::vector<Record> batch;
  for (;;) {
    {
      std::unique_lock<std::mutex> lk(q_mu_);
      q_cv_.wait(lk, [this] { return stop_ || !pending_.empty(); });
      batch.swap(pending_);
      if (batch.empty() && stop_) break;
    }
    for (const auto& r : batch) WriteRecord(r);
    batch.clear();
    file_.flush();
    if (!file_.good()) {
      BFLOG(ERROR) << "Error writing to the timeline file; timeline stops.";
      break;
    }
  }
}

}  // namespace bfb
