// Fixed-size worker pool. The runtime uses it as the "finalizer" pool that waits
// on CUDA completion events and fires handle callbacks off the scheduling thread
// (role of bluefog/common/thread_pool.h:27-41 in the reference).
#pragma once
#include <condition_variable>
#include <deque>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

namespace bfb {

class ThreadPool {
 public:
  ThreadPool() = default;
  ~ThreadPool() { reset(); }
  void create(int num_threads);
  void execute(std::function<void()> fn);
  // Drains the queue, joins the workers; the pool can be create()d again.
  void reset();
  int size() const { return static_cast<int>(workers_.size()); }

 private:
  void loop();
  std::vector<std::thread> workers_;
  std::deque<std::function<void()>> tasks_;
  std::mutex mu_;
  std::condition_variable cv_;
  bool stopping_ = false;
};

}  // namespace bfb
