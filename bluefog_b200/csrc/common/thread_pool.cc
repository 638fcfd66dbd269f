#include "thread_pool.h"

namespace bfb {

void ThreadPool::create(int num_threads) {
  reset();
  stopping_ = false;
  for (int i = 0; i < num_threads; ++i) workers_.emplace_back([this] { loop(); });
}

void ThreadPool::execute(std::function<void()> fn) {
  {
    std::lock_guard<std::mutex> g(mu_);
    if (workers_.empty()) {  // no pool: run inline
      fn();
      return;
    }
    tasks_.push_back(std::move(fn));
  }
  cv_.notify_one();
}

void ThreadPool::loop() {
  for (;;) {
    std::function<void()> fn;
    {
      std::unique_lock<std::mutex> lk(mu_);
      cv_.wait(lk, [this] { return stopping_ || !tasks_.empty(); });
      if (tasks_.empty()) return;  // stopping and drained
      fn = std::move(tasks_.front());
      tasks_.pop_front();
    }
    fn();
  }
}

void ThreadPool::reset() {
  {
    std::lock_guard<std::mutex> g(mu_);
    stopping_ = true;
  }
  cv_.notify_all();
  for (auto& t : workers_)
    if (t.joinable()) t.join();
  workers_.clear();
}

}  // namespace bfb
