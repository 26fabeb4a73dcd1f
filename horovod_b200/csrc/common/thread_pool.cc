#include "thread_pool.h"

namespace hvd {

void ThreadPool::Start(int num_threads) {
  std::lock_guard<std::mutex> l(mu_);
  if (!workers_.empty()) return;
  stop_ = false;
  for (int i = 0; i < num_threads; ++i)
    workers_.emplace_back([this] { Loop(); });
}

void ThreadPool::Submit(std::function<void()> fn) {
  {
    std::lock_guard<std::mutex> l(mu_);
    work_.push_back(std::move(fn));
  }
  cv_.notify_one();
}

void ThreadPool::Shutdown() {
  {
    std::lock_guard<std::mutex> l(mu_);
    if (workers_.empty()) return;
    stop_ = true;
  }
  cv_.notify_all();
  for (auto& t : workers_) t.join();
  workers_.clear();
}

void ThreadPool::Loop() {
  for (;;) {
    std::function<void()> fn;
    {
      std::unique_lock<std::mutex> l(mu_);
      cv_.wait(l, [this] { return stop_ || !work_.empty(); });
      if (work_.empty()) return;  // stop_ set and queue drained
      fn = std::move(work_.front());
      work_.pop_front();
    }
    fn();
  }
}

}  // namespace hvd
