// Fixed pool of worker threads draining a FIFO of closures. The GPU path
// uses it to wait for completion events off the background thread.
//
// Parity: horovod/common/thread_pool.cc:20-64.
#pragma once

#include <condition_variable>
#include <deque>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

namespace hvd {

class ThreadPool {
public:
  ThreadPool() = default;
  ~ThreadPool() { Shutdown(); }
  void Start(int num_threads);
  void Submit(std::function<void()> fn);
  // Runs everything already queued, then joins the workers.
  void Shutdown();
  bool running() const { return !workers_.empty(); }

private:
  void Loop();
  std::mutex mu_;
  std::condition_variable cv_;
  std::deque<std::function<void()>> work_;
  std::vector<std::thread> workers_;
  bool stop_ = false;
};

}  // namespace hvd
