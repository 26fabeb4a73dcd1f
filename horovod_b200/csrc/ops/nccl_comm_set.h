// The NCCL communicators of one executor, and what elastic jobs need from
// them: while the host waits for a collective, ask every communicator for an
// asynchronous error (a peer that died, a failed link) and, on the first one,
// abort them all so that the kernels stuck in them return and the wait ends
// with an error instead of never.
//
// Parity: horovod/common/ops/nccl_operations.cc:109-122 (ErrorCheck /
// AbortComm on ncclCommGetAsyncError) and horovod/common/ops/
// cuda_operations.cc:102-148 (event polling with that check in elastic mode).
#pragma once

#include <chrono>
#include <cstdint>
#include <map>
#include <mutex>
#include <thread>

#include "../common/common.h"

namespace hvd {

struct NcclApi;

class NcclCommSet {
public:
  explicit NcclCommSet(const NcclApi* api = nullptr) : api_(api) {}
  void set_api(const NcclApi* api) { api_ = api; }

  void* Find(int32_t key);
  void Put(int32_t key, void* comm);
  bool empty();
  // True once CheckAsyncErrors() has aborted the communicators; cleared by
  // DestroyAll() (shutdown, elastic reset).
  bool failed();
  // OK, or the first asynchronous error; then every communicator has been
  // aborted and the set is empty and marked failed.
  Status CheckAsyncErrors();
  void DestroyAll();
  // Held by the thread that issues NCCL calls for the duration of one
  // response, and by CheckAsyncErrors() while it aborts: no call is issued
  // on a communicator that is being torn down.
  std::mutex& issue_mutex() { return issue_mu_; }

private:
  const NcclApi* api_;
  std::mutex mu_;        // comms_, failed_
  std::mutex issue_mu_;
  std::map<int32_t, void*> comms_;
  bool failed_ = false;
};

// Waits for `ready()` (1 = done, 0 = not yet, negative = the query failed)
// and calls `check()` between polls. When `check()` reports an error (having
// unblocked the device work), the wait goes on for at most `grace` so that
// the work can drain, and that error is returned.
template <class Ready, class Check>
Status WaitPolling(Ready ready, Check check, std::chrono::microseconds pause,
                   std::chrono::milliseconds grace) {
  while (true) {
    int r = ready();
    if (r > 0) return Status::OK();
    if (r < 0) return Status::UnknownError("the completion query failed");
    Status st = check();
    if (!st.ok()) {
      auto until = std::chrono::steady_clock::now() + grace;
      while (ready() == 0 && std::chrono::steady_clock::now() < until)
        std::this_thread::sleep_for(pause);
      return st;
    }
    std::this_thread::sleep_for(pause);
  }
}

}  // namespace hvd
