#include "common.h"

#include <chrono>

#include <pthread.h>
#include <sched.h>

namespace hvd {

const char* const SHUT_DOWN_ERROR_MESSAGE =
    "Horovod has been shut down. This was caused by an exception on one of "
    "the ranks or an attempt to run a collective after one of the ranks "
    "finished execution. If the shutdown was caused by an exception, you "
    "should see the exception in the log before the first shutdown message.";

const char* const DUPLICATE_NAME_ERROR_MESSAGE =
    "Requested to run a collective on a tensor name that is already pending: "
    "a name may be in flight only once. Pass distinct names, or wait for the "
    "earlier operation to finish.";

int64_t NowMicros() {
  return std::chrono::duration_cast<std::chrono::microseconds>(
             std::chrono::steady_clock::now().time_since_epoch())
      .count();
}

void SetThreadAffinity(int core) {
  if (core < 0) return;
  cpu_set_t set;
  CPU_ZERO(&set);
  CPU_SET(core, &set);
  pthread_setaffinity_np(pthread_self(), sizeof(set), &set);
}

}  // namespace hvd
