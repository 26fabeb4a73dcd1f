#include "common.h"

#include <chrono>
#include <cstdlib>
#include <string>
#include <vector>

#include <pthread.h>
#include <sched.h>

#include "env.h"
#include "logging.h"

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

// HOROVOD_THREAD_AFFINITY is one core for every rank, or one core per local
// rank separated by commas (horovod/common/common.cc:119-200);
// -1 (no pinning) when unset, malformed or too short for this local rank.
int AffinityCore(const std::string& spec, int local_rank) {
  if (spec.empty()) return -1;
  std::vector<std::string> parts;
  size_t at = 0;
  while (true) {
    size_t comma = spec.find(',', at);
    parts.push_back(spec.substr(at, comma == std::string::npos ? comma : comma - at));
    if (comma == std::string::npos) break;
    at = comma + 1;
  }
  const std::string& mine = parts.size() == 1 ? parts[0]
                            : local_rank < static_cast<int>(parts.size()) ? parts[local_rank]
                                                                          : std::string();
  if (mine.empty()) {
    HVD_LOG(WARNING) << HVD_ENV_THREAD_AFFINITY << "=" << spec << " names no core for local rank "
                     << local_rank << "; the background thread is not pinned.";
    return -1;
  }
  char* end = nullptr;
  long core = std::strtol(mine.c_str(), &end, 10);
  if (end == mine.c_str() || *end != '\0' || core < 0) {
    HVD_LOG(WARNING) << HVD_ENV_THREAD_AFFINITY << ": '" << mine << "' is not a core number.";
    return -1;
  }
  return static_cast<int>(core);
}


}  // namespace hvd
