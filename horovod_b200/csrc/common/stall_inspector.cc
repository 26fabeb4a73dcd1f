#include "stall_inspector.h"

#include <algorithm>
#include <sstream>

#include "logging.h"
#include "response_cache.h"

namespace hvd {

bool StallInspector::ShouldPerformCheck() const {
  if (!enabled_) return false;
  // Check once per warning period (every 100 ms when the period is under a
  // second, which only tests use).
  auto period = warning_s_ >= 1
                    ? std::chrono::milliseconds(1000LL * warning_s_)
                    : std::chrono::milliseconds(100);
  return Clock::now() - last_check_ > period;
}

void StallInspector::UpdateCheckTime() { last_check_ = Clock::now(); }

bool StallInspector::CheckForStalledTensors(
    const std::vector<int>& global_ranks) {
  bool should_shut_down = false;
  auto now = Clock::now();
  std::ostringstream msg;
  bool any = false;
  for (auto& kv : uncached_) {
    auto waited =
        std::chrono::duration_cast<std::chrono::seconds>(now - kv.second.start)
            .count();
    if (waited <= warning_s_) continue;
    if (!any) {
      msg << "One or more tensors were submitted to be reduced, gathered or "
             "broadcasted by subset of ranks and are waiting for remainder of "
             "ranks for more than "
          << warning_s_
          << " seconds. This may indicate that different ranks are trying to "
             "submit different tensors or that only subset of ranks is "
             "submitting tensors, which will cause deadlock.\n"
             "Missing ranks:";
      any = true;
    }
    // Group by rank: "rank: [tensor, ...]".
    msg << "\n  " << kv.first << " waiting " << waited << " s for rank(s) [";
    bool first = true;
    for (size_t r = 0; r < kv.second.seen.size(); ++r) {
      if (kv.second.seen[r]) continue;
      if (!first) msg << ", ";
      first = false;
      msg << (r < global_ranks.size() ? global_ranks[r] : static_cast<int>(r));
    }
    msg << "]";
    if (shutdown_s_ > 0 && waited > shutdown_s_) should_shut_down = true;
  }
  if (any) {
    last_report_ = msg.str();
    HVD_LOG(WARNING) << last_report_;
    if (should_shut_down) {
      HVD_LOG(ERROR) << "Stalled ranks exceeded the shutdown time of "
                     << shutdown_s_ << " s: shutting the job down.";
    }
  }
  return should_shut_down;
}

void StallInspector::RecordUncachedTensorStart(const std::string& name,
                                               int rank, int size) {
  auto it = uncached_.find(name);
  if (it == uncached_.end()) {
    Uncached u;
    u.start = Clock::now();
    u.seen.assign(size, false);
    it = uncached_.emplace(name, std::move(u)).first;
  }
  if (rank >= 0 && rank < static_cast<int>(it->second.seen.size()))
    it->second.seen[rank] = true;
}

void StallInspector::RemoveUncachedTensor(const std::string& name) {
  uncached_.erase(name);
}

void StallInspector::RecordCachedTensorStart(const std::string& name) {
  if (!enabled_) return;
  cached_.emplace(name, Clock::now());  // keeps the first time seen
}

void StallInspector::RemoveCachedTensor(const std::string& name) {
  if (!cached_.empty()) cached_.erase(name);
}

void StallInspector::InvalidateStalledCachedTensors(
    CacheCoordinator& coordinator) {
  auto now = Clock::now();
  for (auto& kv : cached_) {
    auto waited =
        std::chrono::duration_cast<std::chrono::seconds>(now - kv.second)
            .count();
    if (waited > warning_s_ && cache_.has_name(kv.first)) {
      uint32_t bit = cache_.peek_cache_bit(kv.first);
      coordinator.record_invalid_bit(bit);
      coordinator.set_uncached_in_queue(true);
    }
  }
}

}  // namespace hvd
