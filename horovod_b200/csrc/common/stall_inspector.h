// Detects collectives that some ranks submitted and others did not.
// The coordinator remembers, per uncached tensor, which ranks have asked and
// when the first one did; past the warning time it logs the missing ranks,
// past the (optional) shutdown time it asks the job to stop. Cached tensors
// that wait too long are invalidated so they go back through the
// coordinator, which can then name the missing ranks.
//
// Parity: horovod/common/stall_inspector.h:30-99, stall_inspector.cc:26-185.
#pragma once

#include <chrono>
#include <string>
#include <unordered_map>
#include <vector>

namespace hvd {

class ResponseCache;
class CacheCoordinator;

class StallInspector {
public:
  explicit StallInspector(ResponseCache& cache) : cache_(cache) {}

  void SetPerformStallCheck(bool v) { enabled_ = v; }
  void SetStallWarningTimeSeconds(int s) { warning_s_ = s; }
  void SetStallShutdownTimeSeconds(int s) { shutdown_s_ = s; }
  int warning_seconds() const { return warning_s_; }
  int shutdown_seconds() const { return shutdown_s_; }

  bool ShouldPerformCheck() const;
  void UpdateCheckTime();

  // Coordinator only. Returns true if the job should shut down.
  // `global_ranks` maps process-set ranks to global ranks for the message.
  bool CheckForStalledTensors(const std::vector<int>& global_ranks);
  void RecordUncachedTensorStart(const std::string& name, int rank, int size);
  void RemoveUncachedTensor(const std::string& name);

  // Every rank.
  void RecordCachedTensorStart(const std::string& name);
  void RemoveCachedTensor(const std::string& name);
  void InvalidateStalledCachedTensors(CacheCoordinator& coordinator);

  // Text of the most recent stall warning (for tests and diagnostics).
  const std::string& last_report() const { return last_report_; }

private:
  using Clock = std::chrono::steady_clock;
  struct Uncached {
    Clock::time_point start;
    std::vector<bool> seen;
  };
  ResponseCache& cache_;
  bool enabled_ = true;
  int warning_s_ = 60;
  int shutdown_s_ = 0;
  Clock::time_point last_check_ = Clock::now();
  std::unordered_map<std::string, Uncached> uncached_;
  std::unordered_map<std::string, Clock::time_point> cached_;
  std::string last_report_;
};

}  // namespace hvd
