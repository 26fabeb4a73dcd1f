// Online autotuner for the knobs that shape throughput: response cache
// on/off (categorical), fusion threshold and cycle time (tuned jointly by
// Bayesian optimisation), plus the hierarchical flags kept for multi-node
// jobs. The coordinator scores each setting as bytes processed per
// microsecond, then broadcasts the winning values.
//
// Parity: horovod/common/parameter_manager.h:42-246, parameter_manager.cc
// :28-528 (warm-ups 3, 10 steps per sample, median of 5 samples, at most 20
// Bayesian samples, seeds (4,5),(32,50),(16,25),(8,10); explicitly set knobs
// are fixed and left out of the search).
#pragma once

#include <chrono>
#include <cstdint>
#include <fstream>
#include <memory>
#include <string>
#include <unordered_set>
#include <vector>

#include "optim/bayesian_optimization.h"

namespace hvd {

class ParameterManager {
public:
  // Plain-old-data snapshot broadcast from the coordinator.
  struct Params {
    uint8_t hierarchical_allreduce;
    uint8_t hierarchical_allgather;
    uint8_t cache_enabled;
    uint8_t active;
    double fusion_threshold_bytes;
    double cycle_time_ms;
  };

  ParameterManager();

  void Initialize(int rank, int root_rank, const std::string& log_file);
  void SetAutoTuning(bool active);
  bool IsAutoTuning() const { return active_; }

  void SetWarmupSamples(int n) { warmups_ = n; }
  void SetStepsPerSample(int n) { steps_per_sample_ = n; }
  void SetBayesOptMaxSamples(int n) { max_bayes_samples_ = n; }
  void SetGaussianProcessNoise(double a) { gp_noise_ = a; }

  // fixed = the user set it explicitly, so it is not tuned.
  void SetHierarchicalAllreduce(bool v, bool fixed = false);
  void SetHierarchicalAllgather(bool v, bool fixed = false);
  void SetCacheEnabled(bool v, bool fixed = false);
  void SetTensorFusionThresholdBytes(int64_t v, bool fixed = false);
  void SetCycleTimeMs(double v, bool fixed = false);

  bool HierarchicalAllreduce() const { return hier_allreduce_.value; }
  bool HierarchicalAllgather() const { return hier_allgather_.value; }
  bool CacheEnabled() const { return cache_enabled_.value; }
  int64_t TensorFusionThresholdBytes() const {
    return static_cast<int64_t>(fusion_bytes_);
  }
  double CycleTimeMs() const { return cycle_ms_; }

  // Called once per cycle with the tensors just processed. Returns true
  // when the parameters changed and must be re-broadcast.
  bool Update(const std::vector<std::string>& tensor_names, int64_t bytes);

  Params GetParams() const;
  void SetParams(const Params& p);

  // Search state, exposed for tests.
  int samples_taken() const { return total_samples_; }

private:
  struct Categorical {
    bool value = false;
    bool fixed = false;
    bool best = false;
    double best_score = -1;
    bool done = false;
    int tried = 0;
  };
  bool Tune(double score);
  bool NextCategorical(double score);
  bool NextNumeric(double score);
  void ApplyNumeric(const std::vector<double>& x);
  void LogSample(double score);

  bool active_ = false;
  int rank_ = 0, root_rank_ = 0;
  int warmups_ = 3, steps_per_sample_ = 10, max_bayes_samples_ = 20;
  double gp_noise_ = 0.8;
  int warmup_left_ = 3;

  Categorical hier_allreduce_, hier_allgather_, cache_enabled_;
  std::vector<Categorical*> categorical_order_;
  size_t categorical_index_ = 0;

  double fusion_bytes_ = 128.0 * 1024 * 1024;
  double cycle_ms_ = 1.0;
  bool fusion_fixed_ = false, cycle_fixed_ = false;
  std::unique_ptr<BayesianOptimization> bayes_;
  std::vector<std::vector<double>> seeds_;
  size_t seed_index_ = 0;
  int bayes_samples_ = 0;
  bool numeric_done_ = false;

  // Current measurement.
  std::unordered_set<std::string> seen_this_step_;
  int steps_ = 0;
  int64_t bytes_ = 0;
  std::chrono::steady_clock::time_point sample_start_;
  std::vector<double> scores_;  // up to 5, median taken
  int total_samples_ = 0;

  std::ofstream log_;
};

}  // namespace hvd
