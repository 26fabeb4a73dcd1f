#include "parameter_manager.h"

#include <algorithm>

#include "logging.h"

namespace hvd {

namespace {
constexpr int SAMPLES_PER_SETTING = 5;
constexpr double MAX_FUSION_MB = 256.0;  // HBM3e makes big buffers cheap
constexpr double MAX_CYCLE_MS = 100.0;
}  // namespace

ParameterManager::ParameterManager() {
  cache_enabled_.value = true;
  seeds_ = {{4, 5}, {32, 50}, {16, 25}, {8, 10}};
}

void ParameterManager::Initialize(int rank, int root_rank,
                                  const std::string& log_file) {
  rank_ = rank;
  root_rank_ = root_rank;
  if (rank_ == root_rank_ && !log_file.empty()) {
    log_.open(log_file, std::ios::out | std::ios::trunc);
    if (log_.good())
      log_ << "hierarchical_allreduce,hierarchical_allgather,cache_enabled,"
              "cycle_time_ms,tensor_fusion_threshold,score\n";
  }
}

void ParameterManager::SetAutoTuning(bool active) {
  active_ = active;
  if (!active) return;
  warmup_left_ = warmups_;
  categorical_order_.clear();
  for (Categorical* c : {&hier_allreduce_, &hier_allgather_, &cache_enabled_}) {
    if (!c->fixed) categorical_order_.push_back(c);
    c->done = c->fixed;
    c->tried = 0;
    c->best_score = -1;
  }
  categorical_index_ = 0;
  numeric_done_ = fusion_fixed_ && cycle_fixed_;
  if (!numeric_done_) {
    std::vector<std::pair<double, double>> bounds;
    if (!fusion_fixed_) bounds.emplace_back(0.0, MAX_FUSION_MB);
    if (!cycle_fixed_) bounds.emplace_back(1.0, MAX_CYCLE_MS);
    bayes_.reset(new BayesianOptimization(bounds, gp_noise_));
  }
  seed_index_ = 0;
  bayes_samples_ = 0;
  steps_ = 0;
  bytes_ = 0;
  scores_.clear();
  seen_this_step_.clear();
  sample_start_ = std::chrono::steady_clock::now();
}

void ParameterManager::SetHierarchicalAllreduce(bool v, bool fixed) {
  hier_allreduce_.value = v;
  hier_allreduce_.fixed = fixed;
}
void ParameterManager::SetHierarchicalAllgather(bool v, bool fixed) {
  hier_allgather_.value = v;
  hier_allgather_.fixed = fixed;
}
void ParameterManager::SetCacheEnabled(bool v, bool fixed) {
  cache_enabled_.value = v;
  cache_enabled_.fixed = fixed;
}
void ParameterManager::SetTensorFusionThresholdBytes(int64_t v, bool fixed) {
  fusion_bytes_ = static_cast<double>(v);
  fusion_fixed_ = fixed;
}
void ParameterManager::SetCycleTimeMs(double v, bool fixed) {
  cycle_ms_ = v;
  cycle_fixed_ = fixed;
}

ParameterManager::Params ParameterManager::GetParams() const {
  Params p;
  p.hierarchical_allreduce = hier_allreduce_.value;
  p.hierarchical_allgather = hier_allgather_.value;
  p.cache_enabled = cache_enabled_.value;
  p.active = active_;
  p.fusion_threshold_bytes = fusion_bytes_;
  p.cycle_time_ms = cycle_ms_;
  return p;
}

void ParameterManager::SetParams(const Params& p) {
  hier_allreduce_.value = p.hierarchical_allreduce != 0;
  hier_allgather_.value = p.hierarchical_allgather != 0;
  cache_enabled_.value = p.cache_enabled != 0;
  fusion_bytes_ = p.fusion_threshold_bytes;
  cycle_ms_ = p.cycle_time_ms;
  active_ = p.active != 0;
}

bool ParameterManager::Update(const std::vector<std::string>& tensor_names,
                              int64_t bytes) {
  if (!active_) return false;
  // Every rank runs the same count-based bookkeeping (tensor names are the
  // same everywhere), so all ranks agree on when a sample completes and can
  // enter the parameter broadcast together; only the root scores and tunes.
  // A tensor name coming round again marks the start of the next step.
  bool new_step = false;
  for (auto& n : tensor_names) {
    if (seen_this_step_.count(n)) {
      new_step = true;
      break;
    }
  }
  if (new_step) {
    seen_this_step_.clear();
    ++steps_;
  }
  for (auto& n : tensor_names) seen_this_step_.insert(n);
  bytes_ += bytes;
  if (steps_ < steps_per_sample_) return false;

  auto now = std::chrono::steady_clock::now();
  double us = std::chrono::duration<double, std::micro>(now - sample_start_).count();
  double score = us > 0 ? static_cast<double>(bytes_) / us : 0.0;
  steps_ = 0;
  bytes_ = 0;
  sample_start_ = now;
  if (warmup_left_ > 0) {
    --warmup_left_;
    return false;
  }
  scores_.push_back(score);
  if (static_cast<int>(scores_.size()) < SAMPLES_PER_SETTING) return false;
  std::sort(scores_.begin(), scores_.end());
  double median = scores_[scores_.size() / 2];
  scores_.clear();
  ++total_samples_;
  // The next setting gets its own warm-up. Every rank resets it here (not in
  // Tune(), which only the root runs) so that the sample boundaries, and with
  // them the parameter broadcasts, stay aligned across ranks.
  warmup_left_ = warmups_;
  if (rank_ == root_rank_) Tune(median);
  return true;
}

void ParameterManager::LogSample(double score) {
  if (log_.good() && log_.is_open()) {
    log_ << hier_allreduce_.value << "," << hier_allgather_.value << ","
         << cache_enabled_.value << "," << cycle_ms_ << ","
         << static_cast<int64_t>(fusion_bytes_) << "," << score << std::endl;
  }
  HVD_LOG(INFO) << "Autotune: [hier_allreduce=" << hier_allreduce_.value
                << " hier_allgather=" << hier_allgather_.value
                << " cache=" << cache_enabled_.value
                << " cycle_ms=" << cycle_ms_
                << " fusion_bytes=" << static_cast<int64_t>(fusion_bytes_)
                << "] score " << score << " bytes/us";
}

bool ParameterManager::Tune(double score) {
  LogSample(score);
  if (categorical_index_ < categorical_order_.size())
    return NextCategorical(score);
  if (!numeric_done_) return NextNumeric(score);
  return false;
}

bool ParameterManager::NextCategorical(double score) {
  Categorical* c = categorical_order_[categorical_index_];
  if (score > c->best_score) {
    c->best_score = score;
    c->best = c->value;
  }
  ++c->tried;
  if (c->tried < 2) {
    c->value = !c->value;  // measure the other setting
    return true;
  }
  c->value = c->best;
  c->done = true;
  ++categorical_index_;
  if (categorical_index_ < categorical_order_.size()) {
    // The next categorical starts from its current value; nothing changes
    // until its second trial unless the best flipped back.
    return true;
  }
  if (numeric_done_) {
    active_ = false;
    return true;
  }
  // Move on to the joint numeric search with the first seed point.
  ApplyNumeric(seeds_[seed_index_]);
  return true;
}

void ParameterManager::ApplyNumeric(const std::vector<double>& seed) {
  // Seeds are (fusion MB, cycle ms) pairs; a fixed knob keeps its value.
  if (!fusion_fixed_) fusion_bytes_ = seed[0] * 1024.0 * 1024.0;
  if (!cycle_fixed_) cycle_ms_ = seed[1];
}

bool ParameterManager::NextNumeric(double score) {
  std::vector<double> x;
  if (!fusion_fixed_) x.push_back(fusion_bytes_ / (1024.0 * 1024.0));
  if (!cycle_fixed_) x.push_back(cycle_ms_);
  // The first numeric sample measured whatever was configured when the
  // categorical phase ended (a seed if there was one to apply).
  bayes_->AddSample(x, score);
  ++bayes_samples_;
  if (bayes_samples_ >= max_bayes_samples_) {
    std::vector<double> best = bayes_->best_x();
    size_t i = 0;
    if (!fusion_fixed_) fusion_bytes_ = best[i++] * 1024.0 * 1024.0;
    if (!cycle_fixed_) cycle_ms_ = best[i++];
    numeric_done_ = true;
    active_ = false;
    HVD_LOG(INFO) << "Autotune finished: fusion_bytes="
                  << static_cast<int64_t>(fusion_bytes_)
                  << " cycle_ms=" << cycle_ms_ << " best score "
                  << bayes_->best_y();
    LogSample(bayes_->best_y());
    return true;
  }
  std::vector<double> next;
  if (++seed_index_ < seeds_.size()) {
    const auto& s = seeds_[seed_index_];
    if (!fusion_fixed_) next.push_back(s[0]);
    if (!cycle_fixed_) next.push_back(s[1]);
  } else {
    next = bayes_->NextSample();
  }
  size_t i = 0;
  if (!fusion_fixed_) fusion_bytes_ = next[i++] * 1024.0 * 1024.0;
  if (!cycle_fixed_) cycle_ms_ = next[i++];
  return true;
}

}  // namespace hvd
