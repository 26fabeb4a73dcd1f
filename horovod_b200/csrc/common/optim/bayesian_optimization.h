// Bayesian optimisation of a noisy black-box score over a box-bounded
// continuous domain: Gaussian-process surrogate + expected improvement.
//
// Parity: horovod/common/optim/bayesian_optimization.cc:66-182 (EI with
// xi = 0.01, random restarts). The acquisition is maximised here by
// multi-start pattern search instead of L-BFGS.
#pragma once

#include <cstdint>
#include <random>
#include <utility>
#include <vector>

#include "gaussian_process.h"

namespace hvd {

class BayesianOptimization {
public:
  // bounds[i] = (low, high) of dimension i; alpha = GP noise; xi = EI
  // exploration margin.
  BayesianOptimization(std::vector<std::pair<double, double>> bounds,
                       double alpha, double xi = 0.01, uint64_t seed = 0);

  void AddSample(const std::vector<double>& x, double y);
  // Point with the highest expected improvement over the best sample so far.
  std::vector<double> NextSample();
  void Clear();
  size_t num_samples() const { return y_.size(); }
  const std::vector<double>& best_x() const { return best_x_; }
  double best_y() const { return best_y_; }

  // Expected improvement at a normalised point (exposed for tests).
  double ExpectedImprovement(const std::vector<double>& unit_x) const;

private:
  std::vector<double> Normalise(const std::vector<double>& x) const;
  std::vector<double> Denormalise(const std::vector<double>& u) const;

  std::vector<std::pair<double, double>> bounds_;
  double alpha_;
  double xi_;
  std::mt19937_64 rng_;
  std::vector<std::vector<double>> x_;  // normalised to [0,1]^d
  std::vector<double> y_;               // raw scores
  double y_scale_ = 1.0;
  std::vector<double> best_x_;
  double best_y_ = 0.0;
  GaussianProcess gp_;
};

}  // namespace hvd
