#include "bayesian_optimization.h"

#include <algorithm>
#include <cmath>

namespace hvd {

namespace {
double NormPdf(double z) { return std::exp(-0.5 * z * z) / std::sqrt(2 * M_PI); }
double NormCdf(double z) { return 0.5 * std::erfc(-z / std::sqrt(2.0)); }
}  // namespace

BayesianOptimization::BayesianOptimization(
    std::vector<std::pair<double, double>> bounds, double alpha, double xi,
    uint64_t seed)
    : bounds_(std::move(bounds)), alpha_(alpha), xi_(xi), rng_(seed),
      gp_(alpha) {}

std::vector<double> BayesianOptimization::Normalise(
    const std::vector<double>& x) const {
  std::vector<double> u(x.size());
  for (size_t i = 0; i < x.size(); ++i) {
    double span = bounds_[i].second - bounds_[i].first;
    u[i] = span > 0 ? (x[i] - bounds_[i].first) / span : 0.0;
  }
  return u;
}

std::vector<double> BayesianOptimization::Denormalise(
    const std::vector<double>& u) const {
  std::vector<double> x(u.size());
  for (size_t i = 0; i < u.size(); ++i)
    x[i] = bounds_[i].first + u[i] * (bounds_[i].second - bounds_[i].first);
  return x;
}

void BayesianOptimization::AddSample(const std::vector<double>& x, double y) {
  if (y_.empty() || y > best_y_) {
    best_y_ = y;
    best_x_ = x;
  }
  x_.push_back(Normalise(x));
  y_.push_back(y);
}

void BayesianOptimization::Clear() {
  x_.clear();
  y_.clear();
  best_x_.clear();
  best_y_ = 0;
}

double BayesianOptimization::ExpectedImprovement(
    const std::vector<double>& u) const {
  double mean, sd;
  gp_.Predict(u, &mean, &sd);
  if (sd <= 1e-12) return 0.0;
  double best = best_y_ / y_scale_;
  double imp = mean - best - xi_;
  double z = imp / sd;
  return imp * NormCdf(z) + sd * NormPdf(z);
}

std::vector<double> BayesianOptimization::NextSample() {
  size_t d = bounds_.size();
  std::uniform_real_distribution<double> uni(0.0, 1.0);
  if (y_.empty()) {
    std::vector<double> u(d);
    for (auto& v : u) v = uni(rng_);
    return Denormalise(u);
  }
  // Scores are scaled to unit magnitude so the fixed noise term and xi mean
  // the same thing whatever the unit of the score.
  y_scale_ = 0;
  for (double v : y_) y_scale_ = std::max(y_scale_, std::fabs(v));
  if (y_scale_ <= 0) y_scale_ = 1.0;
  std::vector<double> ys(y_.size());
  for (size_t i = 0; i < y_.size(); ++i) ys[i] = y_[i] / y_scale_;
  gp_.Fit(x_, ys);

  std::vector<double> best_u(d, 0.5);
  double best_ei = -1.0;
  const int restarts = 20;
  for (int r = 0; r < restarts; ++r) {
    std::vector<double> u(d);
    for (auto& v : u) v = uni(rng_);
    double ei = ExpectedImprovement(u);
    double step = 0.25;
    while (step > 1e-3) {  // pattern search inside the unit box
      bool moved = false;
      for (size_t i = 0; i < d; ++i) {
        for (double dir : {-1.0, 1.0}) {
          std::vector<double> c = u;
          c[i] = std::min(1.0, std::max(0.0, c[i] + dir * step));
          double e = ExpectedImprovement(c);
          if (e > ei) {
            ei = e;
            u = c;
            moved = true;
          }
        }
      }
      if (!moved) step *= 0.5;
    }
    if (ei > best_ei) {
      best_ei = ei;
      best_u = u;
    }
  }
  return Denormalise(best_u);
}

}  // namespace hvd
