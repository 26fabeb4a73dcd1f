// Gaussian-process regression with an RBF kernel on small dense problems
// (tens of samples, a few dimensions), used by the autotuner.
//
// Parity: horovod/common/optim/gaussian_process.cc:45-180. The reference
// relies on Eigen and an L-BFGS library; this version carries its own
// Cholesky solver and fits the kernel length scale by a bracketed search on
// the log marginal likelihood.
#pragma once

#include <vector>

namespace hvd {

class GaussianProcess {
public:
  // alpha is the observation-noise variance added to the kernel diagonal.
  explicit GaussianProcess(double alpha = 0.8) : alpha_(alpha) {}

  // x: n rows of d features. y: n targets.
  void Fit(const std::vector<std::vector<double>>& x,
           const std::vector<double>& y);
  // Posterior mean and standard deviation at one point.
  void Predict(const std::vector<double>& x, double* mean, double* std) const;
  double length_scale() const { return length_; }
  bool fitted() const { return !x_.empty(); }

private:
  double Kernel(const std::vector<double>& a, const std::vector<double>& b,
                double length) const;
  // Factorises K(length)+alpha*I and returns the log marginal likelihood.
  double Factor(double length, std::vector<double>* chol,
                std::vector<double>* weights) const;

  double alpha_;
  double length_ = 1.0;
  double y_mean_ = 0.0;
  std::vector<std::vector<double>> x_;
  std::vector<double> y_;        // centred targets
  std::vector<double> chol_;     // n*n lower-triangular factor, row-major
  std::vector<double> weights_;  // (K + alpha I)^-1 y
};

}  // namespace hvd
