#include "gaussian_process.h"

#include <cmath>
#include <limits>

namespace hvd {

double GaussianProcess::Kernel(const std::vector<double>& a,
                               const std::vector<double>& b,
                               double length) const {
  double d2 = 0;
  for (size_t i = 0; i < a.size(); ++i) d2 += (a[i] - b[i]) * (a[i] - b[i]);
  return std::exp(-0.5 * d2 / (length * length));
}

double GaussianProcess::Factor(double length, std::vector<double>* chol,
                               std::vector<double>* weights) const {
  size_t n = x_.size();
  std::vector<double>& L = *chol;
  L.assign(n * n, 0.0);
  for (size_t i = 0; i < n; ++i)
    for (size_t j = 0; j <= i; ++j)
      L[i * n + j] = Kernel(x_[i], x_[j], length) + (i == j ? alpha_ : 0.0);
  // In-place Cholesky (lower).
  for (size_t j = 0; j < n; ++j) {
    double d = L[j * n + j];
    for (size_t k = 0; k < j; ++k) d -= L[j * n + k] * L[j * n + k];
    if (d <= 1e-12) return -std::numeric_limits<double>::infinity();
    d = std::sqrt(d);
    L[j * n + j] = d;
    for (size_t i = j + 1; i < n; ++i) {
      double s = L[i * n + j];
      for (size_t k = 0; k < j; ++k) s -= L[i * n + k] * L[j * n + k];
      L[i * n + j] = s / d;
    }
  }
  // Solve L z = y, then L^T w = z.
  std::vector<double>& w = *weights;
  w = y_;
  for (size_t i = 0; i < n; ++i) {
    double s = w[i];
    for (size_t k = 0; k < i; ++k) s -= L[i * n + k] * w[k];
    w[i] = s / L[i * n + i];
  }
  double quad = 0;
  for (size_t i = 0; i < n; ++i) quad += w[i] * w[i];
  for (size_t ii = n; ii-- > 0;) {
    double s = w[ii];
    for (size_t k = ii + 1; k < n; ++k) s -= L[k * n + ii] * w[k];
    w[ii] = s / L[ii * n + ii];
  }
  double logdet = 0;
  for (size_t i = 0; i < n; ++i) logdet += std::log(L[i * n + i]);
  return -0.5 * quad - logdet - 0.5 * n * std::log(2 * M_PI);
}

void GaussianProcess::Fit(const std::vector<std::vector<double>>& x,
                          const std::vector<double>& y) {
  x_ = x;
  y_mean_ = 0;
  for (double v : y) y_mean_ += v;
  if (!y.empty()) y_mean_ /= static_cast<double>(y.size());
  y_.resize(y.size());
  for (size_t i = 0; i < y.size(); ++i) y_[i] = y[i] - y_mean_;
  if (x_.empty()) return;
  // Coarse log-spaced scan of the length scale, then refine around the best.
  double best_l = 1.0, best_ll = -std::numeric_limits<double>::infinity();
  std::vector<double> chol, w;
  for (int i = -10; i <= 10; ++i) {
    double l = std::pow(10.0, i / 5.0);  // 1e-2 .. 1e2
    double ll = Factor(l, &chol, &w);
    if (ll > best_ll) {
      best_ll = ll;
      best_l = l;
    }
  }
  double lo = best_l / std::pow(10.0, 0.2), hi = best_l * std::pow(10.0, 0.2);
  for (int it = 0; it < 24; ++it) {  // golden-section in log space
    double a = std::log(lo), b = std::log(hi);
    double m1 = std::exp(b - 0.618 * (b - a)), m2 = std::exp(a + 0.618 * (b - a));
    double f1 = Factor(m1, &chol, &w), f2 = Factor(m2, &chol, &w);
    if (f1 > f2) hi = m2; else lo = m1;
  }
  length_ = std::sqrt(lo * hi);
  Factor(length_, &chol_, &weights_);
}

void GaussianProcess::Predict(const std::vector<double>& x, double* mean,
                              double* std) const {
  size_t n = x_.size();
  if (n == 0) {
    *mean = 0;
    *std = 1;
    return;
  }
  std::vector<double> k(n);
  double m = 0;
  for (size_t i = 0; i < n; ++i) {
    k[i] = Kernel(x, x_[i], length_);
    m += k[i] * weights_[i];
  }
  // v = L^-1 k ; var = k(x,x) - v.v
  for (size_t i = 0; i < n; ++i) {
    double s = k[i];
    for (size_t j = 0; j < i; ++j) s -= chol_[i * n + j] * k[j];
    k[i] = s / chol_[i * n + i];
  }
  double var = 1.0;
  for (size_t i = 0; i < n; ++i) var -= k[i] * k[i];
  *mean = m + y_mean_;
  *std = var > 0 ? std::sqrt(var) : 0.0;
}

}  // namespace hvd
