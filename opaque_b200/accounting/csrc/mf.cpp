// Matrix-factorisation strategies whose columns are shifted copies of one coefficient sequence (lower-triangular
// Toeplitz C, column k = c[0..] starting at row k, truncated to n rows), optionally column-normalised (C~ = C D^-1 with
// D = diag(||C[:, k]||)): DP-lambda-CGD (c_u = lambda^u) and banded-inverse-square-root strategies (c = power-series
// inverse of the banded C^-1 taps).
//
//   * sensitivities under min-separation b and at most k participations: the largest norm of a sum of participating
//     columns.  All coefficient sequences handled here are non-negative, so every Gram entry is non-negative and the
//     worst record takes part in a full window of allowed positions; the maximum is taken over all such windows.
//   * "balls-in-bins" Gram matrices: G_ij = <m_i, m_j>, m_i = sum over epochs e of column (b e + i), for i, j < b,
//     optionally with each column passed through a momentum filter (m[t] = beta m[t-1] + col[t]) and weighted per row by
//     learning-rate weights.  These feed the Monte-Carlo accountant of balls-in-bins participation.
//
// Reference counterparts (Rust): packages/opaque-accounting/src/matrix_factorization/{lambda_cgd,bisr,gram_matrix}.rs.
// This file computes everything numerically from the coefficient sequence (O(n) per inner product via lag products)
// instead of per-strategy closed forms, so one code path serves lambda-CGD, BISR and any other Toeplitz strategy.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <stdexcept>
#include <vector>

#include "pld.hpp"

namespace obacc {

namespace {

struct ToeplitzColumns {
  std::vector<double> c;          // coefficients, length n (zero padded)
  std::vector<double> norm;       // ||column k|| (1 when not normalised)
  std::size_t n;

  ToeplitzColumns(const std::vector<double>& coef, std::size_t n_, bool normalized) : c(n_, 0.0), norm(n_, 1.0), n(n_) {
    for (std::size_t i = 0; i < n && i < coef.size(); ++i) c[i] = coef[i];
    if (normalized) {
      // ||col_k||^2 = sum_{u < n - k} c_u^2: suffix of a prefix sum
      std::vector<double> pre(n + 1, 0.0);
      for (std::size_t u = 0; u < n; ++u) pre[u + 1] = pre[u] + c[u] * c[u];
      for (std::size_t k = 0; k < n; ++k) norm[k] = std::sqrt(std::max(pre[n - k], 1e-300));
    }
  }
  // <col_a, col_b> / (d_a d_b) for a <= b:  sum_{u < n - b} c_u c_{u + (b - a)}
  double inner(std::size_t a, std::size_t b) const {
    if (a > b) std::swap(a, b);
    const std::size_t g = b - a;
    double s = 0.0;
    for (std::size_t u = 0; u + b < n; ++u) s += c[u] * c[u + g];
    return s / (norm[a] * norm[b]);
  }
};

std::size_t epochs_for(std::size_t n, std::size_t b, std::int64_t max_part) {
  const std::size_t inferred = (n + b - 1) / b;
  return max_part < 0 ? inferred : std::min<std::size_t>(inferred, static_cast<std::size_t>(max_part));
}

double window_sens_sq(const ToeplitzColumns& t, std::size_t b, std::size_t k) {
  double best = 0.0;
  const std::size_t n = t.n;
  for (std::size_t start = 0; start < std::min(b, n); ++start) {
    std::vector<std::size_t> pos;
    for (std::size_t p = start; p < n; p += b) pos.push_back(p);
    const std::size_t kk = std::min(k, pos.size());
    for (std::size_t off = 0; off + kk <= pos.size(); ++off) {
      double tot = 0.0;
      for (std::size_t i = 0; i < kk; ++i) {
        tot += t.inner(pos[off + i], pos[off + i]);
        for (std::size_t j = i + 1; j < kk; ++j) tot += 2.0 * t.inner(pos[off + i], pos[off + j]);
      }
      best = std::max(best, tot);
    }
  }
  return best;
}

std::vector<double> bnb_gram(const ToeplitzColumns& t, std::size_t b, std::size_t epochs, double momentum,
                             const std::vector<double>* lr_weights) {
  const std::size_t n = t.n;
  if (lr_weights != nullptr && lr_weights->size() != n) throw std::invalid_argument("lr_weights must have n_steps entries");
  // momentum-filtered coefficients: cb[u] = sum_{j <= u} beta^{u-j} c_j  (the filter commutes with the shift)
  std::vector<double> cb(n, 0.0);
  for (std::size_t u = 0; u < n; ++u) cb[u] = (u ? momentum * cb[u - 1] : 0.0) + t.c[u];
  std::vector<double> m(b * n, 0.0);                     // m[i][t]
  for (std::size_t i = 0; i < b; ++i)
    for (std::size_t e = 0; e < epochs; ++e) {
      const std::size_t k = b * e + i;
      if (k >= n) break;
      const double inv = 1.0 / t.norm[k];
      for (std::size_t r = k; r < n; ++r) m[i * n + r] += cb[r - k] * inv;
    }
  if (lr_weights != nullptr)
    for (std::size_t i = 0; i < b; ++i)
      for (std::size_t r = 0; r < n; ++r) m[i * n + r] *= (*lr_weights)[r];
  std::vector<double> g(b * b, 0.0);
  for (std::size_t i = 0; i < b; ++i)
    for (std::size_t j = i; j < b; ++j) {
      double s = 0.0;
      for (std::size_t r = 0; r < n; ++r) s += m[i * n + r] * m[j * n + r];
      g[i * b + j] = g[j * b + i] = s;
    }
  return g;
}

std::vector<double> lambda_coefs(double lambda, std::size_t n) {
  if (!(lambda >= 0.0 && lambda < 1.0)) throw std::invalid_argument("lambda must be in [0, 1)");
  std::vector<double> c(n, 0.0);
  double p = 1.0;
  for (std::size_t u = 0; u < n; ++u) {
    c[u] = p;
    p *= lambda;
    if (p < 1e-300) break;
  }
  return c;
}

void check(std::size_t n, std::int64_t min_sep, double momentum) {
  if (n == 0) throw std::invalid_argument("n_steps must be >= 1");
  if (min_sep < 1) throw std::invalid_argument("min_sep must be >= 1");
  if (!(momentum >= 0.0 && momentum < 1.0)) throw std::invalid_argument("momentum must be in [0, 1)");
}

}  // namespace

// First n entries of column 0 of C for a banded inverse C^-1 with taps t (power-series inverse).
std::vector<double> inverse_toeplitz_coefficients(const std::vector<double>& taps, std::size_t n) {
  if (taps.empty() || taps[0] == 0.0) throw std::invalid_argument("the inverse needs a non-zero leading tap");
  std::vector<double> c(n, 0.0);
  for (std::size_t k = 0; k < n; ++k) {
    double s = k == 0 ? 1.0 : 0.0;
    for (std::size_t j = 1; j <= k && j < taps.size(); ++j) s -= taps[j] * c[k - j];
    c[k] = s / taps[0];
  }
  return c;
}

double toeplitz_columns_sens_sq(const std::vector<double>& coef, std::size_t n, std::int64_t min_sep, std::int64_t max_part,
                                bool normalized) {
  check(n, min_sep, 0.0);
  const ToeplitzColumns t(coef, n, normalized);
  const std::size_t b = static_cast<std::size_t>(min_sep);
  return window_sens_sq(t, b, epochs_for(n, b, max_part));
}

std::vector<double> toeplitz_columns_bnb_gram(const std::vector<double>& coef, std::size_t n, std::int64_t min_sep,
                                              std::int64_t max_part, bool normalized, double momentum,
                                              const std::vector<double>* lr_weights) {
  check(n, min_sep, momentum);
  const ToeplitzColumns t(coef, n, normalized);
  const std::size_t b = static_cast<std::size_t>(min_sep);
  return bnb_gram(t, b, epochs_for(n, b, max_part), momentum, lr_weights);
}

double lambda_cgd_sens_sq(double lambda, std::size_t n, std::int64_t min_sep, std::int64_t max_part, bool normalized) {
  return toeplitz_columns_sens_sq(lambda_coefs(lambda, n), n, min_sep, max_part, normalized);
}

double lambda_cgd_max_column_norm(double lambda, std::size_t n) {
  if (!(lambda >= 0.0 && lambda < 1.0)) throw std::invalid_argument("lambda must be in [0, 1)");
  const double l2 = lambda * lambda;
  if (l2 == 0.0) return 1.0;
  return std::sqrt((1.0 - std::pow(l2, static_cast<double>(n))) / (1.0 - l2));
}

std::vector<double> lambda_cgd_bnb_gram(double lambda, std::size_t n, std::int64_t min_sep, std::int64_t max_part,
                                        bool normalized, double momentum, const std::vector<double>* lr_weights) {
  return toeplitz_columns_bnb_gram(lambda_coefs(lambda, n), n, min_sep, max_part, normalized, momentum, lr_weights);
}

}  // namespace obacc
