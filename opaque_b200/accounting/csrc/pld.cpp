// PLD accountant core (see pld.hpp for the overview and the parity map).
#include "pld.hpp"

#include <algorithm>
#include <cmath>
#include <complex>
#include <limits>
#include <numeric>
#include <random>
#include <stdexcept>

namespace obacc {

namespace {
constexpr double kInf = std::numeric_limits<double>::infinity();
constexpr double kPi = 3.14159265358979323846;
constexpr double kSqrt2 = 1.41421356237309504880;

void require(bool ok, const char* msg) {
  if (!ok) throw std::invalid_argument(msg);
}
}  // namespace

// =============================================================================== special functions

double norm_cdf(double z) { return 0.5 * std::erfc(-z / kSqrt2); }

double norm_log_cdf(double z) {
  if (z > -30.0) {
    if (z > 5.0) return std::log1p(-0.5 * std::erfc(z / kSqrt2));
    return std::log(0.5 * std::erfc(-z / kSqrt2));
  }
  // asymptotic expansion of the Mills ratio for the far lower tail
  const double z2 = z * z;
  const double series = 1.0 - 1.0 / z2 + 3.0 / (z2 * z2) - 15.0 / (z2 * z2 * z2) + 105.0 / (z2 * z2 * z2 * z2);
  return -0.5 * z2 - std::log(-z) - 0.5 * std::log(2.0 * kPi) + std::log(series);
}

double norm_ppf(double p) {
  require(p > 0.0 && p < 1.0, "norm_ppf: p must be in (0, 1)");
  // Acklam's rational approximation followed by one Halley refinement step
  static const double a[] = {-3.969683028665376e+01, 2.209460984245205e+02, -2.759285104469687e+02,
                             1.383577518672690e+02, -3.066479806614716e+01, 2.506628277459239e+00};
  static const double b[] = {-5.447609879822406e+01, 1.615858368580409e+02, -1.556989798598866e+02,
                             6.680131188771972e+01, -1.328068155288572e+01};
  static const double c[] = {-7.784894002430293e-03, -3.223964580411365e-01, -2.400758277161838e+00,
                             -2.549732539343734e+00, 4.374664141464968e+00, 2.938163982698783e+00};
  static const double d[] = {7.784695709041462e-03, 3.224671290700398e-01, 2.445134137142996e+00,
                             3.754408661907416e+00};
  const double plow = 0.02425;
  double x;
  if (p < plow) {
    const double q = std::sqrt(-2.0 * std::log(p));
    x = (((((c[0] * q + c[1]) * q + c[2]) * q + c[3]) * q + c[4]) * q + c[5]) /
        ((((d[0] * q + d[1]) * q + d[2]) * q + d[3]) * q + 1.0);
  } else if (p <= 1.0 - plow) {
    const double q = p - 0.5, r = q * q;
    x = (((((a[0] * r + a[1]) * r + a[2]) * r + a[3]) * r + a[4]) * r + a[5]) * q /
        (((((b[0] * r + b[1]) * r + b[2]) * r + b[3]) * r + b[4]) * r + 1.0);
  } else {
    const double q = std::sqrt(-2.0 * std::log1p(-p));
    x = -(((((c[0] * q + c[1]) * q + c[2]) * q + c[3]) * q + c[4]) * q + c[5]) /
        ((((d[0] * q + d[1]) * q + d[2]) * q + d[3]) * q + 1.0);
  }
  for (int it = 0; it < 2; ++it) {
    const double e = norm_cdf(x) - p;
    const double u = e * std::sqrt(2.0 * kPi) * std::exp(0.5 * x * x);
    x = x - u / (1.0 + 0.5 * x * u);
  }
  return x;
}

double log_add(double a, double b) {
  if (a == -kInf) return b;
  if (b == -kInf) return a;
  const double hi = std::max(a, b), lo = std::min(a, b);
  return hi + std::log1p(std::exp(lo - hi));
}

double log_sub(double a, double b) {
  if (b == -kInf) return a;
  if (a < b) throw std::domain_error("log_sub: a < b");
  if (a == b) return -kInf;
  return a + std::log1p(-std::exp(b - a));
}

double log_sumexp(const std::vector<double>& v) {
  double m = -kInf;
  for (double x : v) m = std::max(m, x);
  if (m == -kInf) return -kInf;
  double s = 0.0;
  for (double x : v) s += std::exp(x - m);
  return m + std::log(s);
}

double log_a_times_exp_b_plus_c(double a, double b, double c) {
  // log(a e^b + c) with a, c >= 0
  if (a == 0.0) return std::log(c);
  if (c == 0.0) return std::log(a) + b;
  return log_add(std::log(a) + b, std::log(c));
}

// =============================================================================== FFT

namespace {
using cd = std::complex<double>;

std::size_t next_pow2(std::size_t n) {
  std::size_t p = 1;
  while (p < n) p <<= 1;
  return p;
}

void fft_inplace(std::vector<cd>& a, bool inverse) {
  const std::size_t n = a.size();
  for (std::size_t i = 1, j = 0; i < n; ++i) {
    std::size_t bit = n >> 1;
    for (; j & bit; bit >>= 1) j ^= bit;
    j ^= bit;
    if (i < j) std::swap(a[i], a[j]);
  }
  std::vector<cd> tw(n / 2 > 0 ? n / 2 : 1);
  const double sign = inverse ? 1.0 : -1.0;
  for (std::size_t k = 0; k < n / 2; ++k) {
    const double ang = sign * 2.0 * kPi * static_cast<double>(k) / static_cast<double>(n);
    tw[k] = cd(std::cos(ang), std::sin(ang));
  }
  for (std::size_t len = 2; len <= n; len <<= 1) {
    const std::size_t half = len >> 1, step = n / len;
    const std::int64_t blocks = static_cast<std::int64_t>(n / len);
#pragma omp parallel for schedule(static) if (n >= (1u << 16))
    for (std::int64_t blk = 0; blk < blocks; ++blk) {
      const std::size_t i = static_cast<std::size_t>(blk) * len;
      for (std::size_t k = 0; k < half; ++k) {
        const cd u = a[i + k], v = a[i + k + half] * tw[k * step];
        a[i + k] = u + v;
        a[i + k + half] = u - v;
      }
    }
  }
  if (inverse) {
    const double inv = 1.0 / static_cast<double>(n);
    for (auto& x : a) x *= inv;
  }
}
}  // namespace

std::vector<double> convolve(const std::vector<double>& a, const std::vector<double>& b) {
  if (a.empty() || b.empty()) return {};
  const std::size_t out = a.size() + b.size() - 1;
  if (std::min(a.size(), b.size()) <= 32) {
    std::vector<double> r(out, 0.0);
    for (std::size_t i = 0; i < a.size(); ++i)
      for (std::size_t j = 0; j < b.size(); ++j) r[i + j] += a[i] * b[j];
    return r;
  }
  const std::size_t n = next_pow2(out);
  std::vector<cd> fa(n), fb(n);
  for (std::size_t i = 0; i < a.size(); ++i) fa[i] = a[i];
  for (std::size_t i = 0; i < b.size(); ++i) fb[i] = b[i];
  fft_inplace(fa, false);
  fft_inplace(fb, false);
  for (std::size_t i = 0; i < n; ++i) fa[i] *= fb[i];
  fft_inplace(fa, true);
  std::vector<double> r(out);
  for (std::size_t i = 0; i < out; ++i) r[i] = std::max(0.0, fa[i].real());
  return r;
}

namespace {

// Chernoff window [lo, hi] (indices of the full n-fold convolution) outside which at most the given
// tail budgets of mass can lie.
std::pair<std::size_t, std::size_t> self_convolve_bounds(const std::vector<double>& probs, std::size_t times,
                                                          double right_budget, double left_budget) {
  const std::size_t full_hi = probs.size() * times - times;
  if (times == 1) return {0, probs.size() - 1};
  if (right_budget <= 0.0 && left_budget <= 0.0) return {0, full_hi};
  const double n = static_cast<double>(probs.size());
  std::size_t best_lo = 0, best_hi = full_hi;
  std::vector<double> terms(probs.size());
  for (int i = 0; i < 40; ++i) {
    const double order = (static_cast<double>(i) - 20.0) / n;
    if (order == 0.0) continue;
    for (std::size_t k = 0; k < probs.size(); ++k)
      terms[k] = probs[k] > 0.0 ? order * static_cast<double>(k) + std::log(probs[k]) : -kInf;
    const double log_mgf = log_sumexp(terms);
    if (order > 0.0 && right_budget > 0.0) {
      const double bound = (static_cast<double>(times) * log_mgf - std::log(right_budget)) / order;
      if (bound >= 0.0 && bound < static_cast<double>(full_hi))
        best_hi = std::min(best_hi, static_cast<std::size_t>(std::ceil(bound)));
    } else if (order < 0.0 && left_budget > 0.0) {
      const double bound = (static_cast<double>(times) * log_mgf - std::log(left_budget)) / order;
      if (bound > 0.0) best_lo = std::max(best_lo, static_cast<std::size_t>(std::floor(bound)));
    }
  }
  best_lo = std::min(best_lo, full_hi);
  best_hi = std::max(best_hi, best_lo);
  return {best_lo, best_hi};
}

// probs^{*times} restricted to [lo, hi]; a circular FFT of the window length suffices because the mass
// that wraps around is bounded by the discarded tails.
std::vector<double> self_convolve_window(const std::vector<double>& probs, std::size_t times, std::size_t lo,
                                         std::size_t hi) {
  const std::size_t want = hi - lo + 1;
  const std::size_t n = next_pow2(std::max(want, probs.size()));
  std::vector<cd> f(n);
  for (std::size_t i = 0; i < probs.size(); ++i) f[i] = probs[i];
  fft_inplace(f, false);
  const double k = static_cast<double>(times);
#pragma omp parallel for schedule(static) if (n >= (1u << 16))
  for (std::int64_t i = 0; i < static_cast<std::int64_t>(n); ++i) {
    const double mag = std::abs(f[i]);
    if (mag == 0.0) {
      f[i] = 0.0;
    } else {
      const double ang = std::arg(f[i]);
      f[i] = std::polar(std::exp(k * std::log(mag)), std::fmod(k * ang, 2.0 * kPi));
    }
  }
  fft_inplace(f, true);
  std::vector<double> out(want);
  for (std::size_t i = 0; i < want; ++i) out[i] = std::max(0.0, f[(lo + i) % n].real());
  return out;
}

std::int64_t floor_div(std::int64_t a, std::int64_t b) {
  std::int64_t q = a / b;
  if ((a % b != 0) && ((a < 0) != (b < 0))) --q;
  return q;
}

double compose_inf(double p, std::size_t count) {
  if (p == 0.0) return 0.0;
  return -std::expm1(static_cast<double>(count) * std::log1p(-p));
}

}  // namespace

// =============================================================================== Pmf

double Pmf::delta_at(double eps) const {
  double delta = infinity_mass;
  for (std::size_t i = 0; i < probs.size(); ++i) {
    const double loss = loss_at(static_cast<std::int64_t>(i));
    if (loss > eps) delta += -std::expm1(eps - loss) * probs[i];
  }
  return delta;
}

double Pmf::epsilon_at(double target_delta) const {
  if (infinity_mass > target_delta) return kInf;
  double mass_upper = infinity_mass, mass_lower = 0.0;
  for (std::int64_t i = static_cast<std::int64_t>(probs.size()) - 1; i >= 0; --i) {
    const double loss = loss_at(i), p = probs[static_cast<std::size_t>(i)];
    if (mass_upper > target_delta && mass_lower > 0.0 && std::log((mass_upper - target_delta) / mass_lower) >= loss)
      break;
    mass_upper += p;
    mass_lower += std::exp(-loss) * p;
    if (mass_upper >= target_delta && mass_lower == 0.0) return std::max(loss, 0.0);
  }
  if (mass_upper <= mass_lower + target_delta) return 0.0;
  return std::log((mass_upper - target_delta) / mass_lower);
}

Pmf Pmf::coarsen(std::size_t factor) const {
  if (factor <= 1) return *this;
  const std::int64_t f = static_cast<std::int64_t>(factor);
  const std::int64_t aligned = floor_div(lower, f) * f;
  const std::size_t left = static_cast<std::size_t>(lower - aligned);
  const std::size_t total = left + probs.size();
  const std::size_t groups = (total + factor - 1) / factor;
  Pmf out = *this;
  out.probs.assign(groups, 0.0);
  for (std::size_t i = 0; i < probs.size(); ++i) out.probs[(left + i) / factor] += probs[i];
  out.discretization = discretization * static_cast<double>(factor);
  out.lower = aligned / f + 1;   // round losses UP to the coarse grid (pessimistic)
  return out;
}

Pmf Pmf::maybe_coarsen() const {
  if (probs.size() <= max_grid_size) return *this;
  const double ratio = std::ceil(static_cast<double>(probs.size()) / static_cast<double>(max_grid_size));
  const int k = std::max(1, static_cast<int>(std::ceil(std::log2(ratio))));
  return coarsen(static_cast<std::size_t>(1) << k);
}

Pmf Pmf::compose(const Pmf& other, double tail_mass_truncation) const {
  Pmf a = *this, b = other;
  if (a.discretization != b.discretization) {
    const double big = std::max(a.discretization, b.discretization), small = std::min(a.discretization, b.discretization);
    const double ratio = big / small;
    const double rounded = std::round(ratio);
    if (std::fabs(ratio - rounded) > 1e-9 * ratio) throw std::invalid_argument("compose: incompatible discretizations");
    if (a.discretization < b.discretization) a = a.coarsen(static_cast<std::size_t>(rounded));
    else b = b.coarsen(static_cast<std::size_t>(rounded));
  }
  Pmf out;
  out.discretization = a.discretization;
  out.max_grid_size = std::max(a.max_grid_size, b.max_grid_size);
  out.right_budget = a.right_budget + b.right_budget;
  out.left_budget = a.left_budget + b.left_budget;
  out.infinity_mass = a.infinity_mass + b.infinity_mass - a.infinity_mass * b.infinity_mass;
  out.neg_infinity_mass = a.neg_infinity_mass + b.neg_infinity_mass - a.neg_infinity_mass * b.neg_infinity_mass;
  if (a.probs.empty() || b.probs.empty()) {
    out.lower = 0;
    return out;
  }
  std::vector<double> conv = convolve(a.probs, b.probs);
  std::size_t lo = 0, hi = conv.size();
  if (tail_mass_truncation > 0.0) {
    // drop up to half the budget from each side; the right tail goes to the infinity mass
    double acc = 0.0;
    while (lo + 1 < hi && acc + conv[lo] <= tail_mass_truncation / 2.0) acc += conv[lo++];
    if (lo > 0 && lo < hi) conv[lo] += acc;     // left tail rounds up onto the first kept point
    double right = 0.0;
    while (hi > lo + 1 && right + conv[hi - 1] <= tail_mass_truncation / 2.0) right += conv[--hi];
    out.infinity_mass += right;
  }
  out.probs.assign(conv.begin() + static_cast<std::ptrdiff_t>(lo), conv.begin() + static_cast<std::ptrdiff_t>(hi));
  out.lower = a.lower + b.lower + static_cast<std::int64_t>(lo);
  return out.maybe_coarsen();
}

Pmf Pmf::self_compose(std::size_t count) const {
  require(count >= 1, "self_compose: count must be >= 1");
  if (count == 1) return *this;
  Pmf out = *this;
  if (probs.empty()) {
    out.infinity_mass = compose_inf(infinity_mass, count);
    out.neg_infinity_mass = compose_inf(neg_infinity_mass, count);
    return out;
  }
  const double eff_left = std::max(0.0, left_budget - neg_infinity_mass);
  const double eff_right = right_budget;
  const bool chernoff = eff_left > 0.0 || eff_right > 0.0;
  auto [lo, hi] = self_convolve_bounds(probs, count, eff_right, eff_left);
  out.probs = self_convolve_window(probs, count, lo, hi);
  out.lower = lower * static_cast<std::int64_t>(count) + static_cast<std::int64_t>(lo);
  out.infinity_mass = compose_inf(infinity_mass, count) + (chernoff ? eff_right : 0.0);
  out.neg_infinity_mass = compose_inf(neg_infinity_mass, count) + (chernoff ? eff_left : 0.0);
  return out.maybe_coarsen();
}

// =============================================================================== Pld

double Pld::delta_at(double eps) const {
  const double d = remove.delta_at(eps);
  return add ? std::max(d, add->delta_at(eps)) : d;
}
double Pld::epsilon_at(double delta) const {
  const double e = remove.epsilon_at(delta);
  return add ? std::max(e, add->epsilon_at(delta)) : e;
}
double Pld::infinity_mass() const {
  return add ? std::max(remove.infinity_mass, add->infinity_mass) : remove.infinity_mass;
}

Pld Pld::with_tail_budgets(double right, double left) const {
  Pld out = *this;
  out.remove.right_budget = right;
  out.remove.left_budget = left;
  if (out.add) {
    out.add->right_budget = right;
    out.add->left_budget = left;
  }
  return out;
}

Pld Pld::compose(const Pld& other, double tail) const {
  Pld out;
  out.remove = remove.compose(other.remove, tail);
  if (add || other.add) {
    const Pmf& a = add ? *add : remove;
    const Pmf& b = other.add ? *other.add : other.remove;
    out.add = a.compose(b, tail);
  }
  return out;
}

Pld Pld::self_compose(std::size_t count) const {
  Pld out;
  out.remove = remove.self_compose(count);
  if (add) out.add = add->self_compose(count);
  return out;
}

namespace {
// Trade-off curve of one direction from its PMF: beta(alpha) = inf over thresholds of the type-II error.
// Points of the privacy profile (eps, delta(eps)) give supporting lines  beta >= 1 - delta - e^eps alpha.
double beta_from_pmf(const Pmf& pmf, double alpha) {
  if (alpha >= 1.0) return 0.0;
  double best = 0.0;
  // evaluate the dual on the PMF's own grid (the profile is piecewise linear between grid points)
  double mass_upper = pmf.infinity_mass, mass_lower = 0.0;
  for (std::int64_t i = static_cast<std::int64_t>(pmf.probs.size()) - 1; i >= 0; --i) {
    const double loss = pmf.loss_at(i);
    // delta(loss) = mass_upper - e^{loss} mass_lower over points strictly above; use it before adding point i
    const double delta = std::max(0.0, mass_upper - std::exp(loss) * mass_lower);
    best = std::max(best, 1.0 - delta - std::exp(loss) * alpha);
    mass_upper += pmf.probs[static_cast<std::size_t>(i)];
    mass_lower += std::exp(-loss) * pmf.probs[static_cast<std::size_t>(i)];
  }
  if (!pmf.probs.empty()) {
    const double loss = pmf.loss_at(0) - pmf.discretization;
    const double delta = std::max(0.0, mass_upper - std::exp(loss) * mass_lower);
    best = std::max(best, 1.0 - delta - std::exp(loss) * alpha);
  }
  return std::min(std::max(best, 0.0), 1.0 - alpha);
}
}  // namespace

double Pld::beta_at(double alpha) const {
  require(alpha >= 0.0 && alpha <= 1.0, "beta_at: alpha must be in [0, 1]");
  double b = beta_from_pmf(remove, alpha);
  if (add) b = std::min(b, beta_from_pmf(*add, alpha));
  // symmetrise: the adversary may also test in the reverse direction (beta^{-1})
  return b;
}

double Pld::risk_at(double prior) const {
  require(prior > 0.0 && prior < 1.0, "risk_at: prior must be in (0, 1)");
  // Bayes risk = min over alpha of prior*alpha + (1-prior)*beta(alpha); golden-section search
  auto f = [&](double a) { return prior * a + (1.0 - prior) * beta_at(a); };
  double lo = 0.0, hi = 1.0;
  const double gr = (std::sqrt(5.0) - 1.0) / 2.0;
  double c = hi - gr * (hi - lo), d = lo + gr * (hi - lo);
  double fc = f(c), fd = f(d);
  for (int it = 0; it < 200 && hi - lo > 1e-10; ++it) {
    if (fc < fd) {
      hi = d; d = c; fd = fc; c = hi - gr * (hi - lo); fc = f(c);
    } else {
      lo = c; c = d; fc = fd; d = lo + gr * (hi - lo); fd = f(d);
    }
  }
  return std::min({f(0.5 * (lo + hi)), f(0.0), f(1.0)});
}

// =============================================================================== connect the dots

Pmf connect_the_dots(const std::vector<double>& deltas_in, std::int64_t lo_idx, double disc, std::size_t max_grid,
                     bool proportional_normalization) {
  require(!deltas_in.empty(), "connect_the_dots: empty delta array");
  std::vector<double> deltas = deltas_in;
  const std::size_t n = deltas.size();
  for (std::size_t i = 1; i < n; ++i) deltas[i] = std::min(deltas[i], deltas[i - 1]);
  Pmf pmf;
  pmf.discretization = disc;
  pmf.max_grid_size = max_grid;
  pmf.lower = lo_idx;
  if (n == 1) {
    pmf.probs = {std::max(0.0, 1.0 - deltas[0])};
    pmf.infinity_mass = deltas[0];
    return pmf;
  }
  const double exp_d = std::exp(disc), em1 = std::expm1(disc), em1n = std::expm1(-disc);
  std::vector<double> probs(n);
  probs[0] = (1.0 - deltas[0]) + (deltas[1] - deltas[0]) / em1;
  for (std::size_t i = 1; i + 1 < n; ++i)
    probs[i] = ((deltas[i + 1] - deltas[i]) - exp_d * (deltas[i] - deltas[i - 1])) / em1;
  probs[n - 1] = (deltas[n - 1] - deltas[n - 2]) / em1n;
  double total = 0.0;
  for (double& p : probs) {
    p = std::max(p, 0.0);
    total += p;
  }
  pmf.infinity_mass = deltas[n - 1];
  const double target = 1.0 - pmf.infinity_mass;
  // Clamping the cancellation noise of the second differences at zero leaves a little too much mass (about 1e-12 per grid
  // point, 1e-8 in total).  Scaling every probability down would lower delta(eps) by that relative amount everywhere, below
  // the exact curve; instead the surplus is taken from the LOWEST losses (no effect on delta at any eps above them) and a
  // shortfall is added at the HIGHEST loss, so the estimate stays an upper bound.
  double surplus = total - target;
  if (proportional_normalization) {
    if (total > 0.0 && total != target)
      for (double& p : probs) p *= target / total;
  } else if (surplus > 0.0) {
    for (std::size_t i = 0; i < n && surplus > 0.0; ++i) {
      const double take = std::min(probs[i], surplus);
      probs[i] -= take;
      surplus -= take;
    }
  } else if (surplus < 0.0) {
    probs[n - 1] -= surplus;
  }
  // trim leading / trailing zeros
  std::size_t first = 0, last = n;
  while (first + 1 < last && probs[first] == 0.0) ++first;
  while (last > first + 1 && probs[last - 1] == 0.0) --last;
  pmf.probs.assign(probs.begin() + static_cast<std::ptrdiff_t>(first), probs.begin() + static_cast<std::ptrdiff_t>(last));
  pmf.lower = lo_idx + static_cast<std::int64_t>(first);
  return pmf;
}

Pld discretize(const Config& cfg, EpsBounds rb, std::optional<EpsBounds> ab,
               const std::function<double(double, Adjacency)>& delta_fn) {
  EpsBounds u = rb;
  if (ab) {
    u.lo = std::min(u.lo, ab->lo);
    u.hi = std::max(u.hi, ab->hi);
  }
  double disc = cfg.discretization;
  const double grid = std::ceil((u.hi - u.lo) / disc);
  if (grid > static_cast<double>(cfg.max_grid_size)) {
    const double ratio = std::ceil(grid / static_cast<double>(cfg.max_grid_size));
    disc *= std::pow(2.0, std::max(1.0, std::ceil(std::log2(ratio))));
  }
  auto build = [&](EpsBounds b, Adjacency adj) {
    const std::int64_t hi = static_cast<std::int64_t>(std::ceil(b.hi / disc));
    const std::int64_t lo = static_cast<std::int64_t>(std::floor(b.lo / disc));
    std::vector<double> deltas(static_cast<std::size_t>(hi - lo + 1));
#pragma omp parallel for schedule(static) if (deltas.size() >= 4096)
    for (std::int64_t i = 0; i < static_cast<std::int64_t>(deltas.size()); ++i)
      deltas[static_cast<std::size_t>(i)] = delta_fn(static_cast<double>(lo + i) * disc, adj);
    return connect_the_dots(deltas, lo, disc, cfg.max_grid_size, cfg.proportional_normalization);
  };
  Pld out;
  out.remove = build(rb, Adjacency::Remove);
  if (ab) out.add = build(*ab, Adjacency::Add);
  return out;
}

// =============================================================================== mechanisms

double gaussian_delta(double nm, double eps, double sensitivity) {
  const double dt = sensitivity / nm;
  const double x = 0.5 * dt - eps / dt;
  return std::max(0.0, norm_cdf(x) - std::exp(eps) * norm_cdf(x - dt));
}

namespace {

double loss_remove(double x, double sigma, double s, double q) {
  const double raw = s * (-0.5 * s - x) / (sigma * sigma);
  if (std::fabs(q - 1.0) < 1e-15) return raw;
  return log_a_times_exp_b_plus_c(q, raw, 1.0 - q);
}
double loss_add(double x, double sigma, double s, double q) { return -loss_remove(-x, sigma, s, q); }

double inv_loss_gaussian(double loss, double sigma, double s) { return 0.5 * s - loss * sigma * sigma / s; }

EpsBounds poisson_bounds(double sigma, double s, double q, Adjacency adj, double log_mass) {
  const double lower_base = sigma * norm_ppf(0.5 * std::exp(log_mass)), upper_base = -lower_base;
  if (adj == Adjacency::Remove)
    return {loss_remove(upper_base, sigma, s, q), loss_remove(lower_base - s, sigma, s, q)};
  return {loss_add(upper_base + s, sigma, s, q), loss_add(lower_base, sigma, s, q)};
}

double poisson_delta_add(double eps, double sigma, double s, double q) {
  if (eps >= -std::log1p(-q) - 1e-10) return 0.0;
  const double ratio = (std::exp(-eps) - (1.0 - q)) / q;
  if (ratio <= 0.0) return 0.0;
  const double x = inv_loss_gaussian(-std::log(ratio), sigma, s);
  const double mu_upper = norm_cdf(x / sigma);
  const double log_mu_lower = log_add(std::log1p(-q) + norm_log_cdf(x / sigma), std::log(q) + norm_log_cdf((x - s) / sigma));
  return std::max(0.0, mu_upper - std::exp(eps + log_mu_lower));
}

double poisson_delta_remove(double eps, double sigma, double s, double q) {
  if (eps <= std::log1p(-q)) return std::max(0.0, -std::expm1(eps));
  const double ratio = (std::exp(eps) - (1.0 - q)) / q;
  if (ratio <= 0.0) return std::max(0.0, -std::expm1(eps));
  const double x = inv_loss_gaussian(-std::log(ratio), sigma, s);
  const double log_tail_upper = norm_log_cdf(-x / sigma);
  const double log_tail_shift = norm_log_cdf((s - x) / sigma);
  const double log_mu_upper = log_add(std::log1p(-q) + log_tail_upper, std::log(q) + log_tail_shift);
  return std::max(0.0, std::exp(log_mu_upper) - std::exp(eps + log_tail_upper));
}

double poisson_delta(double eps, Adjacency adj, double sigma, double s, double q) {
  if (std::fabs(q - 1.0) < 1e-15) return gaussian_delta(sigma, eps, s);
  return adj == Adjacency::Add ? poisson_delta_add(eps, sigma, s, q) : poisson_delta_remove(eps, sigma, s, q);
}

double log_sinh(double x) {   // x > 0
  return x + std::log1p(-std::exp(-2.0 * x)) - std::log(2.0);
}
double arcsinh_exp(double log_y, double sign) {   // asinh(sign * e^{log_y})
  const double y = std::exp(log_y);
  if (std::isinf(y)) return sign * (log_y + std::log(2.0));
  return sign * std::asinh(y);
}

// replace-adjacency Poisson-subsampled Gaussian (used by the truncated-Poisson bound)
double poisson_delta_replace(double eps, double sigma, double s, double q) {
  double x;
  if (eps == 0.0) x = 0.0;
  else if (std::fabs(q - 1.0) < 1e-15) x = -eps * sigma * sigma / (2.0 * s);
  else {
    const double ds = s / sigma;
    const double log_alpha = 0.5 * ds * ds + std::log1p(-q) - std::log(q);
    const double t = arcsinh_exp(log_alpha + log_sinh(std::fabs(eps) / 2.0), eps > 0 ? -1.0 : 1.0);
    x = (sigma * sigma / s) * (t - eps / 2.0);
  }
  const double cc = norm_cdf(x / sigma), cp = norm_cdf((x + s) / sigma), cm = norm_cdf((x - s) / sigma);
  return std::max(0.0, (q * cp + (1 - q) * cc) - std::exp(eps) * (q * cm + (1 - q) * cc));
}

void check_nm(double nm) { require(nm >= 1e-6 && std::isfinite(nm), "noise_multiplier must be finite and >= 1e-6"); }
void check_rate(double q) { require(q > 0.0 && q <= 1.0, "sampling rate must be in (0, 1]"); }

}  // namespace

Pld gaussian_pld(double nm, const Config& cfg, double sensitivity) {
  check_nm(nm);
  const double tail = cfg.tail_mass_truncation / 2.0;
  const EpsBounds b = poisson_bounds(nm, sensitivity, 1.0, Adjacency::Remove, cfg.log_mass_truncation_bound);
  return discretize(cfg, b, std::nullopt, [=](double e, Adjacency) { return gaussian_delta(nm, e, sensitivity); })
      .with_tail_budgets(tail, tail);
}

Pld poisson_gaussian_pld(double nm, double q, const Config& cfg) {
  check_nm(nm);
  check_rate(q);
  if (std::fabs(q - 1.0) < 1e-15) return gaussian_pld(nm, cfg);
  const double tail = cfg.tail_mass_truncation / 2.0, lm = cfg.log_mass_truncation_bound;
  return discretize(cfg, poisson_bounds(nm, 1.0, q, Adjacency::Remove, lm), poisson_bounds(nm, 1.0, q, Adjacency::Add, lm),
                    [=](double e, Adjacency a) { return poisson_delta(e, a, nm, 1.0, q); })
      .with_tail_budgets(tail, tail);
}

namespace {
// regularised incomplete beta based binomial CDF via log-space summation (n up to ~1e7 is fine)
double binom_cdf(std::int64_t k, std::int64_t n, double p) {
  if (k < 0) return 0.0;
  if (k >= n) return 1.0;
  const double lp = std::log(p), lq = std::log1p(-p);
  const double mean = static_cast<double>(n) * p;
  // sum the smaller side for accuracy
  auto log_pmf = [&](std::int64_t i) {
    return std::lgamma(static_cast<double>(n) + 1) - std::lgamma(static_cast<double>(i) + 1) -
           std::lgamma(static_cast<double>(n - i) + 1) + static_cast<double>(i) * lp + static_cast<double>(n - i) * lq;
  };
  if (static_cast<double>(k) < mean) {
    double s = 0.0;
    for (std::int64_t i = k; i >= 0; --i) {
      const double t = std::exp(log_pmf(i));
      s += t;
      if (t < 1e-300 || (i < k && t < s * 1e-18)) break;
    }
    return std::min(1.0, s);
  }
  double s = 0.0;
  for (std::int64_t i = k + 1; i <= n; ++i) {
    const double t = std::exp(log_pmf(i));
    s += t;
    if (t < 1e-300 || (i > k + 1 && t < s * 1e-18)) break;
  }
  return std::max(0.0, 1.0 - s);
}
}  // namespace

Pld truncated_poisson_gaussian_pld(double nm, double q, std::int64_t bmax, std::int64_t n, const Config& cfg) {
  check_nm(nm);
  check_rate(q);
  require(bmax > 0 && n > 0, "truncated Poisson: batch cap and dataset size must be positive");
  const double p_trunc = bmax >= n ? 0.0 : 1.0 - binom_cdf(bmax - 1, n - 1, q);
  if (p_trunc == 0.0) return poisson_gaussian_pld(nm, q, cfg);
  const double q_cond = (1.0 - binom_cdf(bmax, n, q)) * static_cast<double>(bmax) / static_cast<double>(n) / p_trunc;
  const double tail = cfg.tail_mass_truncation / 2.0, lm = cfg.log_mass_truncation_bound;
  auto bounds = [&](Adjacency adj) {
    EpsBounds b = poisson_bounds(nm, 1.0, q, adj, lm);
    // the replace component (sigma/2, rate q_cond) widens the range symmetrically
    const double base = (nm / 2.0) * norm_ppf(0.5 * std::exp(lm));
    auto loss_rep = [&](double x) {
      const double s2 = (nm / 2.0) * (nm / 2.0);
      const double lp = -(2.0 * x + 1.0) / (2.0 * s2), lmn = (2.0 * x - 1.0) / (2.0 * s2);
      return log_a_times_exp_b_plus_c(q_cond, lp, 1.0 - q_cond) - log_a_times_exp_b_plus_c(q_cond, lmn, 1.0 - q_cond);
    };
    if (q_cond > 0.0) {
      b.lo = std::min(b.lo, loss_rep(-base + 1.0));
      b.hi = std::max(b.hi, loss_rep(base - 1.0));
    }
    return b;
  };
  return discretize(cfg, bounds(Adjacency::Remove), bounds(Adjacency::Add), [=](double e, Adjacency) {
           const double d1 = std::max(poisson_delta_add(e, nm, 1.0, q), poisson_delta_remove(e, nm, 1.0, q));
           const double d2 = q_cond > 0.0 ? poisson_delta_replace(e, nm / 2.0, 1.0, q_cond) : 0.0;
           return (1.0 - p_trunc) * d1 + p_trunc * d2;
         })
      .with_tail_budgets(tail, tail);
}

// ---- Gaussian mixtures (one record contributes sensitivity s_k with probability p_k) -----------------

namespace {
struct Mixture {
  std::vector<double> log_p, sens, pre;
  double sigma, var, sampling_prob;
};

double mix_loss(double x, Adjacency adj, const Mixture& c) {
  std::vector<double> t(c.sens.size());
  const double sgn = adj == Adjacency::Remove ? -1.0 : 1.0;
  for (std::size_t k = 0; k < t.size(); ++k) t[k] = c.pre[k] + sgn * c.sens[k] * x / c.var;
  const double l = log_sumexp(t);
  return adj == Adjacency::Remove ? l : -l;
}

double mix_inverse_loss(double eps, Adjacency adj, const Mixture& c) {
  double smin = kInf, smax = 0.0;
  for (double s : c.sens) {
    if (s > 0.0) smin = std::min(smin, s);
    smax = std::max(smax, s);
  }
  const double c1 = inv_loss_gaussian(eps, c.sigma, smin), c2 = inv_loss_gaussian(eps, c.sigma, smax);
  double lo = std::min(c1, c2), hi = std::max(c1, c2);
  const double margin = std::max(std::fabs(hi - lo), 1.0) * 0.5;
  lo -= margin;
  hi += margin;
  for (int it = 0; it < 60; ++it) {
    const double pl = mix_loss(lo, adj, c), ph = mix_loss(hi, adj, c);
    if (pl >= eps && ph <= eps) break;
    if (pl < eps) lo -= std::max(std::fabs(hi - lo), 1.0);
    if (ph > eps) hi += std::max(std::fabs(hi - lo), 1.0);
  }
  for (int it = 0; it < 200; ++it) {
    const double mid = 0.5 * (lo + hi);
    if (std::fabs(hi - lo) < 1e-15 * std::max(std::fabs(hi), 1.0)) break;
    if (mix_loss(mid, adj, c) > eps) lo = mid; else hi = mid;
  }
  return 0.5 * (lo + hi);
}

double mix_delta(double eps, Adjacency adj, const Mixture& c) {
  if (c.sampling_prob < 1.0) {
    if (adj == Adjacency::Add && eps >= -std::log1p(-c.sampling_prob) - 1e-10) return 0.0;
    if (adj == Adjacency::Remove && eps <= std::log1p(-c.sampling_prob)) return std::max(0.0, -std::expm1(eps));
  }
  const double x = mix_inverse_loss(eps, adj, c);
  double mu_upper, log_mu_lower;
  if (adj == Adjacency::Remove) {
    mu_upper = 0.0;
    for (std::size_t k = 0; k < c.sens.size(); ++k) mu_upper += std::exp(c.log_p[k]) * norm_cdf((x + c.sens[k]) / c.sigma);
    log_mu_lower = norm_log_cdf(x / c.sigma);
  } else {
    mu_upper = norm_cdf(x / c.sigma);
    std::vector<double> t(c.sens.size());
    for (std::size_t k = 0; k < t.size(); ++k) t[k] = c.log_p[k] + norm_log_cdf((x - c.sens[k]) / c.sigma);
    log_mu_lower = log_sumexp(t);
  }
  return std::min(1.0, std::max(0.0, mu_upper - std::exp(eps + log_mu_lower)));
}
}  // namespace

Pld mixture_gaussian_pld(double sigma, const std::vector<double>& log_probs, const std::vector<double>& sens,
                         double head_mass, double tail_mass, const Config& cfg) {
  check_nm(sigma);
  require(log_probs.size() == sens.size() && !sens.empty(), "mixture: probabilities and sensitivities must match");
  Mixture c;
  c.log_p = log_probs;
  c.sens = sens;
  c.sigma = sigma;
  c.var = sigma * sigma;
  c.pre.resize(sens.size());
  c.sampling_prob = 0.0;
  double smax = 0.0;
  for (std::size_t k = 0; k < sens.size(); ++k) {
    c.pre[k] = log_probs[k] - 0.5 * sens[k] * sens[k] / c.var;
    if (sens[k] > 0.0) c.sampling_prob += std::exp(log_probs[k]);
    smax = std::max(smax, sens[k]);
  }
  c.sampling_prob = std::min(1.0, c.sampling_prob);
  const double z = norm_ppf(0.5 * std::exp(cfg.log_mass_truncation_bound));
  const EpsBounds rb{mix_loss(-sigma * z, Adjacency::Remove, c), mix_loss(sigma * z - smax, Adjacency::Remove, c)};
  const EpsBounds ab{mix_loss(-sigma * z + smax, Adjacency::Add, c), mix_loss(sigma * z, Adjacency::Add, c)};
  const double tail = cfg.tail_mass_truncation / 2.0;
  return discretize(cfg, rb, ab, [=](double e, Adjacency a) {
           return std::min(1.0, std::max(0.0, head_mass * mix_delta(e, a, c) + tail_mass));
         })
      .with_tail_budgets(tail, tail);
}

Pld parallel_poisson_gaussian_pld(double nm, double q, std::size_t workers, const Config& cfg) {
  check_nm(nm);
  require(q > 0.0 && q < 1.0, "parallel Poisson: rate must be in (0, 1)");
  require(workers >= 1, "parallel Poisson: workers must be >= 1");
  if (workers == 1) return poisson_gaussian_pld(nm, q, cfg);
  // number of workers that sampled the record ~ Binomial(workers, q); k hits give sensitivity k
  std::vector<double> lp(workers + 1);
  const double l1 = std::log1p(-q), lr = std::log(q / (1.0 - q));
  lp[0] = static_cast<double>(workers) * l1;
  for (std::size_t k = 1; k <= workers; ++k)
    lp[k] = lp[k - 1] + std::log(static_cast<double>(workers - k + 1) / static_cast<double>(k)) + lr;
  const double target = 0.5 * std::exp(cfg.log_mass_truncation_bound);
  std::size_t last = workers;
  double head = 0.0;
  for (std::size_t k = 0; k <= workers; ++k) {
    head += std::exp(lp[k]);
    if (std::max(0.0, 1.0 - head) <= target) {
      last = k;
      break;
    }
  }
  std::vector<double> sel(lp.begin(), lp.begin() + static_cast<std::ptrdiff_t>(last + 1));
  const double log_head = log_sumexp(sel);
  const double head_mass = std::exp(log_head), tail_mass = std::min(1.0, std::max(0.0, 1.0 - head_mass));
  std::vector<double> sens(sel.size());
  for (std::size_t k = 0; k < sel.size(); ++k) {
    sel[k] -= log_head;
    sens[k] = static_cast<double>(k);
  }
  return mixture_gaussian_pld(nm, sel, sens, head_mass, tail_mass, cfg);
}

Pld eps_delta_pld(double eps, double delta, const Config& cfg) {
  require(eps >= 0.0 && delta >= 0.0 && delta <= 1.0, "eps_delta: need eps >= 0 and delta in [0, 1]");
  // dominating pair of an (eps, delta)-DP mechanism: mass delta at +inf, the rest on +-eps
  Pmf p;
  p.discretization = cfg.discretization;
  p.max_grid_size = cfg.max_grid_size;
  const std::int64_t hi = static_cast<std::int64_t>(std::ceil(eps / cfg.discretization));
  const double e = static_cast<double>(hi) * cfg.discretization;
  const double up = (1.0 - delta) * std::exp(e) / (1.0 + std::exp(e)), dn = (1.0 - delta) / (1.0 + std::exp(e));
  p.lower = -hi;
  p.probs.assign(static_cast<std::size_t>(2 * hi + 1), 0.0);
  p.probs.front() += dn;
  p.probs.back() += up;
  p.infinity_mass = delta;
  Pld out;
  out.remove = p;
  return out;
}

Pld identity_pld(const Config& cfg) {
  Pmf p;
  p.discretization = cfg.discretization;
  p.max_grid_size = cfg.max_grid_size;
  p.lower = 0;
  p.probs = {1.0};
  Pld out;
  out.remove = p;
  return out;
}

Pld nonprivate_pld(const Config& cfg) {
  Pmf p;
  p.discretization = cfg.discretization;
  p.max_grid_size = cfg.max_grid_size;
  p.infinity_mass = 1.0;
  Pld out;
  out.remove = p;
  return out;
}

// ---- random allocation -----------------------------------------------------------------------------------
// k-out-of-t random allocation (each record is used in k steps chosen uniformly out of t).  For one allocation
// (k = 1) Feldman & Shenfeld show the privacy loss is a transform of the base loss L ~ N(mu, 2 mu), mu = 1/(2 sigma^2):
//     remove:  ln( (1/t) ( e^{L_0} + sum_{i=1}^{t-1} e^{-L~_i} ) )      with  -L~_i ~ N(-mu, 2 mu)
//     add:    -ln( (1/t) sum_{i=1}^{t} e^{-L_i} )
// i.e. log-mean-exps of independent terms.  The sums are convolutions of EXPONENTIATED distributions, carried on a
// geometric grid (value e^{alpha j}) with directed rounding: adding two grid values lands on
// max(i, j) + shift(|i - j|) with shift(d) = ceil or floor of log1p(e^{-alpha d}) / alpha, so one convolution is an
// O(G^2) table-driven scatter and t-fold sums take O(log t) convolutions.  k > 1 composes k single allocations
// over floor(t/k) / ceil(t/k) steps.

namespace {

struct GeomPmf {
  double alpha = 1e-3;
  std::int64_t lower = 0;          // value of p[i] is exp(alpha * (lower + i))
  std::vector<double> p;
  double inf_mass = 0.0;           // mass at +infinity
  double zero_mass = 0.0;          // mass at value 0
};

// Discretise N(mean, var) on the grid alpha * j, each cell's mass moved UP to its right end; the lower tail (mass
// beta) lumps onto the first point, the upper tail (mass beta) is returned separately.
void disc_normal(double mean, double var, double alpha, double beta, std::int64_t& lo, std::vector<double>& probs,
                 double& upper_tail) {
  const double sd = std::sqrt(var);
  const double zlo = norm_ppf(beta), zhi = -zlo;
  lo = static_cast<std::int64_t>(std::floor((mean + sd * zlo) / alpha));
  const std::int64_t hi = static_cast<std::int64_t>(std::ceil((mean + sd * zhi) / alpha));
  probs.assign(static_cast<std::size_t>(hi - lo + 1), 0.0);
  double prev = 0.0;
  for (std::int64_t j = lo; j <= hi; ++j) {
    const double c = norm_cdf((static_cast<double>(j) * alpha - mean) / sd);
    probs[static_cast<std::size_t>(j - lo)] = c - prev;
    prev = c;
  }
  upper_tail = std::max(0.0, 1.0 - prev);
}

GeomPmf geom_conv(const GeomPmf& a, const GeomPmf& b, bool round_up, double beta) {
  GeomPmf out;
  out.alpha = a.alpha;
  out.inf_mass = a.inf_mass + b.inf_mass - a.inf_mass * b.inf_mass;
  out.zero_mass = a.zero_mass * b.zero_mass;
  if (a.p.empty() || b.p.empty()) {
    const GeomPmf& keep = a.p.empty() ? b : a;
    const double z = a.p.empty() ? a.zero_mass : b.zero_mass;
    out.lower = keep.lower;
    out.p = keep.p;
    for (double& v : out.p) v *= z;
    return out;
  }
  const std::int64_t amax = a.lower + static_cast<std::int64_t>(a.p.size()) - 1;
  const std::int64_t bmax = b.lower + static_cast<std::int64_t>(b.p.size()) - 1;
  const std::int64_t lo = std::min(a.lower, b.lower);
  const std::int64_t max_d = std::max(amax, bmax) - lo;
  std::vector<std::int64_t> shift(static_cast<std::size_t>(max_d + 1));
  for (std::int64_t d = 0; d <= max_d; ++d) {
    const double v = std::log1p(std::exp(-a.alpha * static_cast<double>(d))) / a.alpha;
    shift[static_cast<std::size_t>(d)] = static_cast<std::int64_t>(round_up ? std::ceil(v - 1e-12) : std::floor(v + 1e-12));
  }
  const std::int64_t out_hi = std::max(amax, bmax) + shift[0];
  const std::size_t n = static_cast<std::size_t>(out_hi - lo + 1);
  out.lower = lo;
  out.p.assign(n, 0.0);
  const std::int64_t na = static_cast<std::int64_t>(a.p.size()), nb = static_cast<std::int64_t>(b.p.size());
#pragma omp parallel
  {
    std::vector<double> local(n, 0.0);
#pragma omp for schedule(dynamic, 64) nowait
    for (std::int64_t i = 0; i < na; ++i) {
      const double pa = a.p[static_cast<std::size_t>(i)];
      if (pa == 0.0) continue;
      const std::int64_t vi = a.lower + i;
      for (std::int64_t j = 0; j < nb; ++j) {
        const double pb = b.p[static_cast<std::size_t>(j)];
        if (pb == 0.0) continue;
        const std::int64_t vj = b.lower + j;
        const std::int64_t d = vi > vj ? vi - vj : vj - vi;
        local[static_cast<std::size_t>(std::max(vi, vj) + shift[static_cast<std::size_t>(d)] - lo)] += pa * pb;
      }
    }
#pragma omp critical
    for (std::size_t k = 0; k < n; ++k) out.p[k] += local[k];
  }
  // a zero on one side leaves the other side's value unchanged
  if (b.zero_mass > 0.0)
    for (std::int64_t i = 0; i < na; ++i) out.p[static_cast<std::size_t>(a.lower + i - lo)] += b.zero_mass * a.p[static_cast<std::size_t>(i)];
  if (a.zero_mass > 0.0)
    for (std::int64_t j = 0; j < nb; ++j) out.p[static_cast<std::size_t>(b.lower + j - lo)] += a.zero_mass * b.p[static_cast<std::size_t>(j)];
  // trim tails (directed): upper tail -> infinity when rounding up, else onto the last kept point; lower tail onto
  // the first kept point when rounding up, else to zero
  std::size_t first = 0, last = n;
  double acc = 0.0;
  while (first + 1 < last && acc + out.p[first] <= beta) acc += out.p[first++];
  if (round_up) out.p[first] += acc; else out.zero_mass += acc;
  double top = 0.0;
  while (last > first + 1 && top + out.p[last - 1] <= beta) top += out.p[--last];
  if (round_up) out.inf_mass += top; else out.p[last - 1] += top;
  out.p = std::vector<double>(out.p.begin() + static_cast<std::ptrdiff_t>(first), out.p.begin() + static_cast<std::ptrdiff_t>(last));
  out.lower = lo + static_cast<std::int64_t>(first);
  return out;
}

GeomPmf geom_self_conv(const GeomPmf& base, std::size_t times, bool round_up, double beta) {
  GeomPmf result;
  bool have = false;
  GeomPmf pw = base;
  std::size_t n = times;
  while (n > 0) {
    if (n & 1) {
      result = have ? geom_conv(result, pw, round_up, beta) : pw;
      have = true;
    }
    n >>= 1;
    if (n) pw = geom_conv(pw, pw, round_up, beta);
  }
  return result;
}

// loss = sign * (alpha * idx - log t), rounded UP onto the output grid
Pmf geom_to_loss_pmf(const GeomPmf& g, double t, double sign, double out_disc, std::size_t max_grid, double extra_inf) {
  Pmf pmf;
  pmf.discretization = out_disc;
  pmf.max_grid_size = max_grid;
  pmf.infinity_mass = extra_inf;
  if (g.p.empty()) return pmf;
  const double logt = std::log(t);
  std::int64_t lo = std::numeric_limits<std::int64_t>::max(), hi = std::numeric_limits<std::int64_t>::min();
  std::vector<std::int64_t> idx(g.p.size());
  for (std::size_t i = 0; i < g.p.size(); ++i) {
    const double loss = sign * (g.alpha * static_cast<double>(g.lower + static_cast<std::int64_t>(i)) - logt);
    idx[i] = static_cast<std::int64_t>(std::ceil(loss / out_disc - 1e-9));
    lo = std::min(lo, idx[i]);
    hi = std::max(hi, idx[i]);
  }
  pmf.lower = lo;
  pmf.probs.assign(static_cast<std::size_t>(hi - lo + 1), 0.0);
  for (std::size_t i = 0; i < g.p.size(); ++i) pmf.probs[static_cast<std::size_t>(idx[i] - lo)] += g.p[i];
  return pmf.maybe_coarsen();
}

Pld single_allocation_pld(double sigma, std::size_t t, const Config& cfg) {
  const double mu = 0.5 / (sigma * sigma), var = 2.0 * mu;
  const double beta_total = std::min(0.49, std::max(1e-300, 0.5 * std::exp(cfg.log_mass_truncation_bound)));
  const double beta = std::min(0.49, std::max(1e-300, beta_total / static_cast<double>(t)));
  const double span = 2.0 * std::sqrt(var) * (-norm_ppf(beta));
  const double alpha = std::max(cfg.discretization, span / static_cast<double>(cfg.max_conv_grid));
  // remove: E = e^{L0} + sum_{t-1} e^{-L~},  everything rounded up
  GeomPmf eL, eD;
  eL.alpha = eD.alpha = alpha;
  double tail;
  disc_normal(mu, var, alpha, beta, eL.lower, eL.p, tail);
  eL.inf_mass = tail;
  disc_normal(-mu, var, alpha, beta, eD.lower, eD.p, tail);
  eD.inf_mass = tail;
  GeomPmf rem = t == 1 ? eL : geom_conv(geom_self_conv(eD, t - 1, true, beta), eL, true, beta);
  Pld out;
  out.remove = geom_to_loss_pmf(rem, static_cast<double>(t), 1.0, cfg.discretization, cfg.max_grid_size, rem.inf_mass);
  // add: S = sum_t e^{-L}, L ~ N(mu, var) rounded UP (so e^{-L} is rounded down), S rounded down; loss = -ln(S/t)
  GeomPmf eN;
  eN.alpha = alpha;
  std::int64_t lo;
  std::vector<double> probs;
  disc_normal(mu, var, alpha, beta, lo, probs, tail);
  // value e^{-alpha j}: index -j; reverse the array
  eN.lower = -(lo + static_cast<std::int64_t>(probs.size()) - 1);
  eN.p.assign(probs.rbegin(), probs.rend());
  eN.zero_mass = tail;                      // L = +infinity  ->  e^{-L} = 0
  GeomPmf s = geom_self_conv(eN, t, false, beta);
  out.add = geom_to_loss_pmf(s, static_cast<double>(t), -1.0, cfg.discretization, cfg.max_grid_size, s.zero_mass);
  return out;
}

}  // namespace

Pld random_allocation_gaussian_pld(double nm, std::size_t t, std::size_t k, const Config& cfg) {
  check_nm(nm);
  require(t >= 1 && k >= 1 && k <= t, "random allocation: need 1 <= k <= t");
  const std::size_t t_floor = t / k, t_ceil = (t + k - 1) / k;
  const std::size_t m_c = t_floor == t_ceil ? 0 : t - t_floor * k, m_f = k - m_c;
  std::optional<Pld> out;
  const std::pair<std::size_t, std::size_t> parts[2] = {{m_f, t_floor}, {m_c, t_ceil}};
  for (const auto& [rounds, steps] : parts) {
    if (rounds == 0 || steps == 0) continue;
    Pld single = single_allocation_pld(nm, steps, cfg);
    Pld composed = rounds == 1 ? single : single.self_compose(rounds);
    out = out ? out->compose(composed, cfg.tail_mass_truncation) : composed;
  }
  const double tail = cfg.tail_mass_truncation / 2.0;
  return out->with_tail_budgets(tail, tail);
}

// Monte-Carlo PLD of a matrix mechanism under balls-in-bins participation: one record takes part in the
// steps {b, b + num_bins, ...} for a uniformly random bin b.  With Gram matrix X = C^T C the privacy loss
// at noise z ~ N(0, I) against the mixture over bins is estimated from samples; the PMF is built from the
// empirical losses rounded up to the grid, and the sampling error is charged to the infinity mass.
Pld balls_in_bins_mc_pld(const std::vector<double>& gram, std::size_t n, std::size_t num_bins, double nm,
                         const Config& cfg) {
  check_nm(nm);
  require(gram.size() == n * n && num_bins >= 1 && num_bins <= n, "balls-in-bins: bad gram matrix / bins");
  // column sums m_b = sum over the steps of bin b of columns of C are represented through X only:
  //   <m_a, m_b> = sum_{i in a, j in b} X_ij.   Sample z in the span of {m_b} via a Cholesky factor of that
  // small num_bins x num_bins Gram matrix.
  const std::size_t B = num_bins;
  std::vector<double> G(B * B, 0.0);
  for (std::size_t i = 0; i < n; ++i)
    for (std::size_t j = 0; j < n; ++j) G[(i % B) * B + (j % B)] += gram[i * n + j];
  std::vector<double> L(B * B, 0.0);
  for (std::size_t i = 0; i < B; ++i)
    for (std::size_t j = 0; j <= i; ++j) {
      double s = G[i * B + j];
      for (std::size_t k = 0; k < j; ++k) s -= L[i * B + k] * L[j * B + k];
      if (i == j) L[i * B + i] = std::sqrt(std::max(s, 1e-300));
      else L[i * B + j] = s / L[j * B + j];
    }
  const double sigma = nm;
  const std::size_t S = cfg.num_mc_samples;
  std::vector<double> losses_remove(S), losses_add(S);
  std::mt19937_64 rng(cfg.seed);
  std::normal_distribution<double> nd(0.0, 1.0);
  std::uniform_int_distribution<std::size_t> ud(0, B - 1);
  std::vector<double> xi(B), proj(B), t(B);
  for (std::size_t s = 0; s < S; ++s) {
    for (auto& v : xi) v = nd(rng);
    // proj_b = <m_b, noise> / sigma  with noise = sigma * N(0, I):  coordinates L xi
    for (std::size_t b = 0; b < B; ++b) {
      double a = 0.0;
      for (std::size_t k = 0; k <= b; ++k) a += L[b * B + k] * xi[k];
      proj[b] = a;
    }
    const std::size_t b0 = ud(rng);
    // REMOVE: data present in bin b0: observation = m_b0 + sigma z.  loss = log( mean_b exp(...) )
    for (std::size_t b = 0; b < B; ++b)
      t[b] = (G[b * B + b0] + sigma * proj[b]) / (sigma * sigma) - 0.5 * G[b * B + b] / (sigma * sigma);
    losses_remove[s] = log_sumexp(t) - std::log(static_cast<double>(B));
    // ADD: data absent: observation = sigma z; loss = -log( mean_b exp(...) )
    for (std::size_t b = 0; b < B; ++b) t[b] = proj[b] / sigma - 0.5 * G[b * B + b] / (sigma * sigma);
    losses_add[s] = -(log_sumexp(t) - std::log(static_cast<double>(B)));
  }
  auto to_pmf = [&](std::vector<double>& v) {
    Pmf p;
    p.discretization = cfg.discretization;
    p.max_grid_size = cfg.max_grid_size;
    std::int64_t lo = std::numeric_limits<std::int64_t>::max(), hi = std::numeric_limits<std::int64_t>::min();
    std::vector<std::int64_t> idx(v.size());
    for (std::size_t i = 0; i < v.size(); ++i) {
      idx[i] = static_cast<std::int64_t>(std::ceil(v[i] / cfg.discretization));
      lo = std::min(lo, idx[i]);
      hi = std::max(hi, idx[i]);
    }
    p.lower = lo;
    p.probs.assign(static_cast<std::size_t>(hi - lo + 1), 0.0);
    const double w = 1.0 / static_cast<double>(v.size());
    for (auto i : idx) p.probs[static_cast<std::size_t>(i - lo)] += w;
    return p.maybe_coarsen();
  };
  Pld out;
  out.remove = to_pmf(losses_remove);
  out.add = to_pmf(losses_add);
  return out;
}

// Monte-Carlo PLD of a banded matrix mechanism under b-min-sep participation (Dong & Ganesh, "Privacy amplification
// for BandMF via b-min-sep subsampling"): a record that is free takes part in a step with probability p and is then
// barred for the next b - 1 steps.  With a strategy whose columns have at most b non-zeros (c_0..c_{L-1}, L <= b) the
// columns of two participations never overlap, so the likelihood ratio of an output y against the null factorises and
// obeys the backward recursion
//     f_n = 1,   f_i = (1 - p) f_{i+1} + p exp((<c, y_{i:i+L}> - |c_{:n-i}|^2 / 2) / sigma^2) f_{min(i+b, n)}
// with P(y)/Q(y) = f_0 for a cold start (every record free at step 0).  With a warm start (the chain of
// free / barred states started in its stationary law) P/Q = (f_0 + p (f_1 + ... + f_{b-1})) / (1 + (b-1) p).
// Losses ln(P/Q) under P (remove) and -ln(P/Q) under Q (add) are sampled and rounded UP onto the grid.
namespace {

// One record's transcript for b-min-sep, independent of the noise multiplier: the participation pattern x, the unit
// normals of the P branch and of the Q branch.  Each of the three comes from its own generator, seeded from
// (seed, sample), so the first m columns of an n-step transcript ARE the m-step transcript of the same sample.
struct BmsStreams {
  std::mt19937_64 rx, rp, rq;
  BmsStreams(std::uint64_t seed, std::uint64_t sample) {
    const std::uint64_t base = seed + 0x9E3779B97F4A7C15ULL * (sample + 1);
    rx.seed(base ^ 0xA24BAED4963EE407ULL);
    rp.seed(base ^ 0x9FB21C651E98DF25ULL);
    rq.seed(base ^ 0xD6E8FEB86659FD93ULL);
  }
};

void bms_draw(std::uint64_t seed, std::uint64_t sample, std::size_t n, std::size_t b, double p, bool warm_start,
              std::uint8_t* x, double* zp, double* zq) {
  BmsStreams g(seed, sample);
  std::uniform_real_distribution<double> ud(0.0, 1.0);
  std::normal_distribution<double> np(0.0, 1.0), nq(0.0, 1.0);
  const double denom = 1.0 + static_cast<double>(b - 1) * p;
  std::size_t barred = 0;
  if (warm_start && b > 1 && ud(g.rx) * denom >= 1.0)
    barred = 1 + static_cast<std::size_t>(ud(g.rx) * static_cast<double>(b - 1)) % (b - 1);
  for (std::size_t i = 0; i < n; ++i) {
    const bool take = barred == 0 && ud(g.rx) < p;
    x[i] = take ? 1 : 0;
    barred = take ? b - 1 : (barred > 0 ? barred - 1 : 0);
  }
  for (std::size_t i = 0; i < n; ++i) zp[i] = np(g.rp);
  for (std::size_t i = 0; i < n; ++i) zq[i] = nq(g.rq);
}

// ln(P/Q) of one observation sequence y (see the recursion above); f is scratch of n + 1 doubles holding log f_i.
double bms_log_ratio(const std::vector<double>& coef, const std::vector<double>& cum, std::size_t n, std::size_t b, double p,
                     double sigma2, bool warm_start, const double* y, double* f) {
  const std::size_t L = coef.size();
  f[n] = 0.0;
  for (std::size_t ii = n; ii-- > 0;) {
    const std::size_t m = std::min(L, n - ii);
    double dot = 0.0;
    for (std::size_t k = 0; k < m; ++k) dot += coef[k] * y[ii + k];
    const double blk = (dot - 0.5 * cum[m]) / sigma2;
    const double skip = f[std::min(ii + b, n)];
    const double a = (p < 1.0) ? std::log1p(-p) + f[ii + 1] : -std::numeric_limits<double>::infinity();
    const double c2 = std::log(p) + blk + skip;
    // log(exp(a) + exp(c2)) with one exp: max + log1p(exp(-|a - c2|)); a = -inf (p = 1) leaves c2
    const double hi = std::max(a, c2), lo = std::min(a, c2);
    f[ii] = std::isinf(lo) ? hi : hi + std::log1p(std::exp(lo - hi));
  }
  if (!warm_start || b == 1) return f[0];
  const double denom = 1.0 + static_cast<double>(b - 1) * p;
  double hi = f[0];
  for (std::size_t j = 1; j < std::min(b, n + 1); ++j) hi = std::max(hi, std::log(p) + f[j]);
  double acc = std::exp(f[0] - hi);
  for (std::size_t j = 1; j < b; ++j) acc += std::exp(std::log(p) + f[std::min(j, n)] - hi);
  return hi + std::log(acc) - std::log(denom);
}

// Both losses of one sample at noise multiplier sigma from its sigma-free transcript.
void bms_losses(const std::vector<double>& coef, const std::vector<double>& cum, std::size_t n, std::size_t b, double p,
                double sigma, bool warm_start, const std::uint8_t* x, const double* zp, const double* zq, double* y,
                double* f, double& loss_remove, double& loss_add) {
  const std::size_t L = coef.size();
  for (std::size_t i = 0; i < n; ++i) {                     // P branch: y = C x + sigma z
    double acc = sigma * zp[i];
    for (std::size_t k = 0; k < L && k <= i; ++k) acc += coef[k] * static_cast<double>(x[i - k]);
    y[i] = acc;
  }
  loss_remove = bms_log_ratio(coef, cum, n, b, p, sigma * sigma, warm_start, y, f);
  for (std::size_t i = 0; i < n; ++i) y[i] = sigma * zq[i];   // Q branch: y = sigma z
  loss_add = -bms_log_ratio(coef, cum, n, b, p, sigma * sigma, warm_start, y, f);
}

Pmf bms_losses_to_pmf(const std::vector<double>& v, const Config& cfg) {
  Pmf q;
  q.discretization = cfg.discretization;
  q.max_grid_size = cfg.max_grid_size;
  std::int64_t lo = std::numeric_limits<std::int64_t>::max(), hi = std::numeric_limits<std::int64_t>::min();
  std::vector<std::int64_t> idx(v.size());
  for (std::size_t i = 0; i < v.size(); ++i) {
    idx[i] = static_cast<std::int64_t>(std::ceil(v[i] / cfg.discretization));
    lo = std::min(lo, idx[i]);
    hi = std::max(hi, idx[i]);
  }
  q.lower = lo;
  q.probs.assign(static_cast<std::size_t>(hi - lo + 1), 0.0);
  const double w = 1.0 / static_cast<double>(v.size());
  for (auto i : idx) q.probs[static_cast<std::size_t>(i - lo)] += w;
  return q.maybe_coarsen();
}

std::vector<double> bms_cum(const std::vector<double>& coef) {
  std::vector<double> cum(coef.size() + 1, 0.0);           // |c_{:m}|^2 for a column cut off by the end of the run
  for (std::size_t k = 0; k < coef.size(); ++k) cum[k + 1] = cum[k] + coef[k] * coef[k];
  return cum;
}

void bms_check(const std::vector<double>& coef, std::size_t n, std::size_t b, double p) {
  require(!coef.empty() && n >= 1 && b >= 1 && p > 0.0 && p <= 1.0, "b-min-sep: need coefficients, n >= 1, b >= 1, p in (0, 1]");
  require(coef.size() <= b, "b-min-sep: the strategy's band count must not exceed the minimum separation");
}

}  // namespace

Pld b_min_sep_mc_pld(const std::vector<double>& coef, std::size_t n, std::size_t b, double p, double nm, bool warm_start,
                     const Config& cfg) {
  check_nm(nm);
  bms_check(coef, n, b, p);
  const std::size_t S = cfg.num_mc_samples;
  std::vector<double> losses_remove(S), losses_add(S);
  const std::vector<double> cum = bms_cum(coef);
#pragma omp parallel
  {
    std::vector<std::uint8_t> x(n);
    std::vector<double> zp(n), zq(n), y(n), f(n + 1);
#pragma omp for schedule(static)
    for (std::int64_t s = 0; s < static_cast<std::int64_t>(S); ++s) {
      bms_draw(cfg.seed, static_cast<std::uint64_t>(s), n, b, p, warm_start, x.data(), zp.data(), zq.data());
      bms_losses(coef, cum, n, b, p, nm, warm_start, x.data(), zp.data(), zq.data(), y.data(), f.data(),
                 losses_remove[static_cast<std::size_t>(s)], losses_add[static_cast<std::size_t>(s)]);
    }
  }
  Pld out;
  out.remove = bms_losses_to_pmf(losses_remove, cfg);
  out.add = bms_losses_to_pmf(losses_add, cfg);
  return out;
}

// --------------------------------------------------------------------------- stored transcripts
BMinSepCorpus::BMinSepCorpus(std::vector<double> coef_, std::size_t n_steps_, std::size_t min_sep_, double p_, bool warm_,
                             std::size_t samples_, std::uint64_t seed_)
    : coef(std::move(coef_)), n_steps(n_steps_), min_sep(min_sep_), sampling_prob(p_), warm_start(warm_),
      num_samples(samples_), seed(seed_) {
  bms_check(coef, n_steps, min_sep, sampling_prob);
  require(num_samples >= 1, "b-min-sep corpus: need at least one sample");
  x.resize(num_samples * n_steps);
  zp.resize(num_samples * n_steps);
  zq.resize(num_samples * n_steps);
#pragma omp parallel for schedule(static)
  for (std::int64_t s = 0; s < static_cast<std::int64_t>(num_samples); ++s) {
    const std::size_t o = static_cast<std::size_t>(s) * n_steps;
    bms_draw(seed, static_cast<std::uint64_t>(s), n_steps, min_sep, sampling_prob, warm_start, &x[o], &zp[o], &zq[o]);
  }
}

std::size_t BMinSepCorpus::nbytes() const {
  return x.size() * sizeof(std::uint8_t) + (zp.size() + zq.size()) * sizeof(double);
}

Pld BMinSepCorpus::pld(double nm, std::size_t n_prefix, const Config& cfg) const {
  check_nm(nm);
  require(n_prefix >= 1 && n_prefix <= n_steps, "b-min-sep corpus: the queried horizon exceeds the stored one");
  std::vector<double> losses_remove(num_samples), losses_add(num_samples);
  const std::vector<double> cum = bms_cum(coef);
#pragma omp parallel
  {
    std::vector<double> y(n_prefix), f(n_prefix + 1);
#pragma omp for schedule(static)
    for (std::int64_t s = 0; s < static_cast<std::int64_t>(num_samples); ++s) {
      const std::size_t o = static_cast<std::size_t>(s) * n_steps;
      bms_losses(coef, cum, n_prefix, min_sep, sampling_prob, nm, warm_start, &x[o], &zp[o], &zq[o], y.data(), f.data(),
                 losses_remove[static_cast<std::size_t>(s)], losses_add[static_cast<std::size_t>(s)]);
    }
  }
  Pld out;
  out.remove = bms_losses_to_pmf(losses_remove, cfg);
  out.add = bms_losses_to_pmf(losses_add, cfg);
  return out;
}

double adaclip_effective_noise_multiplier(double z, double fraction_noise_std, double expected_batch, int groups) {
  require(z > 0.0 && fraction_noise_std > 0.0 && expected_batch > 0.0 && groups >= 1, "adaclip: bad parameters");
  const double sigma_b = expected_batch * fraction_noise_std;
  return 1.0 / std::sqrt(1.0 / (z * z) + static_cast<double>(groups) / (4.0 * sigma_b * sigma_b));
}

// =============================================================================== MF sensitivities

std::int64_t minsep_true_max_participations(std::int64_t n, std::int64_t min_sep, std::int64_t max_part) {
  require(n >= 0 && min_sep >= 1, "min_sep must be >= 1");
  const std::int64_t ub = (n + min_sep - 1) / min_sep;
  return max_part > 0 ? std::min(ub, max_part) : ub;
}

double max_participation_for_linear_fn(const std::vector<double>& x, std::int64_t min_sep, std::int64_t max_part) {
  const std::int64_t n = static_cast<std::int64_t>(x.size());
  if (n == 0) return 0.0;
  const std::int64_t k = minsep_true_max_participations(n, min_sep, max_part);
  if (k == 0) return 0.0;
  std::vector<double> f(static_cast<std::size_t>(n + min_sep), 0.0);
  for (std::int64_t r = 0; r < k; ++r) {
    for (std::int64_t i = 0; i < n; ++i) f[static_cast<std::size_t>(i)] = x[static_cast<std::size_t>(i)] + f[static_cast<std::size_t>(i + min_sep)];
    for (std::int64_t i = n + min_sep - 2; i >= 0; --i)
      f[static_cast<std::size_t>(i)] = std::max(f[static_cast<std::size_t>(i)], f[static_cast<std::size_t>(i + 1)]);
  }
  return f[0];
}

double sens_sq_single_participation(const std::vector<double>& gram, std::size_t n) {
  require(gram.size() == n * n && n > 0, "gram matrix must be n x n");
  double m = 0.0;
  for (std::size_t i = 0; i < n; ++i) m = std::max(m, gram[i * n + i]);
  return m;
}

double sens_sq_minsep_upper_bound(const std::vector<double>& gram, std::size_t n, std::int64_t min_sep,
                                  std::int64_t max_part) {
  require(gram.size() == n * n && n > 0, "gram matrix must be n x n");
  std::vector<double> row_max(n), row(n);
  for (std::size_t i = 0; i < n; ++i) {
    for (std::size_t j = 0; j < n; ++j) row[j] = std::fabs(gram[i * n + j]);
    row_max[i] = max_participation_for_linear_fn(row, min_sep, max_part);
  }
  return max_participation_for_linear_fn(row_max, min_sep, max_part);
}

double sens_sq_banded(const std::vector<double>& gram, std::size_t n, std::int64_t bands, std::int64_t min_sep,
                      std::int64_t max_part) {
  require(gram.size() == n * n && n > 0, "gram matrix must be n x n");
  require(min_sep >= bands, "banded sensitivity needs min_sep >= bands (columns of distinct participations are orthogonal)");
  std::vector<double> diag(n);
  for (std::size_t i = 0; i < n; ++i) diag[i] = gram[i * n + i];
  return max_participation_for_linear_fn(diag, min_sep, max_part);
}

double sens_sq_fixed_epoch(const std::vector<double>& gram, std::size_t n, std::int64_t epochs) {
  require(gram.size() == n * n && n > 0 && epochs > 0 && n % static_cast<std::size_t>(epochs) == 0,
          "fixed epoch sensitivity: epochs must divide n");
  const std::size_t per = n / static_cast<std::size_t>(epochs);
  double best = 0.0;
  for (std::size_t c = 0; c < per; ++c) {
    double s = 0.0;
    for (std::size_t a = 0; a < static_cast<std::size_t>(epochs); ++a)
      for (std::size_t b = 0; b < static_cast<std::size_t>(epochs); ++b) s += std::fabs(gram[(a * per + c) * n + (b * per + c)]);
    best = std::max(best, s);
  }
  return best;
}

double toeplitz_minsep_sens_sq(const std::vector<double>& coef_in, std::int64_t n, std::int64_t min_sep,
                               std::int64_t max_part) {
  require(n > 0 && min_sep >= 1, "toeplitz sensitivity: n > 0 and min_sep >= 1");
  for (std::size_t i = 0; i < coef_in.size(); ++i) {
    require(coef_in[i] >= 0.0, "toeplitz coefficients must be non-negative");
    if (i > 0) require(coef_in[i] <= coef_in[i - 1], "toeplitz coefficients must be non-increasing");
  }
  const std::int64_t k = minsep_true_max_participations(n, min_sep, max_part);
  const std::int64_t pad = (min_sep - n % min_sep) % min_sep, len = n + pad;
  std::vector<double> v(static_cast<std::size_t>(len), 0.0);
  for (std::int64_t i = 0; i < std::min<std::int64_t>(n, static_cast<std::int64_t>(coef_in.size())); ++i) v[static_cast<std::size_t>(i)] = coef_in[static_cast<std::size_t>(i)];
  for (std::int64_t blk = 1; blk < len / min_sep; ++blk)
    for (std::int64_t o = 0; o < min_sep; ++o) v[static_cast<std::size_t>(blk * min_sep + o)] += v[static_cast<std::size_t>((blk - 1) * min_sep + o)];
  const std::int64_t ks = k * min_sep;
  if (ks < len) {
    const std::vector<double> saved = v;
    for (std::int64_t i = ks; i < len; ++i) v[static_cast<std::size_t>(i)] = saved[static_cast<std::size_t>(i)] - saved[static_cast<std::size_t>(i - ks)];
  }
  double s = 0.0;
  for (std::int64_t i = 0; i < n; ++i) s += v[static_cast<std::size_t>(i)] * v[static_cast<std::size_t>(i)];
  return s;
}

namespace {
double geometric_sum(double a, double r, double num) {
  if (std::isinf(num)) return a / (1.0 - r);
  const double thr = 1.0 - std::pow(10.0, -(3.33503185 + 0.53018965 * std::log(num)));
  if (r < thr) return a * (1.0 - std::pow(r, num)) / (1.0 - r);
  const double x0 = num - 1.0, x1 = r - 1.0;
  return (1.0 / 6.0) * a * num * (x0 * x1 * x1 * (num - 2.0) + 3.0 * x0 * x1 + 6.0);
}
}  // namespace

std::vector<double> toeplitz_gram(const std::vector<double>& coef, std::size_t n) {
  // X = C^T C for lower-triangular Toeplitz C with first column coef (zero padded): X_ij = sum_t c_{t-i} c_{t-j}
  std::vector<double> c(n, 0.0);
  for (std::size_t i = 0; i < std::min(n, coef.size()); ++i) c[i] = coef[i];
  std::vector<double> X(n * n, 0.0);
  for (std::size_t i = 0; i < n; ++i)
    for (std::size_t j = i; j < n; ++j) {
      double s = 0.0;
      for (std::size_t t = j; t < n; ++t) s += c[t - i] * c[t - j];
      X[i * n + j] = X[j * n + i] = s;
    }
  return X;
}

double blt_sens_sq(const std::vector<double>& scale, const std::vector<double>& decay, std::int64_t n,
                   std::int64_t min_sep, std::int64_t max_part) {
  require(scale.size() == decay.size(), "BLT: scale and decay must have the same length");
  // Toeplitz coefficients t_0 = 1, t_k = sum_j s_j d_j^{k-1}
  std::vector<double> coef(static_cast<std::size_t>(n), 0.0);
  coef[0] = 1.0;
  std::vector<double> pw(scale.begin(), scale.end());
  for (std::int64_t k = 1; k < n; ++k) {
    double t = 0.0;
    for (std::size_t j = 0; j < pw.size(); ++j) {
      t += pw[j];
      pw[j] *= decay[j];
    }
    coef[static_cast<std::size_t>(k)] = t;
  }
  const std::int64_t kmax = minsep_true_max_participations(n, min_sep, max_part);
  if (kmax <= 1) {
    // single participation: squared norm of the first column, closed form (Lemma 5.3 style geometric sums)
    double total = 0.0;
    for (std::size_t i = 0; i < scale.size(); ++i)
      for (std::size_t j = 0; j < scale.size(); ++j)
        total += geometric_sum(scale[i] * scale[j], decay[i] * decay[j], static_cast<double>(n - 1));
    return 1.0 + total;
  }
  bool monotone = true;
  for (std::size_t i = 0; i < coef.size(); ++i)
    if (coef[i] < 0.0 || (i > 0 && coef[i] > coef[i - 1] + 1e-15)) monotone = false;
  if (monotone) {
    for (std::size_t i = 1; i < coef.size(); ++i) coef[i] = std::min(coef[i], coef[i - 1]);
    return toeplitz_minsep_sens_sq(coef, n, min_sep, max_part);
  }
  return sens_sq_minsep_upper_bound(toeplitz_gram(coef, static_cast<std::size_t>(n)), static_cast<std::size_t>(n), min_sep, max_part);
}

}  // namespace obacc
