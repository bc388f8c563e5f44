// Privacy-loss-distribution (PLD) accountant core, C++17, CPU only.
//
// A mechanism is represented by pessimistic discretised privacy-loss PMFs on a uniform grid
// (spacing `discretization`) for the REMOVE direction and, when the mechanism is not symmetric, the
// ADD direction.  PMFs are built from a hockey-stick oracle delta(eps) with the "connect the dots"
// construction (Doroshenko et al.), composed by FFT convolution and self-composed by
// IFFT(FFT^k) inside a Chernoff-bounded output window whose discarded tail is moved to the
// infinity mass (so results stay upper bounds).
//
// Parity: packages/opaque-accounting/src/{discretization/connect_the_dots.rs, pld/pmf/dense.rs,
// pld/metrics.rs, numerics/{fft,truncation,logspace,special}.rs, amplification/*.rs,
// matrix_factorization/sensitivity.rs, transformations/adaclip.rs}.
#pragma once
#include <cstdint>
#include <functional>
#include <optional>
#include <string>
#include <vector>

namespace obacc {

struct Config {
  double discretization = 1e-4;
  double log_mass_truncation_bound = -50.0;
  std::size_t max_grid_size = 10'000'000;
  double tail_mass_truncation = 1e-15;
  std::size_t max_conv_grid = 32768;
  std::size_t num_mc_samples = 100000;
  std::uint64_t seed = 42;
  // true: rescale a discretised PMF to unit mass (what the reference library's pinned values contain; lowers delta by
  // ~1e-8 relative); false: remove surplus mass from the lowest losses only, which keeps delta an upper bound
  bool proportional_normalization = false;
};

enum class Adjacency { Remove = 0, Add = 1, Replace = 2 };

struct EpsBounds {
  double lo, hi;
};

struct Pmf {
  double discretization = 1e-4;
  std::int64_t lower = 0;              // grid index of probs[0]: loss = (lower + i) * discretization
  std::vector<double> probs;
  double infinity_mass = 0.0;
  double neg_infinity_mass = 0.0;
  std::size_t max_grid_size = 10'000'000;
  double right_budget = 0.0, left_budget = 0.0;   // tail mass a self-composition may discard

  double loss_at(std::int64_t i) const { return static_cast<double>(lower + i) * discretization; }
  double delta_at(double eps) const;
  double epsilon_at(double delta) const;
  Pmf compose(const Pmf& other, double tail_mass_truncation) const;
  Pmf self_compose(std::size_t count) const;
  Pmf coarsen(std::size_t factor) const;
  Pmf maybe_coarsen() const;
};

struct Pld {
  Pmf remove;
  std::optional<Pmf> add;

  bool symmetric() const { return !add.has_value(); }
  double delta_at(double eps) const;
  double epsilon_at(double delta) const;
  double infinity_mass() const;
  double advantage() const { return delta_at(0.0); }
  double beta_at(double alpha) const;       // trade-off curve: type-II error at type-I error alpha
  double risk_at(double prior) const;       // Bayes risk of the best membership test at a prior
  Pld compose(const Pld& other, double tail_mass_truncation = 1e-15) const;
  Pld self_compose(std::size_t count) const;
  Pld with_tail_budgets(double right, double left) const;
};

// ---- numerics -------------------------------------------------------------------------------------
double norm_cdf(double z);
double norm_log_cdf(double z);
double norm_ppf(double p);
double log_add(double a, double b);
double log_sub(double a, double b);
double log_sumexp(const std::vector<double>& v);
double log_a_times_exp_b_plus_c(double a, double b, double c);
std::vector<double> convolve(const std::vector<double>& a, const std::vector<double>& b);

// ---- builders ---------------------------------------------------------------------------------------
Pmf connect_the_dots(const std::vector<double>& deltas, std::int64_t lo_idx, double disc, std::size_t max_grid,
                     bool proportional_normalization = false);
Pld discretize(const Config& cfg, EpsBounds remove_b, std::optional<EpsBounds> add_b,
               const std::function<double(double, Adjacency)>& delta_fn);

Pld gaussian_pld(double noise_multiplier, const Config& cfg, double sensitivity = 1.0);
Pld eps_delta_pld(double eps, double delta, const Config& cfg);
Pld identity_pld(const Config& cfg);
Pld nonprivate_pld(const Config& cfg);
Pld poisson_gaussian_pld(double noise_multiplier, double rate, const Config& cfg);
Pld truncated_poisson_gaussian_pld(double noise_multiplier, double rate, std::int64_t truncated_batch_size,
                                   std::int64_t dataset_size, const Config& cfg);
Pld parallel_poisson_gaussian_pld(double noise_multiplier, double rate, std::size_t workers, const Config& cfg);
Pld mixture_gaussian_pld(double sigma, const std::vector<double>& log_probs, const std::vector<double>& sens,
                         double head_mass, double tail_mass, const Config& cfg);
Pld random_allocation_gaussian_pld(double noise_multiplier, std::size_t num_bins, std::size_t k, const Config& cfg);
Pld b_min_sep_mc_pld(const std::vector<double>& coef, std::size_t n, std::size_t b, double p, double noise_multiplier,
                     bool warm_start, const Config& cfg);

// Noise-multiplier-free Monte-Carlo transcripts of b-min-sep (participation patterns and unit normals of both
// branches), kept so that a calibration search evaluates many noise multipliers on ONE set of samples.  A query may
// use any prefix n <= n_steps of the stored horizon: it equals a fresh corpus of that length with the same seed.
// pld(nm, n_steps, cfg) equals b_min_sep_mc_pld(...) with cfg.seed == seed and cfg.num_mc_samples == num_samples.
// Parity: packages/opaque-accounting/src/amplification/b_min_sep/registry.rs of the reference (handles to stored
// corpora, K-prefix queries); here the corpus is a C++ object owned by Python.
struct BMinSepCorpus {
  std::vector<double> coef;
  std::size_t n_steps, min_sep;
  double sampling_prob;
  bool warm_start;
  std::size_t num_samples;
  std::uint64_t seed;
  std::vector<std::uint8_t> x;     // [num_samples * n_steps]
  std::vector<double> zp, zq;      // [num_samples * n_steps] each

  BMinSepCorpus(std::vector<double> coef, std::size_t n_steps, std::size_t min_sep, double sampling_prob, bool warm_start,
                std::size_t num_samples, std::uint64_t seed);
  std::size_t nbytes() const;
  Pld pld(double noise_multiplier, std::size_t n_prefix, const Config& cfg) const;
};
Pld balls_in_bins_mc_pld(const std::vector<double>& gram_row_major, std::size_t n, std::size_t num_bins,
                         double noise_multiplier, const Config& cfg);

double gaussian_delta(double noise_multiplier, double eps, double sensitivity = 1.0);
double adaclip_effective_noise_multiplier(double z, double fraction_noise_std, double expected_batch, int groups);

// ---- matrix-factorisation sensitivities -----------------------------------------------------------
// All take the Gram matrix X = C^T C (row-major n x n) or Toeplitz coefficients of C.
std::int64_t minsep_true_max_participations(std::int64_t n, std::int64_t min_sep, std::int64_t max_part);
double max_participation_for_linear_fn(const std::vector<double>& x, std::int64_t min_sep, std::int64_t max_part);
double sens_sq_single_participation(const std::vector<double>& gram, std::size_t n);
double sens_sq_minsep_upper_bound(const std::vector<double>& gram, std::size_t n, std::int64_t min_sep,
                                  std::int64_t max_part);
double sens_sq_banded(const std::vector<double>& gram, std::size_t n, std::int64_t bands, std::int64_t min_sep,
                      std::int64_t max_part);
double sens_sq_fixed_epoch(const std::vector<double>& gram, std::size_t n, std::int64_t epoch_len);
double toeplitz_minsep_sens_sq(const std::vector<double>& coef, std::int64_t n, std::int64_t min_sep,
                               std::int64_t max_part);
double blt_sens_sq(const std::vector<double>& scale, const std::vector<double>& decay, std::int64_t n,
                   std::int64_t min_sep, std::int64_t max_part);
std::vector<double> toeplitz_gram(const std::vector<double>& coef, std::size_t n);

// ---- Toeplitz-column strategies, optionally column-normalised (mf.cpp): lambda-CGD, banded inverse square root ----
// max_part < 0 means "as many as min_sep allows".
std::vector<double> inverse_toeplitz_coefficients(const std::vector<double>& taps, std::size_t n);
double toeplitz_columns_sens_sq(const std::vector<double>& coef, std::size_t n, std::int64_t min_sep, std::int64_t max_part,
                                bool normalized);
std::vector<double> toeplitz_columns_bnb_gram(const std::vector<double>& coef, std::size_t n, std::int64_t min_sep,
                                              std::int64_t max_part, bool normalized, double momentum,
                                              const std::vector<double>* lr_weights);
double lambda_cgd_sens_sq(double lambda, std::size_t n, std::int64_t min_sep, std::int64_t max_part, bool normalized);
double lambda_cgd_max_column_norm(double lambda, std::size_t n);
std::vector<double> lambda_cgd_bnb_gram(double lambda, std::size_t n, std::int64_t min_sep, std::int64_t max_part,
                                        bool normalized, double momentum, const std::vector<double>* lr_weights);

}  // namespace obacc
