// pybind11 surface of the C++ PLD accountant (module ``opaque_b200.accounting._native``).
// Parity: packages/opaque-accounting/src/python/*.rs and core/opaque_accounting.pyi.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "pld.hpp"

namespace py = pybind11;
using namespace obacc;

namespace {
std::int64_t opt_int(const py::object& o) { return o.is_none() ? 0 : o.cast<std::int64_t>(); }
}  // namespace

PYBIND11_MODULE(_native, m) {
  m.doc() = "C++ privacy-loss-distribution accountant";

  py::class_<Config>(m, "DiscretizationConfig")
      .def(py::init([](double disc, double log_mass, std::size_t max_grid, double tail, std::size_t max_conv,
                       std::size_t mc, std::uint64_t seed, bool proportional) {
             if (!(disc > 0.0)) throw std::invalid_argument("discretization must be > 0");
             if (!(tail >= 0.0 && tail < 1.0)) throw std::invalid_argument("tail_mass_truncation must be in [0, 1)");
             Config c;
             c.discretization = disc; c.log_mass_truncation_bound = log_mass; c.max_grid_size = max_grid;
             c.tail_mass_truncation = tail; c.max_conv_grid = max_conv; c.num_mc_samples = mc; c.seed = seed;
             c.proportional_normalization = proportional;
             return c;
           }),
           py::arg("discretization") = 1e-4, py::arg("log_mass_truncation_bound") = -50.0,
           py::arg("max_grid_size") = 10'000'000, py::arg("tail_mass_truncation") = 1e-15,
           py::arg("max_conv_grid") = 32768, py::arg("num_mc_samples") = 100000, py::arg("seed") = 42,
           py::arg("proportional_normalization") = false)
      .def_readwrite("discretization", &Config::discretization)
      .def_readwrite("log_mass_truncation_bound", &Config::log_mass_truncation_bound)
      .def_readwrite("max_grid_size", &Config::max_grid_size)
      .def_readwrite("tail_mass_truncation", &Config::tail_mass_truncation)
      .def_readwrite("max_conv_grid", &Config::max_conv_grid)
      .def_readwrite("num_mc_samples", &Config::num_mc_samples)
      .def_readwrite("seed", &Config::seed)
      .def_readwrite("proportional_normalization", &Config::proportional_normalization);

  py::class_<Pld>(m, "Pld")
      .def("epsilon_at", &Pld::epsilon_at, py::arg("delta"))
      .def("delta_at", &Pld::delta_at, py::arg("epsilon"))
      .def("infinity_mass", &Pld::infinity_mass)
      .def("advantage", &Pld::advantage)
      .def("beta_at", &Pld::beta_at, py::arg("alpha"))
      .def("risk_at", &Pld::risk_at, py::arg("prior"))
      .def("is_symmetric", &Pld::symmetric)
      .def("compose", [](const Pld& a, const Pld& b) { py::gil_scoped_release r; return a.compose(b); })
      .def("self_compose", [](const Pld& a, std::size_t n) { py::gil_scoped_release r; return a.self_compose(n); })
      .def("__or__", [](const Pld& a, const Pld& b) { py::gil_scoped_release r; return a.compose(b); })
      .def("__mul__", [](const Pld& a, std::size_t n) { py::gil_scoped_release r; return a.self_compose(n); })
      .def("__rmul__", [](const Pld& a, std::size_t n) { py::gil_scoped_release r; return a.self_compose(n); })
      .def_property_readonly("grid_size", [](const Pld& p) { return p.remove.probs.size(); })
      .def_property_readonly("discretization", [](const Pld& p) { return p.remove.discretization; })
      .def("pmf", [](const Pld& p, bool add) {
        const Pmf& q = (add && p.add) ? *p.add : p.remove;
        return py::make_tuple(q.lower, q.discretization, q.probs, q.infinity_mass);
      }, py::arg("add") = false);

  m.def("gaussian_pld", [](double nm, const Config& c) { py::gil_scoped_release r; return gaussian_pld(nm, c); });
  m.def("gaussian_delta", &gaussian_delta, py::arg("noise_multiplier"), py::arg("epsilon"), py::arg("sensitivity") = 1.0);
  m.def("eps_delta_pld", &eps_delta_pld);
  m.def("identity_pld", &identity_pld);
  m.def("nonprivate_pld", &nonprivate_pld);
  m.def("poisson_gaussian_pld", [](double nm, double q, const Config& c) { py::gil_scoped_release r; return poisson_gaussian_pld(nm, q, c); });
  m.def("truncated_poisson_gaussian_pld", [](double nm, double q, std::int64_t b, std::int64_t n, const Config& c) {
    py::gil_scoped_release r; return truncated_poisson_gaussian_pld(nm, q, b, n, c); });
  m.def("parallel_poisson_gaussian_pld", [](double nm, double q, std::size_t w, const Config& c) {
    py::gil_scoped_release r; return parallel_poisson_gaussian_pld(nm, q, w, c); });
  m.def("mixture_gaussian_pld", [](double s, std::vector<double> lp, std::vector<double> se, double head, double tail, const Config& c) {
    py::gil_scoped_release r; return mixture_gaussian_pld(s, lp, se, head, tail, c); });
  m.def("random_allocation_gaussian_pld", [](double nm, std::size_t t, std::size_t k, const Config& c) {
    py::gil_scoped_release r; return random_allocation_gaussian_pld(nm, t, k, c); });
  m.def("mf_gaussian_pld", [](double nm, double sensitivity, const Config& c) {
    const double eff = nm / sensitivity;
    if (!(eff >= 0.01 && eff <= 1000.0)) throw std::invalid_argument("effective noise multiplier sigma/sensitivity must be in [0.01, 1000]");
    py::gil_scoped_release r; return gaussian_pld(eff, c); });
  m.def("balls_in_bins_mc_pld", [](std::vector<double> gram, std::size_t n, std::size_t bins, double nm, const Config& c) {
    py::gil_scoped_release r; return balls_in_bins_mc_pld(gram, n, bins, nm, c); });
  m.def("b_min_sep_mc_pld", [](std::vector<double> coef, std::size_t n, std::size_t b, double p, double nm, bool warm, const Config& c) {
    py::gil_scoped_release r; return b_min_sep_mc_pld(coef, n, b, p, nm, warm, c); },
    py::arg("coef"), py::arg("n_steps"), py::arg("min_sep"), py::arg("sampling_prob"), py::arg("noise_multiplier"),
    py::arg("warm_start"), py::arg("config"));
  py::class_<BMinSepCorpus>(m, "BMinSepCorpus")
      .def(py::init([](std::vector<double> coef, std::size_t n, std::size_t b, double p, bool warm, std::size_t samples,
                       std::uint64_t seed) {
             py::gil_scoped_release r;
             return new BMinSepCorpus(std::move(coef), n, b, p, warm, samples, seed);
           }),
           py::arg("coef"), py::arg("n_steps"), py::arg("min_sep"), py::arg("sampling_prob"), py::arg("warm_start"),
           py::arg("num_samples"), py::arg("seed"))
      .def_readonly("n_steps", &BMinSepCorpus::n_steps)
      .def_readonly("num_samples", &BMinSepCorpus::num_samples)
      .def_readonly("seed", &BMinSepCorpus::seed)
      .def_property_readonly("nbytes", &BMinSepCorpus::nbytes)
      .def("pld", [](const BMinSepCorpus& c, double nm, std::size_t n, const Config& cfg) {
             py::gil_scoped_release r;
             return c.pld(nm, n, cfg);
           }, py::arg("noise_multiplier"), py::arg("n_steps"), py::arg("config"));
  m.def("adaclip_effective_noise_multiplier", &adaclip_effective_noise_multiplier);

  m.def("minsep_true_max_participations", [](std::int64_t n, std::int64_t ms, py::object mp) {
    return minsep_true_max_participations(n, ms, opt_int(mp)); }, py::arg("n"), py::arg("min_sep"), py::arg("max_participations") = py::none());
  m.def("max_participation_for_linear_fn", [](std::vector<double> x, std::int64_t ms, py::object mp) {
    return max_participation_for_linear_fn(x, ms, opt_int(mp)); }, py::arg("x"), py::arg("min_sep"), py::arg("max_participations") = py::none());
  m.def("single_participation_sensitivity_squared", &sens_sq_single_participation);
  m.def("general_sensitivity_squared_upper_bound", [](std::vector<double> g, std::size_t n, std::int64_t ms, py::object mp) {
    return sens_sq_minsep_upper_bound(g, n, ms, opt_int(mp)); }, py::arg("gram"), py::arg("n"), py::arg("min_sep"), py::arg("max_participations") = py::none());
  m.def("banded_sensitivity_squared", [](std::vector<double> g, std::size_t n, std::int64_t bands, std::int64_t ms, py::object mp) {
    return sens_sq_banded(g, n, bands, ms, opt_int(mp)); }, py::arg("gram"), py::arg("n"), py::arg("bands"), py::arg("min_sep"), py::arg("max_participations") = py::none());
  m.def("fixed_epoch_sensitivity_squared", &sens_sq_fixed_epoch);
  m.def("toeplitz_minsep_sensitivity_squared", [](std::vector<double> c, std::int64_t n, std::int64_t ms, py::object mp) {
    return toeplitz_minsep_sens_sq(c, n, ms, opt_int(mp)); }, py::arg("coef"), py::arg("n"), py::arg("min_sep"), py::arg("max_participations") = py::none());
  m.def("blt_sensitivity_squared", [](std::vector<double> s, std::vector<double> d, std::int64_t n, std::int64_t ms, py::object mp) {
    return blt_sens_sq(s, d, n, ms, opt_int(mp)); }, py::arg("scale"), py::arg("decay"), py::arg("n"), py::arg("min_sep") = 1, py::arg("max_participations") = py::none());
  m.def("toeplitz_gram_matrix", &toeplitz_gram);
  // ---- Toeplitz-column strategies (lambda-CGD, banded inverse square root), optionally column-normalised
  auto mp = [](py::object o) -> std::int64_t { return o.is_none() ? -1 : o.cast<std::int64_t>(); };
  m.def("lambda_cgd_sensitivity_squared", [mp](double l, std::size_t n, std::int64_t ms, py::object k, double) {
    return lambda_cgd_sens_sq(l, n, ms, mp(k), false); },
    py::arg("lambda_"), py::arg("n_steps"), py::arg("min_sep") = 1, py::arg("max_participations") = py::none(), py::arg("momentum") = 0.0);
  m.def("lambda_cgd_normalized_sensitivity_squared", [mp](double l, std::size_t n, std::int64_t ms, py::object k, double) {
    return lambda_cgd_sens_sq(l, n, ms, mp(k), true); },
    py::arg("lambda_"), py::arg("n_steps"), py::arg("min_sep") = 1, py::arg("max_participations") = py::none(), py::arg("momentum") = 0.0);
  m.def("lambda_cgd_max_column_norm", &lambda_cgd_max_column_norm, py::arg("lambda_"), py::arg("n_steps"));
  m.def("lambda_cgd_gram_matrix", [mp](double l, std::size_t n, std::int64_t ms, py::object k, bool norm, double beta) {
    const std::int64_t kk = mp(k); py::gil_scoped_release r; return lambda_cgd_bnb_gram(l, n, ms, kk, norm, beta, nullptr); },
    py::arg("lambda_"), py::arg("n_steps"), py::arg("min_sep") = 1, py::arg("max_participations") = py::none(),
    py::arg("normalized") = true, py::arg("momentum") = 0.0);
  m.def("lambda_cgd_gram_matrix_lr", [mp](double l, double beta, std::size_t n, std::int64_t ms, py::object k, bool norm, std::vector<double> w) {
    const std::int64_t kk = mp(k); py::gil_scoped_release r; return lambda_cgd_bnb_gram(l, n, ms, kk, norm, beta, &w); },
    py::arg("lambda_"), py::arg("momentum"), py::arg("n_steps"), py::arg("min_sep"), py::arg("max_participations"),
    py::arg("normalized"), py::arg("lr_weights"));
  m.def("bisr_strategy_coefficients", &inverse_toeplitz_coefficients, py::arg("coefficients"), py::arg("n"));
  m.def("bisr_sensitivity_squared", [mp](std::vector<double> taps, std::size_t n, std::int64_t ms, py::object k, double) {
    return toeplitz_columns_sens_sq(inverse_toeplitz_coefficients(taps, n), n, ms, mp(k), false); },
    py::arg("coefficients"), py::arg("n_steps"), py::arg("min_sep") = 1, py::arg("max_participations") = py::none(), py::arg("momentum") = 0.0);
  m.def("bisr_normalized_sensitivity_squared", [mp](std::vector<double> taps, std::size_t n, std::int64_t ms, py::object k, double) {
    return toeplitz_columns_sens_sq(inverse_toeplitz_coefficients(taps, n), n, ms, mp(k), true); },
    py::arg("coefficients"), py::arg("n_steps"), py::arg("min_sep") = 1, py::arg("max_participations") = py::none(), py::arg("momentum") = 0.0);
  m.def("bisr_gram_matrix", [mp](std::vector<double> taps, std::size_t n, std::int64_t ms, py::object k, bool norm, double beta) {
    const std::int64_t kk = mp(k); py::gil_scoped_release r; return toeplitz_columns_bnb_gram(inverse_toeplitz_coefficients(taps, n), n, ms, kk, norm, beta, nullptr); },
    py::arg("coefficients"), py::arg("n_steps"), py::arg("min_sep") = 1, py::arg("max_participations") = py::none(),
    py::arg("normalized") = true, py::arg("momentum") = 0.0);
  m.def("bisr_gram_matrix_lr", [mp](std::vector<double> taps, double beta, std::size_t n, std::int64_t ms, py::object k, bool norm, std::vector<double> w) {
    const std::int64_t kk = mp(k); py::gil_scoped_release r; return toeplitz_columns_bnb_gram(inverse_toeplitz_coefficients(taps, n), n, ms, kk, norm, beta, &w); },
    py::arg("coefficients"), py::arg("momentum"), py::arg("n_steps"), py::arg("min_sep"), py::arg("max_participations"),
    py::arg("normalized"), py::arg("lr_weights"));
  m.def("toeplitz_bnb_gram_matrix", [mp](std::vector<double> coef, std::size_t n, std::int64_t ms, py::object k, bool norm) {
    const std::int64_t kk = mp(k); py::gil_scoped_release r; return toeplitz_columns_bnb_gram(coef, n, ms, kk, norm, 0.0, nullptr); },
    py::arg("strategy_coef"), py::arg("n_steps"), py::arg("min_sep") = 1, py::arg("max_participations") = py::none(),
    py::arg("normalized") = true);
  m.def("norm_ppf", &norm_ppf);
  m.def("norm_cdf", &norm_cdf);
}
