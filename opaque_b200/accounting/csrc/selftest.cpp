// Stand-alone exercise of the PLD core for sanitizer builds (AddressSanitizer / UndefinedBehaviorSanitizer):
// the same entry points the Python bindings call, with the pinned values checked in-process.  Built and run by the
// CPU test lane with  g++ -fsanitize=address,undefined ; exits non-zero on any mismatch.
#include <cmath>
#include <cstdio>
#include <vector>

#include "pld.hpp"

using namespace obacc;

static int failures = 0;
static void expect_close(const char* what, double got, double want, double tol) {
  const bool ok = std::isfinite(got) && std::fabs(got - want) <= tol * std::fmax(1.0, std::fabs(want));
  std::printf("%-44s got %.10g want %.10g %s\n", what, got, want, ok ? "ok" : "MISMATCH");
  if (!ok) ++failures;
}

int main() {
  Config cfg;
  const Pld g = gaussian_pld(1.1, cfg);
  expect_close("gaussian(1.1) eps at 1e-5", g.epsilon_at(1e-5), 3.9212, 1e-3);
  const Pld p = poisson_gaussian_pld(1.0, 256.0 / 60000.0, cfg).self_compose(200);
  expect_close("poisson(256/60000, sigma 1) x 200 eps at 1e-5", p.epsilon_at(1e-5), 0.37039, 2e-3);
  const Pld c = g.compose(poisson_gaussian_pld(2.0, 0.01, cfg));
  if (!(c.epsilon_at(1e-5) >= g.epsilon_at(1e-5))) { std::printf("composition decreased epsilon\n"); ++failures; }
  const Pld ra1 = random_allocation_gaussian_pld(1.0, 1, 1, cfg);
  expect_close("random allocation t=1 equals gaussian", ra1.epsilon_at(1e-8), gaussian_pld(1.0, cfg).epsilon_at(1e-8), 1e-3);
  const Pld ra = random_allocation_gaussian_pld(1.0, 50, 2, cfg);
  if (!(ra.epsilon_at(1e-6) > 0 && ra.epsilon_at(1e-6) < gaussian_pld(1.0, cfg).self_compose(2).epsilon_at(1e-6))) {
    std::printf("random allocation k=2, t=50 is not amplified\n");
    ++failures;
  }
  const Pld pp = parallel_poisson_gaussian_pld(1.0, 0.01, 4, cfg);
  if (!(pp.delta_at(1.0) >= 0 && pp.delta_at(1.0) <= 1)) { std::printf("delta out of range\n"); ++failures; }
  expect_close("beta(alpha) of eps_delta(1, 0) at 0.1", eps_delta_pld(1.0, 0.0, cfg).beta_at(0.1), 1.0 - std::exp(1.0) * 0.1, 2e-2);
  {   // discretised PLDs never fall below the analytic Gaussian curve (grid points included)
    for (double sigma : {0.7, 1.0, 2.0})
      for (double eps : {0.0, 0.5, 1.0, 2.0}) {
        const double exact = gaussian_delta(sigma, eps, 1.0), got = gaussian_pld(sigma, cfg).delta_at(eps);
        if (!(got >= exact * (1.0 - 1e-12) && got <= exact * (1.0 + 1e-6) + 1e-12)) {
          std::printf("gaussian(%g) delta(%g): got %.15g, analytic %.15g\n", sigma, eps, got, exact);
          ++failures;
        }
      }
  }
  {   // Monte-Carlo accountants: stored transcripts equal the streaming accountant, full horizon and a prefix
    Config mc = cfg;
    mc.num_mc_samples = 2000;
    mc.seed = 5;
    const std::vector<double> coef = {1.0, 0.6, 0.3};
    const BMinSepCorpus corpus(coef, 40, 4, 0.1, true, mc.num_mc_samples, mc.seed);
    expect_close("b-min-sep corpus bytes", static_cast<double>(corpus.nbytes()), 2000.0 * 40.0 * 17.0, 0.0);
    for (std::size_t n : {std::size_t(40), std::size_t(17), std::size_t(1)}) {
      const Pld a = b_min_sep_mc_pld(coef, n, 4, 0.1, 1.3, true, mc);
      const Pld b = corpus.pld(1.3, n, mc);
      expect_close("b-min-sep corpus == streaming (eps at 1e-4)", b.epsilon_at(1e-4), a.epsilon_at(1e-4), 0.0);
    }
    const std::vector<double> gram = toeplitz_gram({1.0, 0.5}, 12);
    const Pld bb = balls_in_bins_mc_pld(gram, 12, 4, 1.5, mc);
    if (!(bb.epsilon_at(1e-4) > 0)) { std::printf("balls-in-bins epsilon not positive\n"); ++failures; }
  }
  std::printf("%s\n", failures ? "FAILED" : "all checks passed");
  return failures ? 1 : 0;
}
