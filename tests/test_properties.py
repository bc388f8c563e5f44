"""Property-based checks (hypothesis) of the substrate: pytrees, keys, serialization, the clipping bound, samplers."""
import math

import numpy as np
import pytest
import torch

hypothesis = pytest.importorskip("hypothesis")
from hypothesis import given, settings, strategies as st  # noqa: E402

from opaque_b200 import pytree as pt  # noqa: E402
from opaque_b200.dpsgd import PoissonSampler  # noqa: E402
from opaque_b200.engine.clipping import clip_pytree  # noqa: E402
from opaque_b200.random import fold_in, key, split  # noqa: E402
from opaque_b200.serialization import from_state_dict, state_dict  # noqa: E402

# derandomize: the same examples on every run, so a green suite stays green
FAST = settings(max_examples=40, deadline=None, derandomize=True)

shapes = st.lists(st.integers(1, 5), min_size=0, max_size=3).map(tuple)
leaves = shapes.map(lambda s: torch.arange(int(np.prod(s)) if s else 1, dtype=torch.float32).reshape(s if s else ()) - 1.5)
trees = st.recursive(leaves, lambda children: st.one_of(
    st.lists(children, min_size=1, max_size=3), st.lists(children, min_size=1, max_size=3).map(tuple),
    st.dictionaries(st.text("abcdef", min_size=1, max_size=3), children, min_size=1, max_size=3)), max_leaves=8)


@FAST
@given(trees)
def test_flatten_unflatten_round_trips_and_map_preserves_structure(tree):
    flat, td = pt.tree_flatten(tree)
    again = pt.tree_unflatten(td, flat)
    assert pt.tree_structure(again) == td
    assert all(torch.equal(a, b) for a, b in zip(pt.tree_leaves(again), flat))
    doubled = pt.tree_map(lambda x: 2 * x, tree)
    assert pt.tree_structure(doubled) == td
    total = math.sqrt(sum(float((x.double() ** 2).sum()) for x in flat))
    assert math.isclose(float(pt.global_norm(tree)), total, rel_tol=1e-6, abs_tol=1e-12)


@FAST
@given(trees)
def test_state_dict_round_trips_any_tensor_tree(tree):
    template = pt.tree_map(torch.zeros_like, tree)
    restored = from_state_dict(template, state_dict(tree))
    assert pt.tree_structure(restored) == pt.tree_structure(tree)
    assert all(torch.equal(a, b) for a, b in zip(pt.tree_leaves(restored), pt.tree_leaves(tree)))


@FAST
@given(st.integers(0, 2 ** 63 - 1), st.lists(st.one_of(st.integers(-2 ** 40, 2 ** 40), st.text(max_size=8)), min_size=1, max_size=4))
def test_fold_in_is_deterministic_and_left_folding(seed, data):
    k = key(seed)
    assert fold_in(k, *data) == fold_in(k, *data)
    step = k
    for item in data:
        step = fold_in(step, item)
    assert step == fold_in(k, *data)
    kids = split(k, 3)
    assert len({c.seed for c in kids}) == 3 and all(c == fold_in(k, i) for i, c in enumerate(kids))


@FAST
@given(trees, st.floats(1e-3, 1e3), st.sampled_from([torch.float32, torch.bfloat16, torch.float16]), st.floats(1e-3, 1e4))
def test_clipped_record_respects_the_bound_as_stored(tree, C, dtype, magnitude):
    record = pt.tree_map(lambda x: (x * magnitude).to(dtype), tree)
    clipped, aux = clip_pytree(record, C)
    stored = math.sqrt(sum(float((x.double() ** 2).sum()) for x in pt.tree_leaves(clipped)))
    assert stored <= C * (1 + 1e-12)                         # the bound holds on the values in their storage dtype
    before = math.sqrt(sum(float((x.double() ** 2).sum()) for x in pt.tree_leaves(record)))
    if math.isfinite(before) and before <= 0.5 * C:          # records well inside the bound pass (almost) unchanged
        assert stored >= 0.98 * before


@FAST
@given(st.integers(50, 400), st.floats(0.05, 0.9), st.integers(0, 10 ** 6), st.integers(1, 5))
def test_poisson_sampler_resumes_exactly_and_stays_in_range(n, rate, seed, consumed):
    a = PoissonSampler(range(n), rate, n_steps=consumed + 3, key=key(seed))
    it = iter(a)
    head = [next(it) for _ in range(consumed)]
    saved = state_dict(a)
    tail = list(it)
    b = from_state_dict(PoissonSampler(range(n), rate, n_steps=consumed + 3, key=key(seed)), saved)
    assert list(b) == tail and len(tail) == 3
    for batch in head + tail:
        assert batch == sorted(set(batch)) and (not batch or (0 <= batch[0] and batch[-1] < n))


SLOW = settings(max_examples=12, deadline=None, derandomize=True)


@SLOW
@given(st.floats(0.6, 3.0), st.floats(0.001, 0.2), st.integers(1, 300), st.floats(1e-8, 1e-3))
def test_accountant_is_monotone_and_self_consistent(sigma, q, steps, delta):
    from opaque_b200.dpsgd import accounting as dp
    run = dp.poisson(dp.gaussian(sigma), q) * steps
    eps = run.epsilon_at(delta)
    assert eps >= 0 and math.isfinite(eps)
    assert run.delta_at(eps) <= delta * (1 + 1e-6) + 1e-15          # (eps, delta) is a valid pair of the same curve
    assert (dp.poisson(dp.gaussian(sigma * 1.25), q) * steps).epsilon_at(delta) <= eps + 1e-9      # more noise, less loss
    assert (dp.poisson(dp.gaussian(sigma), q) * (steps + 50)).epsilon_at(delta) >= eps - 1e-9       # more steps, more loss
    assert run.epsilon_at(delta * 10) <= eps + 1e-9                                                 # larger delta, smaller eps
    unamplified = (dp.gaussian(sigma) * steps).epsilon_at(delta)
    assert eps <= unamplified + 1e-6                                                                # subsampling never hurts
    assert 0.0 <= run.delta_at(0.0) <= 1.0


@SLOW
@given(st.floats(0.5, 4.0), st.floats(0.01, 8.0))
def test_gaussian_pld_matches_the_analytic_curve(sigma, eps):
    from scipy.stats import norm
    from opaque_b200.dpsgd import accounting as dp
    exact = norm.cdf(0.5 / sigma - eps * sigma) - math.exp(eps) * norm.cdf(-0.5 / sigma - eps * sigma)
    got = dp.gaussian(sigma).delta_at(eps)
    assert got >= exact - 1e-9                      # pessimistic
    assert got <= exact + 2e-3 * max(exact, 1e-6) + 1e-7


@FAST
@given(st.floats(1e-2, 1e2), st.floats(1e-2, 1e2), st.floats(1e-3, 1e3), st.sampled_from([torch.float32, torch.bfloat16]))
def test_per_group_clipping_bounds_every_group_and_the_whole(c_a, c_b, magnitude, dtype):
    from opaque_b200.engine.clipping import auto_scale_pytree, per_group
    torch.manual_seed(0)
    record = {"a": {"w": (torch.randn(7, 5) * magnitude).to(dtype)}, "b": {"w": (torch.randn(11) * magnitude).to(dtype),
                                                                          "v": (torch.randn(3, 2) * magnitude).to(dtype)}}
    bound = per_group(record, {"a": c_a, "b": c_b})
    clipped, _ = clip_pytree(record, bound)
    na = float(clipped["a"]["w"].double().norm())
    nb = math.sqrt(float(clipped["b"]["w"].double().norm()) ** 2 + float(clipped["b"]["v"].double().norm()) ** 2)
    assert na <= c_a * (1 + 1e-12) and nb <= c_b * (1 + 1e-12)
    assert math.hypot(na, nb) <= bound.effective * (1 + 1e-12)
    # AUTO-S never lets a record exceed R (its factor is R / (norm + gamma) < R / norm)
    scaled, _ = auto_scale_pytree(record, 1.0, 0.01)
    total = math.sqrt(sum(float(x.double().norm()) ** 2 for x in pt.tree_leaves(scaled)))
    assert total <= 1.0 * (1 + 1e-12)


def _brute_force_sensitivity(C: np.ndarray, min_sep: int, max_participations: int) -> float:
    """max over participation sets (indices at least ``min_sep`` apart, at most ``max_participations`` of them) of the
    norm of the summed columns; valid as the sensitivity because every entry of ``C`` here is non-negative."""
    import itertools
    n = C.shape[1]
    best = 0.0
    for k in range(1, max_participations + 1):
        for idx in itertools.combinations(range(n), k):
            if all(b - a >= min_sep for a, b in zip(idx, idx[1:])):
                best = max(best, float(np.linalg.norm(C[:, list(idx)].sum(1))))
    return best


@settings(max_examples=25, deadline=None, derandomize=True)
@given(st.integers(4, 9), st.integers(1, 4), st.integers(1, 3), st.sampled_from(["identity", "band", "blt", "bsr"]))
def test_strategy_sensitivity_dominates_brute_force(n, min_sep, max_participations, kind):
    from scipy.linalg import toeplitz
    from opaque_b200.dpftrl import band_mf_strategy, blt_strategy, bsr_strategy, identity_strategy
    s = {"identity": identity_strategy(), "band": band_mf_strategy(bands=3), "blt": blt_strategy(max_buffers=2),
         "bsr": bsr_strategy(bandwidth=3, alpha=1.0, beta=0.0)}[kind]
    c = np.pad(np.asarray(s.coefficients(n), float), (0, n))[:n]
    assert (c >= -1e-12).all()
    C = np.tril(toeplitz(c))
    brute = _brute_force_sensitivity(C, min_sep, max_participations)
    got = s.sensitivity(n, min_sep, max_participations)
    assert got >= brute * (1 - 1e-9)                    # never below the true sensitivity
    assert got <= brute * 1.5 + 1e-9                    # and not vacuous on these small cases


@settings(max_examples=15, deadline=None, derandomize=True)
@given(st.floats(0.5, 3.0), st.floats(0.01, 0.5), st.floats(0.0, 3.0))
def test_poisson_subsampled_gaussian_pld_dominates_the_hockey_stick_integral(sigma, q, eps):
    """One step, both adjacency directions, against a dense numerical integral of max(0, P - e^eps Q)."""
    from scipy.stats import norm
    from opaque_b200.dpsgd import accounting as dp
    x = np.linspace(-12 * sigma - 1, 12 * sigma + 2, 400_001)
    base, shifted = norm.pdf(x, 0.0, sigma), norm.pdf(x, 1.0, sigma)
    mix = (1 - q) * base + q * shifted
    dx = x[1] - x[0]
    remove = float(np.maximum(mix - math.exp(eps) * base, 0.0).sum() * dx)       # P = with the record, Q = without
    add = float(np.maximum(base - math.exp(eps) * mix, 0.0).sum() * dx)
    exact = max(remove, add)
    got = dp.poisson(dp.gaussian(sigma), q).delta_at(eps)
    assert got >= exact - 1e-7 - 1e-4 * exact           # the integral itself carries ~1e-7 of quadrature error
    assert got <= exact * (1 + 5e-3) + 1e-6


@settings(max_examples=8, deadline=None, derandomize=True)
@given(st.floats(0.7, 2.5), st.floats(0.0, 2.5), st.sampled_from([2, 3]))
def test_random_allocation_pld_dominates_the_exact_divergence(sigma, eps, t):
    """One record lands in exactly one of ``t`` steps: P = (1/t) sum_j N(e_j, sigma^2 I), Q = N(0, sigma^2 I).  The exact
    hockey-stick divergences (both directions) are integrated on a dense grid in t dimensions."""
    from opaque_b200.dpsgd import accounting as dp
    m = 601 if t == 2 else 141
    g = np.linspace(-7 * sigma, 7 * sigma + 1, m)
    dx = g[1] - g[0]
    axes = np.meshgrid(*([g] * t), indexing="ij")
    log_q = sum(-0.5 * (a / sigma) ** 2 for a in axes) - t * math.log(sigma * math.sqrt(2 * math.pi))
    # P / Q = (1/t) sum_j exp((2 y_j - 1) / (2 sigma^2))
    ratio = sum(np.exp((2 * a - 1) / (2 * sigma ** 2)) for a in axes) / t
    q = np.exp(log_q)
    vol = dx ** t
    remove = float(np.maximum(q * ratio - math.exp(eps) * q, 0.0).sum() * vol)
    add = float(np.maximum(q - math.exp(eps) * q * ratio, 0.0).sum() * vol)
    exact = max(remove, add)
    got = dp.random_allocation(dp.gaussian(sigma), t).delta_at(eps)
    slack = 2e-3 if t == 2 else 2e-2                  # quadrature error of the coarse 3-D grid
    assert got >= exact * (1 - slack) - 1e-6
    assert got <= max(dp.gaussian(sigma).delta_at(eps), exact) * (1 + 1e-9) + 1e-9       # never worse than no amplification


@pytest.mark.parametrize("n,p,sigma", [(8, 0.3, 1.5), (16, 0.1, 1.0), (4, 0.6, 2.0)])
def test_b_min_sep_monte_carlo_reduces_to_poisson_composition_without_separation(n, p, sigma):
    """One band and no separation: every step takes the record independently with probability p, which is n-fold
    Poisson-subsampled Gaussian composition — known exactly from the PLD accountant."""
    from opaque_b200.accounting.core import DiscretizationConfig, native
    from opaque_b200.dpsgd import accounting as dp
    mc = native.b_min_sep_mc_pld([1.0], n, 1, p, sigma, False, DiscretizationConfig(num_mc_samples=200_000).to_native())
    exact = dp.poisson(dp.gaussian(sigma), p) * n
    for eps in (0.5, 1.0):
        assert abs(mc.delta_at(eps) - exact.delta_at(eps)) < 0.05 * exact.delta_at(eps)


@pytest.mark.parametrize("t,sigma", [(4, 1.0), (3, 0.8)])
def test_balls_in_bins_monte_carlo_matches_random_allocation_for_the_identity_strategy(t, sigma):
    """``C = I`` and one epoch of ``t`` bins is random allocation of one participation, which the PLD accountant covers."""
    from opaque_b200.accounting.core import DiscretizationConfig, native
    from opaque_b200.dpsgd import accounting as dp
    mc = native.balls_in_bins_mc_pld(np.eye(t).reshape(-1).tolist(), t, t, sigma,
                                     DiscretizationConfig(num_mc_samples=200_000).to_native())
    exact = dp.random_allocation(dp.gaussian(sigma), t)
    for eps in (0.5, 1.0):
        assert abs(mc.delta_at(eps) - exact.delta_at(eps)) < 0.05 * exact.delta_at(eps)


def test_accountant_front_ends_agree_where_their_definitions_coincide():
    from opaque_b200.dpftrl import accounting as fa, identity_strategy
    from opaque_b200.dpsgd import accounting as dp
    g, q, n, delta = dp.gaussian(1.2), 0.05, 100, 1e-6
    plain = (dp.poisson(g, q) * n).epsilon_at(delta)
    assert math.isclose((dp.parallel_poisson(g, q, 1) * n).epsilon_at(delta), plain, rel_tol=1e-9)        # one worker
    cyclic = fa.poisson(fa.mf_gaussian(1.2, identity_strategy(), n_steps=n), q, n_steps=n).epsilon_at(delta)
    assert math.isclose(cyclic, plain, rel_tol=1e-9)                                                     # C = I, one band
    capped = (dp.poisson(g, q, truncated_batch_size=80, dataset_size=1000) * n).epsilon_at(delta)
    assert capped >= plain                                                                               # the cap costs privacy
    assert math.isclose((dp.k_out_of_t(g, 1, 20) * 5).epsilon_at(delta), (dp.random_allocation(g, 20) * 5).epsilon_at(delta), rel_tol=1e-12)
    every_step, composed = dp.k_out_of_t(g, 20, 20).epsilon_at(delta), (g * 20).epsilon_at(delta)
    assert composed <= every_step <= composed * 1.002                                                    # k = t: plain composition
