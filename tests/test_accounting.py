"""C++ PLD accountant against pinned reference values and closed forms; process algebra; calibration."""
import json
import math

import pytest

import opaque_b200.accounting as acc
from opaque_b200.accounting.core import (Composed, Identity, PerStep, Repeated, native, process_from_wire,
                                          process_to_wire)
from opaque_b200.dpsgd import accounting as d
from opaque_b200.serialization import from_state_dict, state_dict


def _phi(x):
    return 0.5 * math.erfc(-x / math.sqrt(2))


def test_gaussian_matches_closed_form():
    p = d.gaussian(1.1)
    assert abs(p.epsilon_at(1e-5) - 3.92) < 0.01
    for eps in (0.0, 0.5, 1.0, 2.0):
        exact = _phi(0.5 / 1.1 - eps * 1.1) - math.exp(eps) * _phi(-0.5 / 1.1 - eps * 1.1)
        assert abs(p.delta_at(eps) - exact) < 2e-6
    assert abs(d.gaussian(0.5).delta_at(0.0) - 0.6826894921) < 1e-6
    # trade-off curve of a mu-GDP mechanism: beta(alpha) = Phi(Phi^-1(1-alpha) - mu)
    assert abs(d.gaussian(1.0).beta_at(0.1) - _phi(1.2815515655 - 1.0)) < 2e-4
    assert abs(d.gaussian(1.0).advantage() - (2 * _phi(0.5) - 1)) < 1e-5
    assert abs(d.gaussian(1.0).risk_at(0.5) - (1 - (2 * _phi(0.5) - 1)) / 2) < 1e-4


def test_composition_of_gaussians_is_gaussian():
    # n Gaussians with multiplier s compose to one with s / sqrt(n)
    a = (d.gaussian(2.0) * 4).epsilon_at(1e-6)
    b = d.gaussian(1.0).epsilon_at(1e-6)
    assert abs(a - b) < 2e-3
    c = (d.gaussian(2.0) | d.gaussian(2.0) | d.gaussian(2.0) | d.gaussian(2.0)).epsilon_at(1e-6)
    assert abs(c - b) < 2e-3


@pytest.mark.parametrize("workers,expected", [(1, 0.23982423090879623), (2, 0.5325659019424767),
                                              (4, 1.124570816812394), (8, 2.255585330074185)])
def test_parallel_poisson_pinned_values(workers, expected):
    """The reference's pinned values: reproduced to 1e-6 with its mass normalisation, and bounded from above (by a few
    1e-6) by the default, which never rescales a discretised PMF downwards."""
    from opaque_b200.accounting.core import DiscretizationConfig, set_discretization
    process = d.parallel_poisson(d.gaussian(0.8), 0.001, workers) * 500
    with set_discretization(DiscretizationConfig(proportional_normalization=True)):
        assert abs(process.epsilon_at(1e-5) - expected) < 1e-6
    strict = (d.parallel_poisson(d.gaussian(0.8), 0.001, workers) * 500).epsilon_at(1e-5)
    assert expected - 1e-9 <= strict < expected + 2e-5


def test_calibration_pinned_value_and_safety():
    budget = acc.epsilon_budget(3.0, 1e-5)
    res = acc.calibrate(budget, lambda nm: d.poisson(d.gaussian(nm), 0.032) * 100, 0.3, 10.0)
    assert abs(res.param - 0.8865) < 0.01 * 0.8865
    assert res.achieved <= 3.0 and math.isclose(res.achieved, 3.0, rel_tol=1e-5)
    # calibrating the sample rate: metric grows with the parameter, safe side is still respected
    res = acc.calibrate(budget, lambda q: d.poisson(d.gaussian(1.0), q) * 100, 1e-3, 0.5, tolerance=1e-3)
    assert res.achieved <= 3.0
    with pytest.raises(ValueError):
        acc.calibrate(budget, lambda nm: d.poisson(d.gaussian(nm), 0.032) * 100, 5.0, 10.0)
    with pytest.raises(ValueError):
        acc.calibrate(budget, lambda nm: d.gaussian(1.0), 0.5, 2.0)


def test_poisson_amplification_monotone_and_truncated():
    e_small = (d.poisson(d.gaussian(1.0), 0.01) * 100).epsilon_at(1e-5)
    e_big = (d.poisson(d.gaussian(1.0), 0.1) * 100).epsilon_at(1e-5)
    e_full = (d.gaussian(1.0) * 100).epsilon_at(1e-5)
    assert e_small < e_big < e_full
    assert abs((d.poisson(d.gaussian(1.0), 1.0) * 3).epsilon_at(1e-5) - (d.gaussian(1.0) * 3).epsilon_at(1e-5)) < 1e-6
    trunc = d.poisson(d.gaussian(1.0), 0.01, truncated_batch_size=15, dataset_size=1000)
    plain = d.poisson(d.gaussian(1.0), 0.01)
    assert (trunc * 50).epsilon_at(1e-5) >= (plain * 50).epsilon_at(1e-5) - 1e-9


def test_adaclip_effective_multiplier():
    a = d.adaclip(d.gaussian(1.0), fraction_noise_std=0.05, expected_batch_size=100.0)
    assert math.isclose(a.effective_noise_multiplier, 1 / math.sqrt(1 + 1 / (4 * 25)))
    assert a.epsilon_at(1e-5) > d.gaussian(1.0).epsilon_at(1e-5)


def test_algebra_flattening_and_identity_elision():
    g = d.gaussian(1.0)
    assert (g * 3) * 2 == Repeated(g, 6)
    assert (g | g) == Repeated(g, 2)
    assert (acc.identity() | g) is g and (g | acc.identity()) is g
    assert isinstance(g * 0, Identity)
    mixed = (g | d.gaussian(2.0)) | d.gaussian(2.0)
    assert isinstance(mixed, Composed) and mixed.right == Repeated(d.gaussian(2.0), 2)
    chain = acc.identity()
    for i in range(3000):                      # thousand-deep spines must not recurse
        chain = chain | d.gaussian(1.0 + (i % 2))
    wire = process_to_wire(chain)
    assert process_from_wire(wire) == chain and hash(chain) == hash(process_from_wire(wire))


def test_accountant_budget_and_json_round_trip():
    a = acc.Accountant(acc.epsilon_budget(0.5, 1e-5))
    step = d.poisson(d.gaussian(1.0), 0.01)
    for _ in range(10):
        a |= step
    assert a.process == Repeated(step, 10) and not a.budget_exceeded()
    a |= step * 5000
    assert a.budget_exceeded()
    b = acc.Accountant.from_state_dict(json.loads(a.to_json()))
    assert b.process == a.process and b.budget == a.budget
    assert from_state_dict(acc.Accountant(), state_dict(a)).process == a.process
    pre = acc.Accountant(prefix=step * 10)
    assert pre.epsilon_at(1e-5) == (step * 10).epsilon_at(1e-5)


def test_eps_delta_identity_nonprivate():
    assert abs(acc.eps_delta(1.0, 1e-6).epsilon_at(1e-6) - 1.0) < 2e-4
    assert (acc.eps_delta(1.0, 1e-6) * 3).epsilon_at(1e-5) <= 3.0 + 1e-3
    assert acc.identity().epsilon_at(1e-9) == 0.0
    assert acc.nonprivate().epsilon_at(0.5) == math.inf
    assert (d.gaussian(1.0) | acc.nonprivate()).epsilon_at(1e-5) == math.inf


def test_discretization_context_and_coarse_grid_is_pessimistic():
    fine = (d.poisson(d.gaussian(1.0), 0.01) * 200).epsilon_at(1e-5)
    with acc.set_discretization(discretization=1e-3):
        assert acc.get_discretization().discretization == 1e-3
        coarse = (d.poisson(d.gaussian(1.0), 0.01) * 200).epsilon_at(1e-5)
    assert acc.get_discretization().discretization == 1e-4
    assert coarse >= fine - 1e-9 and coarse - fine < 0.05


def test_native_sensitivities():
    assert native.minsep_true_max_participations(10, 3, None) == 4
    assert native.minsep_true_max_participations(10, 1, 3) == 3
    assert native.max_participation_for_linear_fn([1, 2, 3, 4, 5], 2, None) == 9.0
    assert native.max_participation_for_linear_fn([10, 1, 1, 1, 1], 1, 1) == 10.0
    assert native.max_participation_for_linear_fn([1.0] * 9, 3, None) == 3.0
    # identity strategy: k participations -> sensitivity^2 = k
    assert native.toeplitz_minsep_sensitivity_squared([1.0], 12, 3, None) == 4.0
    assert abs(native.norm_ppf(0.975) - 1.959963984540054) < 1e-12


def test_native_lambda_cgd_and_bisr_matrix_functions_match_dense_algebra():
    """Column-normalised Toeplitz strategies in the native core against dense numpy constructions."""
    import itertools

    import numpy as np
    from opaque_b200.accounting.core import native
    n, lam, b, k = 12, 0.65, 3, 3
    C = np.array([[lam ** (i - j) if i >= j else 0.0 for j in range(n)] for i in range(n)])
    d = np.sqrt((C ** 2).sum(0))
    Cn = C / d

    def brute(M, min_sep, kmax):
        best = 0.0
        for r in range(1, kmax + 1):
            for idx in itertools.combinations(range(n), r):
                if all(y - x >= min_sep for x, y in zip(idx, idx[1:])):
                    best = max(best, float((M[:, list(idx)].sum(1) ** 2).sum()))
        return best
    assert math.isclose(native.lambda_cgd_sensitivity_squared(lam, n, b, k), brute(C, b, k), rel_tol=1e-9)
    assert math.isclose(native.lambda_cgd_normalized_sensitivity_squared(lam, n, b, k), brute(Cn, b, k), rel_tol=1e-9)
    assert math.isclose(native.lambda_cgd_normalized_sensitivity_squared(lam, n, 1, 1), 1.0, rel_tol=1e-12)
    assert math.isclose(native.lambda_cgd_max_column_norm(lam, n), d[0], rel_tol=1e-12)
    # balls-in-bins Gram: m_i = sum over epochs of column (b e + i), momentum filter and per-row weights on top
    E = n // b
    for beta, w in ((0.0, None), (0.8, None), (0.5, np.linspace(1.0, 0.2, n))):
        F = np.array([[beta ** (i - j) if i >= j else 0.0 for j in range(n)] for i in range(n)])
        M = F @ Cn
        if w is not None:
            M = np.diag(w) @ M
        m = np.stack([sum(M[:, b * e + i] for e in range(E)) for i in range(b)])
        want = m @ m.T
        got = (native.lambda_cgd_gram_matrix(lam, n, b, None, True, beta) if w is None else
               native.lambda_cgd_gram_matrix_lr(lam, beta, n, b, None, True, w.tolist()))
        assert np.allclose(np.array(got).reshape(b, b), want, rtol=1e-10)
    # banded inverse square root: C is the dense inverse of the banded C^-1
    taps = [1.0, -0.5, -0.125, -0.0625]
    Cinv = np.array([[taps[i - j] if 0 <= i - j < len(taps) else 0.0 for j in range(n)] for i in range(n)])
    Cb = np.linalg.inv(Cinv)
    assert np.allclose(native.bisr_strategy_coefficients(taps, n), Cb[:, 0])
    assert math.isclose(native.bisr_sensitivity_squared(taps, n, b, k), brute(Cb, b, k), rel_tol=1e-9)
    Cbn = Cb / np.sqrt((Cb ** 2).sum(0))
    assert math.isclose(native.bisr_normalized_sensitivity_squared(taps, n, b, k), brute(Cbn, b, k), rel_tol=1e-9)
    mb = np.stack([sum(Cbn[:, b * e + i] for e in range(E)) for i in range(b)])
    assert np.allclose(np.array(native.bisr_gram_matrix(taps, n, b, None, True, 0.0)).reshape(b, b), mb @ mb.T, rtol=1e-10)
    # the strategy object's own (Python) sensitivity agrees with the native one
    from opaque_b200.dpftrl import noise as N
    st = N.lambda_cgd_strategy(lambda_=lam, normalized=True)
    assert math.isclose(st.sensitivity(n, b, k) ** 2, native.lambda_cgd_normalized_sensitivity_squared(lam, n, b, k), rel_tol=1e-9)
