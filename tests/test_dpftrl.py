"""DP-FTRL strategies vs dense materialisation, noise engine, samplers, accounting, codec."""
import json
import math

import numpy as np
import pytest
import torch
from scipy.linalg import toeplitz

import opaque_b200.accounting as acc
from opaque_b200.dpftrl import (BallsInBinsSampler, BMinSepSampler, CyclicPoissonSampler, SequentialBatchSampler,
                                band_mf_strategy, bisr_strategy, blt_strategy, bsr_strategy, identity_strategy,
                                lambda_cgd_strategy, mf_gaussian_noise)
from opaque_b200.dpftrl import accounting as fa
from opaque_b200.dpftrl import noise as N
from opaque_b200.random import key
from opaque_b200.scheduling import cosine_schedule
from opaque_b200.serialization import from_state_dict, state_dict
from opaque_b200.types import clipped

STRATEGIES = [identity_strategy(), band_mf_strategy(bands=4), bsr_strategy(bandwidth=4, alpha=0.99, beta=0.9),
              bisr_strategy(bandwidth=4), lambda_cgd_strategy(lambda_=0.5, normalized=False), blt_strategy(max_buffers=3)]


@pytest.mark.parametrize("s", STRATEGIES, ids=lambda s: type(s).__name__)
def test_streaming_inverse_matches_dense(s):
    n = 48
    c = np.pad(s.coefficients(n), (0, n))[:n]
    C = np.tril(toeplitz(c))
    Cinv = s.streaming_matrix(n).materialize(n)
    assert np.abs(Cinv @ C - np.eye(n)).max() < 1e-6
    rn = s.streaming_matrix(n).row_norms_squared(n)
    assert np.allclose(rn, (Cinv ** 2).sum(1), rtol=1e-6)
    # sensitivity: brute force over single participation = max column norm
    assert math.isclose(s.sensitivity(n, n, 1), math.sqrt((C ** 2).sum(0).max()), rel_tol=1e-6)
    assert s.sensitivity(n, 8) <= s.sensitivity(n, 1) + 1e-9


def test_sqrt_coefficients_and_bsr_closed_form():
    r = N.sqrt_coefs(6)
    assert np.allclose(r, [1, 0.5, 0.375, 0.3125, 0.2734375, 0.24609375])
    assert np.allclose(np.convolve(r, r)[:6], 1.0)                       # (1-x)^{-1/2} squared = 1/(1-x)
    assert np.allclose(np.convolve(N.inv_sqrt_coefs(6), r)[:6], [1, 0, 0, 0, 0, 0], atol=1e-12)
    c = bsr_strategy(bandwidth=5, alpha=1.0, beta=0.0).coefficients(20)
    assert np.allclose(c, r[:5])


def test_optimised_strategies_beat_identity():
    n = 128
    def loss(s):
        inv = N.inverse_coef(s.coefficients(n), n)
        return N.toeplitz_sensitivity_squared(s.coefficients(n), n, 1, 1) * N.prefix_workload_error(inv)
    base = loss(identity_strategy())
    assert loss(band_mf_strategy(bands=8)) < 0.5 * base
    assert loss(blt_strategy(max_buffers=3)) < 0.5 * base


def test_strategy_methods_accept_the_keyword_form():
    """``n_steps=`` names the horizon; participation keywords a method does not read are accepted and ignored."""
    for s in (identity_strategy(), band_mf_strategy(bands=3), blt_strategy(max_buffers=2), bsr_strategy(bandwidth=3)):
        assert s.sensitivity(n_steps=12, min_sep=3, max_participations=2) == s.sensitivity(12, 3, 2)
        assert np.array_equal(s.coefficients(n_steps=12, min_sep=3, max_participations=None), s.coefficients(12))
        assert np.array_equal(s.gram_matrix(n_steps=6, min_sep=1, max_participations=None), s.gram_matrix(6))
        s.streaming_matrix(n_steps=6, min_sep=1, max_participations=None)
    with pytest.raises(TypeError):
        identity_strategy().coefficients(4, n_steps=4)


def test_band_mf_objective_momentum_and_learning_rate_weights():
    """Unit-norm coefficients that minimise the MEAN squared error of the momentum workload, weighted per step."""
    n = 48
    base = np.asarray(band_mf_strategy(bands=4).coefficients(n))
    assert math.isclose(float(np.linalg.norm(base)), 1.0, rel_tol=1e-12) and np.all(np.diff(base) < 0)
    def objective(c, **kw):
        return N.toeplitz_workload_error(c, n, **kw) * float(np.dot(c, c))
    assert objective(base) < objective(N.sqrt_coefs(4)) and objective(base) < 0.5 * objective(np.array([1.0]))
    for eps in (1e-3, -1e-3):                                  # a stationary point of the scale-invariant objective
        for k in range(4):
            bumped = base.copy(); bumped[k] += eps
            assert objective(bumped) >= objective(base) - 1e-12
    mom = np.asarray(band_mf_strategy(bands=4, momentum=0.5).coefficients(n))
    w = N.momentum_workload_coefs(0.5, n)
    assert objective(mom, workload_coef=w) < objective(base, workload_coef=w)
    weights = np.linspace(1.0, 0.05, n)
    lr = np.asarray(band_mf_strategy(bands=4, lr_schedule=lambda t: float(weights[t])).coefficients(n))
    assert objective(lr, query_weights=weights) < objective(base, query_weights=weights)
    assert math.isclose(N.toeplitz_workload_error(base, n, kind="max"), N.prefix_workload_error(N.inverse_coef(base, n)), rel_tol=1e-9)


def test_lambda_cgd_draws_use_the_unlabelled_step_key():
    """λ-CGD draws ``z_t`` from ``fold_in(key, t)``; the other strategies label the step key ``"mf_gaussian_column"``."""
    from opaque_b200.dpftrl import lambda_cgd_strategy
    from opaque_b200.random import fold_in
    k = key(9)
    def first(strategy):
        nf, st = mf_gaussian_noise({"w": torch.zeros(5)}, strategy, n_steps=4, noise_multiplier=1.0, key=k)
        return nf(clipped({"w": torch.zeros(5)}, 1.0), st)[0].pytree["w"]
    z_plain = N._iid_normal_like({"w": torch.zeros(5)}, 1.0, fold_in(k, 0), torch.float32)["w"]
    z_label = N._iid_normal_like({"w": torch.zeros(5)}, 1.0, fold_in(k, "mf_gaussian_column", 0), torch.float32)["w"]
    assert torch.allclose(first(lambda_cgd_strategy(lambda_=0.5, normalized=False)), z_plain)
    assert torch.allclose(first(identity_strategy()), z_label) and not torch.allclose(z_plain, z_label)


def test_mf_noise_statistics_horizon_and_constant_norm():
    s = blt_strategy(max_buffers=2)
    nf, st = mf_gaussian_noise({"w": torch.zeros(50_000)}, s, n_steps=3, noise_multiplier=2.0, key=key(1))
    rn = s.streaming_matrix(3).row_norms_squared(3)
    for t in range(3):
        out, st = nf(clipped({"w": torch.zeros(50_000)}, 0.5), st)
        assert math.isclose(out.noise_stddev, 1.0 * math.sqrt(rn[t]), rel_tol=1e-9)
        assert abs(float(out.pytree["w"].std()) - out.noise_stddev) < 0.02
    with pytest.raises(RuntimeError):
        nf(clipped({"w": torch.zeros(50_000)}, 0.5), st)
    nf, st = mf_gaussian_noise({"w": torch.zeros(4)}, s, n_steps=3, noise_multiplier=1.0, key=key(1))
    _, st = nf(clipped({"w": torch.zeros(4)}, 1.0), st)
    with pytest.raises(ValueError):
        nf(clipped({"w": torch.zeros(4)}, 2.0), st)


def test_mf_noise_equals_dense_cinv_times_z():
    s = band_mf_strategy(bands=3)
    n = 6
    nf, st = mf_gaussian_noise({"w": torch.zeros(5)}, s, n_steps=n, noise_multiplier=1.0, key=key(3))
    outs = []
    for t in range(n):
        out, st = nf(clipped({"w": torch.zeros(5)}, 1.0), st)
        outs.append(out.pytree["w"])
    X = torch.stack(outs).double().numpy()
    C = np.tril(toeplitz(np.pad(s.coefficients(n), (0, n))[:n]))
    Z = C @ X                                         # recover the iid draws; they must be the keyed normals
    nf2, st2 = mf_gaussian_noise({"w": torch.zeros(5)}, identity_strategy(), n_steps=n, noise_multiplier=1.0, key=key(3))
    for t in range(n):
        z, st2 = nf2(clipped({"w": torch.zeros(5)}, 1.0), st2)
        assert np.allclose(Z[t], z.pytree["w"].double().numpy(), atol=1e-5)


def test_strategy_codec_and_accounting_round_trip():
    s = band_mf_strategy(bands=4, lr_schedule=cosine_schedule(1.0, 0.1, 100))
    wire = N.strategy_to_wire(s)
    assert wire["type"] == "BandMfStrategy" and wire["lr_schedule"]["__opaque_recipe__"] == "CosineSchedule"
    assert N.strategy_from_wire(json.loads(json.dumps(wire))) == s
    p = fa.mf_gaussian(2.0, band_mf_strategy(bands=4), n_steps=64, min_sep=4)
    a = acc.Accountant()
    a |= fa.per_step(p) * 64
    b = acc.Accountant.from_state_dict(json.loads(a.to_json()))
    assert math.isclose(a.epsilon_at(1e-5), b.epsilon_at(1e-5))
    # one Gaussian with multiplier sigma / sensitivity
    eff = 2.0 / band_mf_strategy(bands=4).sensitivity(64, 4)
    from opaque_b200.dpsgd.accounting import gaussian
    assert math.isclose(p.epsilon_at(1e-5), gaussian(eff).epsilon_at(1e-5), rel_tol=1e-9)
    amp = fa.poisson(p, 0.1, n_steps=64)
    assert amp.epsilon_at(1e-5) < p.epsilon_at(1e-5)


def test_samplers_participation_patterns_and_resume():
    cyc = CyclicPoissonSampler(range(400), 1.0, bands=4, n_steps=8, key=key(1))
    batches = list(cyc)
    assert sorted(batches[0]) == list(range(100)) and sorted(batches[5]) == list(range(100, 200))
    bms = BMinSepSampler(range(50), 3, 1.0, 6, key=key(2))
    b = list(bms)
    assert len(b[0]) == 50 and len(b[1]) == 0 and len(b[2]) == 0 and len(b[3]) == 50
    bnb = BallsInBinsSampler(range(90), 3, n_steps=6, key=key(3))
    b = list(bnb)
    assert sorted(b[0] + b[1] + b[2]) == list(range(90)) and b[0] == b[3]
    seq = SequentialBatchSampler(range(10), 4, n_steps=5)
    assert list(seq) == [[0, 1, 2, 3], [4, 5, 6, 7], [0, 1, 2, 3], [4, 5, 6, 7], [0, 1, 2, 3]] and seq.min_sep == 2
    s = CyclicPoissonSampler(range(400), 0.3, bands=2, n_steps=10, key=key(7))
    it = iter(s)
    next(it), next(it), next(it)
    sd = state_dict(s)
    expect = next(it)
    s2 = from_state_dict(CyclicPoissonSampler(range(400), 0.3, bands=2, n_steps=10, key=key(7)), sd)
    assert next(iter(s2)) == expect


def test_b_min_sep_monte_carlo_accountant():
    """Amplified accounting for banded MF under b-min-sep subsampling: limits and monotonicity."""
    import math
    from opaque_b200.accounting.core import DiscretizationConfig, native
    cfg = DiscretizationConfig().to_native()
    # one band, no separation, always sampled: n-fold Gaussian composition = Gaussian with sensitivity sqrt(n)
    mc = native.b_min_sep_mc_pld([1.0], 16, 1, 1.0, 4.0, False, cfg).epsilon_at(1e-4)
    exact = native.gaussian_pld(4.0 / math.sqrt(16), cfg).epsilon_at(1e-4)
    assert abs(mc - exact) < 0.08 * exact
    s = band_mf_strategy(bands=4)
    eps = [fa.b_min_sep(fa.mf_gaussian(2.0, s, n_steps=64), bands=4, n_steps=64, sampling_prob=p).epsilon_at(1e-4) for p in (1.0, 0.3, 0.05)]
    assert eps[0] > eps[1] > eps[2] > 0
    bound = fa.b_min_sep(fa.mf_gaussian(2.0, s, n_steps=64), bands=4, n_steps=64).epsilon_at(1e-4)       # sensitivity-only bound
    assert eps[1] < bound and abs(eps[0] - bound) < 0.1 * bound
    with pytest.raises(ValueError):
        fa.b_min_sep(fa.mf_gaussian(2.0, band_mf_strategy(bands=8), n_steps=64), bands=4, n_steps=64, sampling_prob=0.1).epsilon_at(1e-4)
    proc = fa.b_min_sep(fa.mf_gaussian(2.0, s, n_steps=64), bands=4, n_steps=64, sampling_prob=0.3, warm_start=True)
    a = acc.Accountant()
    a |= proc
    restored = from_state_dict(acc.Accountant(), state_dict(a))
    assert math.isclose(restored.epsilon_at(1e-4), a.epsilon_at(1e-4), rel_tol=1e-12)


def test_paired_second_moment_mf_noise_shares_one_budget():
    """Σg and Σg² each get their own correlated-noise stream; the base deviations split one Mahalanobis budget."""
    import math
    from opaque_b200.dpftrl.noise import SecondMomentMFNoiseState, mf_gaussian_noise
    from opaque_b200.types import SecondMomentClippingOutput, SecondMomentNoiseOutput, clipped
    n, nm = 8, 2.0
    first, second = band_mf_strategy(bands=4), identity_strategy()
    tmpl = {"w": torch.zeros(20000)}
    noise_fn, st = mf_gaussian_noise(tmpl, first, n_steps=n, noise_multiplier=nm, key=key(3), second_moment_strategy=second)
    assert isinstance(st, SecondMomentMFNoiseState)
    c1 = first.sensitivity(n, min_sep=n, max_participations=1)
    c2 = second.sensitivity(n, min_sep=n, max_participations=1)
    C, C2 = 1.5, 0.4
    s1 = (nm / c1) * math.sqrt(C * c1 * (C * c1 + C2 * c2))
    s2 = (nm / c1) * math.sqrt(C2 * c2 * (C * c1 + C2 * c2))
    assert math.isclose((C * c1 / s1) ** 2 + (C2 * c2 / s2) ** 2, (c1 / nm) ** 2, rel_tol=1e-12)     # the joint budget
    out, st1 = noise_fn(SecondMomentClippingOutput(clipped(tmpl, C), clipped(tmpl, C2)), st)
    assert isinstance(out, SecondMomentNoiseOutput) and st1._step_counter == 1
    # step 0 of C^-1 has a unit row for both strategies here (c_0 = 1): realised = base deviation
    assert math.isclose(out.noisy_grads.noise_stddev, s1 * math.sqrt(first.streaming_matrix(n).row_norms_squared(n)[0]), rel_tol=1e-9)
    assert abs(float(out.noisy_grads.pytree["w"].std()) / out.noisy_grads.noise_stddev - 1) < 0.03
    assert abs(float(out.noisy_squared_grads.pytree["w"].std()) / s2 - 1) < 0.03
    corr = float(torch.corrcoef(torch.stack([out.noisy_grads.pytree["w"], out.noisy_squared_grads.pytree["w"]]))[0, 1])
    assert abs(corr) < 0.03                                                                # independent streams
    # resumable through the registry; wrong input kinds are refused both ways
    restored = from_state_dict(st, state_dict(st1))
    a, _ = noise_fn(SecondMomentClippingOutput(clipped(tmpl, C), clipped(tmpl, C2)), st1)
    b, _ = noise_fn(SecondMomentClippingOutput(clipped(tmpl, C), clipped(tmpl, C2)), restored)
    assert torch.equal(a.noisy_grads.pytree["w"], b.noisy_grads.pytree["w"])
    with pytest.raises(TypeError):
        noise_fn(clipped(tmpl, C), st1)
    single_fn, single_st = mf_gaussian_noise(tmpl, first, n_steps=n, noise_multiplier=nm, key=key(3))
    with pytest.raises(TypeError):
        single_fn(SecondMomentClippingOutput(clipped(tmpl, C), clipped(tmpl, C2)), single_st)
    with pytest.raises(ValueError):
        noise_fn(SecondMomentClippingOutput(clipped(tmpl, C * 2), clipped(tmpl, C2)), st1)      # the bound must stay constant


def test_streaming_matrix_algebra_matches_dense_products():
    """Products, diagonal scaling and the momentum-SGD workload against their dense definitions."""
    import numpy as np
    from opaque_b200.dpftrl import noise as N
    n = 7
    fir = N.fir_streaming(np.array([1.0, -0.4, 0.1]))
    inv = N.toeplitz_inverse_streaming(np.array([1.0, 0.5, 0.25]))
    A, B = fir.materialize(n), inv.materialize(n)
    assert np.allclose((fir @ inv).materialize(n), A @ B)
    r, c = np.linspace(1, 2, n), np.linspace(0.5, 1.5, n)
    assert np.allclose(N.scale_rows_and_columns(fir, r, c).materialize(n), np.diag(r) @ A @ np.diag(c))
    assert np.allclose((fir * 3.0).materialize(n), 3.0 * A)
    assert np.allclose(N.diagonal_streaming([2.0, 5.0]).materialize(4), np.diag([2.0, 5.0, 5.0, 5.0]))
    x = torch.randn(n, 3, dtype=torch.float64)
    assert torch.allclose((fir @ x).double(), torch.as_tensor(A) @ x, atol=1e-5)      # streaming states are fp32
    mu, lr = 0.9, np.array([0.1, 0.2, 0.3, 0.4, 0.5, 0.6, 0.7])
    W = np.zeros((n, n))
    for j in range(n):
        mom = acc = 0.0
        for t in range(n):
            mom = mu * mom + (1.0 if t == j else 0.0)
            acc = acc + lr[t] * mom
            W[t, j] = acc
    assert np.allclose(N.momentum_sgd_matrix(mu, lr).materialize(n), W)


def test_lambda_cgd_is_column_normalised_per_row():
    """Normalised λ-CGD: ``C⁻¹`` rows carry ``d_t`` (column norms of ``C``), every column of ``C·diag(d)⁻¹`` has unit norm,
    the streaming operator equals the dense inverse, and the sensitivity equals the brute-force value from the Gram."""
    import itertools
    import numpy as np
    from opaque_b200.dpftrl import noise as N
    n, lam = 9, 0.6
    st = N.lambda_cgd_strategy(lambda_=lam, normalized=True)
    C = np.array([[lam ** (i - j) if i >= j else 0.0 for j in range(n)] for i in range(n)])
    d = np.sqrt((C ** 2).sum(0))
    assert np.allclose(st.row_scales(n), d)
    Cn = C / d[None, :]
    assert np.allclose((Cn ** 2).sum(0), 1.0)
    assert np.allclose(st.streaming_matrix(n).materialize(n), np.linalg.inv(Cn))
    assert np.allclose(st.gram_matrix(n), Cn.T @ Cn)
    for min_sep, k in ((1, 1), (2, None), (3, 2), (1, 3)):
        best = 0.0
        kk = k if k is not None else n
        for r in range(1, kk + 1):
            for idx in itertools.combinations(range(n), r):
                if all(b - a >= min_sep for a, b in zip(idx, idx[1:])):
                    best = max(best, float(np.linalg.norm(Cn[:, list(idx)].sum(1))))
        assert math.isclose(st.sensitivity(n, min_sep, k), best, rel_tol=1e-9), (min_sep, k)
    assert math.isclose(st.row_norm(n, 0), d[0]) and math.isclose(st.row_norm(n, 4), d[4] * math.sqrt(1 + lam * lam))
    mech = st.fused_mechanism(n)
    assert mech["kind"] == "fir" and np.allclose(mech["coef_fn"](5), [d[5], -lam * d[5]])
