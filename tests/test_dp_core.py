"""Clipping engine, Gaussian noise, samplers, adaptive clipping, optimizers (CPU)."""
import math

import numpy as np
import pytest
import torch

from opaque_b200 import optimizers as O
from opaque_b200.dpsgd import (KOutOfTSampler, PoissonSampler, RandomAllocationSampler, adaptive_clipped_grad,
                               auto_clipped_grad, clipped_grad, gaussian_noise, per_group)
from opaque_b200.engine.clipping import clip_pytree, clipped_fun
from opaque_b200.pytree import global_norm
from opaque_b200.random import key
from opaque_b200.serialization import from_state_dict, state_dict
from opaque_b200.types import ClippedPytree, NoisedPytree, SecondMomentClippingOutput, clipped


def _loss(p, x, y):
    return ((p["w"] @ x + p["b"] - y) ** 2).sum()


def _setup(n=8, seed=0):
    torch.manual_seed(seed)
    return {"w": torch.randn(3, 4), "b": torch.randn(3)}, torch.randn(n, 4), torch.randn(n, 3)


def _oracle(W, X, Y, C):
    tot = {k: torch.zeros_like(v) for k, v in W.items()}
    norms = []
    for i in range(X.shape[0]):
        g = torch.func.grad(_loss)(W, X[i], Y[i])
        n = float(global_norm(g))
        norms.append(n)
        c = min(1.0, C / n)
        for k in tot:
            tot[k] += c * g[k]
    return tot, norms


@pytest.mark.parametrize("mb", [None, 1, 3])
def test_clipped_grad_matches_loop_and_is_microbatch_invariant(mb):
    W, X, Y = _setup()
    fn, st = clipped_grad(_loss, clipping_norm=1.0, batch_argnums=(1, 2), return_aux=True, microbatch_size=mb)
    (g, aux), st = fn(W, X, Y, state=st)
    tot, norms = _oracle(W, X, Y, 1.0)
    for k in tot:
        assert torch.allclose(g.pytree[k], tot[k], atol=1e-5)
    assert torch.allclose(aux.grad_norms, torch.tensor(norms), rtol=1e-5)
    assert (aux.clipped_grad_norms <= 1.0).all() and g.max_norm == 1.0 and aux.batch_size == 8


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_clip_bound_holds_on_stored_values(dtype):
    torch.manual_seed(1)
    for _ in range(20):
        tree = {"a": (torch.randn(257) * 3).to(dtype), "b": (torch.randn(5, 7) * 0.1).to(dtype)}
        out, aux = clip_pytree(tree, 0.37)
        stored = math.sqrt(sum(float((v.double() ** 2).sum()) for v in out.values()))
        assert stored <= 0.37


def test_clip_edge_cases():
    t = {"a": torch.tensor([3.0, 4.0])}
    assert torch.equal(clip_pytree(t, float("inf"))[0]["a"], t["a"])
    assert float(clip_pytree(t, 0.0)[0]["a"].abs().sum()) == 0.0
    assert torch.equal(clip_pytree(t, 10.0)[0]["a"], t["a"])
    bad = {"a": torch.tensor([float("nan"), 1.0, float("inf")])}
    out, aux = clip_pytree(bad, 5.0)
    assert torch.equal(out["a"], torch.tensor([0.0, 1.0, 0.0]))
    assert float(clip_pytree(t, 5.0, return_zero=True)[0]["a"].abs().sum()) == 0.0


def test_empty_batch_normalize_and_stats():
    W, X, Y = _setup()
    fn, st = clipped_grad(_loss, clipping_norm=2.0, normalize_by=4.0, batch_argnums=(1, 2), return_stats=True)
    (g, stats), _ = fn(W, X[:0], Y[:0])
    assert g.max_norm == 0.5 and float(g.pytree["w"].abs().sum()) == 0 and stats.batch_size == 0
    (g, stats), _ = fn(W, X, Y)
    tot, norms = _oracle(W, X, Y, 2.0)
    assert torch.allclose(g.pytree["w"], tot["w"] / 4, atol=1e-5)
    assert stats.num_clipped == sum(n > 2.0 for n in norms) and stats.all_finite
    with pytest.raises(ValueError):
        clipped_grad(_loss, argnums=1, clipping_norm=1.0, batch_argnums=(1, 2))
    with pytest.raises(ValueError):
        clipped_grad(_loss, clipping_norm=1.0, return_aux=True, return_stats=True)


def test_per_group_auto_and_second_moment():
    W, X, Y = _setup()
    pg = per_group(W, {"w": 1.0}, fallback=0.5)
    fn, st = clipped_grad(_loss, clipping_norm=pg, batch_argnums=(1, 2))
    g, _ = fn(W, X, Y)
    for i in range(1):
        gi = torch.func.grad(_loss)(W, X[0], Y[0])
    assert math.isclose(g.max_norm.effective, math.sqrt(1.25))
    with pytest.raises(ValueError):
        per_group(W, {"zzz": 1.0})
    fa, sa = auto_clipped_grad(_loss, R=1.0, gamma=0.01, batch_argnums=(1, 2), return_aux=True)
    (g, aux), _ = fa(W, X, Y)
    expected = sum(torch.func.grad(_loss)(W, X[i], Y[i])["w"] / (aux.grad_norms[i] + 0.01) for i in range(8))
    assert torch.allclose(g.pytree["w"], expected, atol=1e-5)
    f2, _ = clipped_grad(_loss, clipping_norm=1.0, batch_argnums=(1, 2), second_moment=True)
    out, _ = f2(W, X, Y)
    assert isinstance(out, SecondMomentClippingOutput) and out.squared_grads.max_norm == 1.0
    assert (out.squared_grads.pytree["w"] >= 0).all()


def test_clipped_fun_generic_output_and_has_aux():
    fn, st = clipped_fun(lambda x: ({"v": x * 2}, x.sum()), has_aux=True, clipping_norm=1.0, return_aux=True)
    (out, aux), _ = fn(torch.tensor([[3.0, 4.0], [0.3, 0.4]]))
    assert torch.allclose(out.pytree["v"], torch.tensor([0.6 + 0.6, 0.8 + 0.8]), atol=1e-5)
    assert torch.allclose(aux.aux, torch.tensor([7.0, 0.7]))


def test_gaussian_noise_statistics_determinism_and_state():
    nf, st = gaussian_noise(noise_multiplier=1.5, key=key(3))
    g = clipped({"a": torch.zeros(200_000), "b": torch.zeros(10)}, 2.0)
    n1, s1 = nf(g, st)
    n2, _ = nf(g, st)
    n3, _ = nf(g, s1)
    assert isinstance(n1, NoisedPytree) and n1.noise_stddev == 3.0 and s1._step_counter == 1
    assert torch.equal(n1.pytree["a"], n2.pytree["a"]) and not torch.equal(n1.pytree["a"], n3.pytree["a"])
    x = n1.pytree["a"]
    assert abs(float(x.mean())) < 0.03 and abs(float(x.std()) - 3.0) < 0.03
    from scipy import stats
    assert stats.kstest((x[:20000] / 3.0).numpy(), "norm").pvalue > 1e-3
    assert torch.equal(gaussian_noise(noise_multiplier=0.0, key=key(1))[0](g, st)[0].pytree["a"], g.pytree["a"])
    with pytest.raises(TypeError):
        nf(n1, st)
    with pytest.raises(TypeError):
        nf({"a": torch.zeros(2)}, st)


def test_bounded_gaussian_and_paired_streams():
    nf, st = gaussian_noise(noise_multiplier=1.0, bound=(0.0, 2.0), key=key(5))
    out, _ = nf(clipped({"a": torch.full((50_000,), 1.0)}, 1.0), st)
    assert float(out.pytree["a"].min()) >= 0.0 and float(out.pytree["a"].max()) <= 2.0
    nf, st = gaussian_noise(noise_multiplier=1.0, key=key(5))
    pair = SecondMomentClippingOutput(clipped({"a": torch.zeros(1000)}, 1.0), clipped({"a": torch.zeros(1000)}, 1.0))
    out, _ = nf(pair, st)
    assert math.isclose(out.noisy_grads.noise_stddev, math.sqrt(2.0))
    assert not torch.equal(out.noisy_grads.pytree["a"], out.noisy_squared_grads.pytree["a"])


def test_poisson_sampler_rate_and_resume():
    s = PoissonSampler(range(10_000), 0.05, n_steps=50, key=key(11))
    sizes = []
    it = iter(s)
    for _ in range(20):
        sizes.append(len(next(it)))
    assert abs(np.mean(sizes) - 500) < 25 and s.expected_batch_size == 500
    sd = state_dict(s)
    nxt = next(it)
    s2 = from_state_dict(PoissonSampler(range(10_000), 0.05, n_steps=50, key=key(11)), sd)
    assert len(s2) == 30 and next(iter(s2)) == nxt
    with pytest.raises(ValueError):
        from_state_dict(PoissonSampler(range(999), 0.05, n_steps=50, key=key(11)), sd)
    capped = PoissonSampler(range(1000), 0.5, n_steps=3, truncated_batch_size=100, key=key(1))
    assert all(len(b) <= 100 for b in capped)


def test_k_out_of_t_and_random_allocation_participation():
    s = KOutOfTSampler(range(200), k=2, t=5, n_steps=10, key=key(2))
    batches = list(s)
    counts = np.zeros(200)
    for b in batches[:5]:
        counts[b] += 1
    assert (counts == 2).all()
    r = RandomAllocationSampler(range(300), num_bins=6, n_steps=12, key=key(4))
    batches = list(r)
    counts = np.zeros(300)
    for b in batches[:6]:
        counts[b] += 1
    assert (counts == 1).all() and batches[0] != batches[6]


def test_adaptive_clipping_tracks_quantile():
    torch.manual_seed(0)
    W = {"w": torch.zeros(4)}

    def loss(p, x):
        return (p["w"] * x).sum()           # gradient = x, norm = |x|
    fn, st = adaptive_clipped_grad(loss, key=key(9), batch_argnums=1, initial_clipping_norm=0.1, learning_rate=0.3,
                                   fraction_noise_std=0.0, target_quantile=0.5)
    for _ in range(60):
        x = torch.randn(256, 4)
        g, st = fn(W, x, state=st)
    median = float(torch.randn(100_000, 4).norm(dim=1).median())
    assert abs(st.clipping_norm - median) / median < 0.15 and st.step == 60


def test_optimizers_against_torch_and_bc_branch():
    torch.manual_seed(0)
    p0, grads = torch.randn(5, 3), [torch.randn(5, 3) for _ in range(5)]
    for name, topt, kw in [("adamw", torch.optim.AdamW, dict(lr=1e-2, weight_decay=0.1)),
                           ("adam", torch.optim.Adam, dict(lr=1e-2, weight_decay=0.1)),
                           ("sgd", torch.optim.SGD, dict(lr=1e-2, momentum=0.9, weight_decay=0.1)),
                           ("rmsprop", torch.optim.RMSprop, dict(lr=1e-2)),
                           ("adagrad", torch.optim.Adagrad, dict(lr=1e-2)),
                           ("radam", torch.optim.RAdam, dict(lr=1e-2)),
                           ("adadelta", torch.optim.Adadelta, dict(lr=1.0))]:
        w = torch.nn.Parameter(p0.clone())
        ref = topt([w], **kw)
        mine_kw = dict(kw)
        if name in ("rmsprop", "adagrad", "adadelta"):
            mine_kw["weight_decay"] = 0.0
        opt = getattr(O, name)(**mine_kw)
        q = {"w": p0.clone()}
        st = opt.init(q)
        for g in grads:
            w.grad = g.clone()
            ref.step()
            u, st = opt.update({"w": g}, st, params=q)
            q = O.apply_updates(q, u)
        assert torch.allclose(q["w"], w.detach(), atol=2e-6), name
    # bias correction: with pure-noise gradients of variance sigma^2, BC steps are larger than plain Adam's
    sigma = 0.5
    plain, bc = O.adamw(lr=1e-2, weight_decay=0.0), O.adamw(lr=1e-2, weight_decay=0.0, noise_bias_correction=True)
    q = {"w": torch.zeros(1000)}
    s1, s2 = plain.init(q), bc.init(q)
    gen = torch.Generator().manual_seed(0)
    for _ in range(20):
        g = 0.5 + sigma * torch.randn(1000, generator=gen)
        from opaque_b200.types import noised
        u1, s1 = plain.update(noised({"w": g}, 1.0, sigma), s1, params=q)
        u2, s2 = bc.update(noised({"w": g}, 1.0, sigma), s2, params=q)
    assert float(u2["w"].abs().mean()) > float(u1["w"].abs().mean()) * 1.2
    assert math.isclose(s2.moment.phi, sigma ** 2 * (1 - 0.999 ** 20), rel_tol=1e-6)
    with pytest.raises(TypeError):
        plain.update(clipped({"w": g}, 1.0), s1, params=q)


def test_optimizer_state_round_trip():
    opt = O.adamw(noise_bias_correction=True)
    q = {"w": torch.ones(3)}
    st = opt.init(q)
    u, st = opt.update({"w": torch.ones(3)}, st, params=q)
    sd = state_dict(st)
    back = from_state_dict(opt.init(q), sd)
    assert back.step == 1 and torch.equal(back.moment.mu["w"], st.moment.mu["w"])


def test_balanced_rank_sampler_deals_one_global_draw_evenly():
    from opaque_b200.dpsgd import BalancedRankSampler, PoissonSampler
    from opaque_b200.random import key
    from opaque_b200.serialization import from_state_dict, state_dict
    world = 4
    per_rank = [list(BalancedRankSampler(PoissonSampler(range(4000), 0.05, n_steps=6, key=key(3)), r, world)) for r in range(world)]
    whole = list(PoissonSampler(range(4000), 0.05, n_steps=6, key=key(3)))
    for step in range(6):
        parts = [per_rank[r][step] for r in range(world)]
        assert sorted(i for p in parts for i in p) == sorted(whole[step])            # the union is the global draw
        assert max(map(len, parts)) - min(map(len, parts)) <= 1                       # sizes differ by at most one
    s = BalancedRankSampler(PoissonSampler(range(4000), 0.05, n_steps=6, key=key(3)), 1, world)
    it = iter(s)
    next(it), next(it)
    resumed = from_state_dict(BalancedRankSampler(PoissonSampler(range(4000), 0.05, n_steps=6, key=key(3)), 1, world), state_dict(s))
    assert list(resumed) == per_rank[1][2:]
