"""Worker of ``tests/test_reference_parity.py``: imports the unmodified reference (``baseline/_ref``, with the two stand-in
modules of ``baseline/shims``) next to this package on the CPU and prints, as one JSON object, the largest differences
between the two on pure-Python building blocks.  Run in its own process so that the reference's imports stay out of the
test session."""
import importlib
import inspect
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path[:0] = [os.path.join(ROOT, "baseline", "shims"), os.path.join(ROOT, "baseline", "_ref"), ROOT]


def both(name):
    return importlib.import_module("opaque." + name), importlib.import_module("opaque_b200." + name)


def flat(t):
    tree = getattr(t, "pytree", None)
    tree = t if tree is None else tree
    leaves = [tree[k] for k in sorted(tree)] if isinstance(tree, dict) else list(tree)
    return torch.cat([x.reshape(-1) for x in leaves])


def main():
    out = {}
    rr, ro = both("random")
    k1, k2 = rr.key(42), ro.key(42)
    out["rng_equal"] = bool(k1.seed == k2.seed and rr.fold_in(k1, 3).seed == ro.fold_in(k2, 3).seed
                            and rr.fold_in(k1, "noise").seed == ro.fold_in(k2, "noise").seed
                            and [a.seed for a in rr.split(k1, 3)] == [a.seed for a in ro.split(k2, 3)])
    sr, so = both("scheduling")
    worst = 0.0
    for name, args in (("cosine_schedule", (1.0, 0.1, 100)), ("linear_schedule", (1.0, 0.0, 50)), ("polynomial_schedule", (1.0, 0.1, 2.0, 40)),
                       ("exponential_schedule", (1.0, 10, 0.5)), ("inverse_sqrt_schedule", (1.0, 10)), ("one_minus_sqrt_schedule", (1.0, 0.0, 30))):
        a, b = getattr(sr, name)(*args), getattr(so, name)(*args)
        worst = max(worst, max(abs(float(a(t)) - float(b(t))) for t in (0, 1, 7, 25, 60, 200)))
    a, b = sr.with_warmup(sr.cosine_schedule(1.0, 0.1, 90), 10), so.with_warmup(so.cosine_schedule(1.0, 0.1, 90), 10)
    worst = max(worst, max(abs(float(a(t)) - float(b(t))) for t in range(0, 120, 7)))
    kw = dict(num_warmup_steps=5, num_stable_steps=20, num_decay_steps=10)
    a, b = sr.warmup_stable_decay(1.0, 0.0, **kw), so.warmup_stable_decay(1.0, 0.0, **kw)
    out["schedules"] = max(worst, max(abs(float(a(t)) - float(b(t))) for t in range(0, 40)))

    dr, do = both("dpsgd")
    fr, fo = both("functional")
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(6, 5), torch.nn.Tanh(), torch.nn.Linear(5, 3))
    X, Y = torch.randn(12, 6), torch.randint(0, 3, (12,))

    def run(D, Fm, R):
        fmodel, params = Fm.make_functional(model, disable_autograd_tracking=True)
        loss = lambda p, x, y: torch.nn.functional.cross_entropy(fmodel(p, x[None]), y[None])
        gf, cs = D.clipped_grad(loss, clipping_norm=0.7, normalize_by=12.0, batch_argnums=(1, 2), return_aux=True, microbatch_size=5)
        (g, aux), cs = gf(params, X, Y, state=cs)
        nf, ns = D.gaussian_noise(noise_multiplier=1.3, key=R.key(9))
        noisy, ns = nf(g, ns)
        return g, noisy, aux
    g1, n1, a1 = run(dr, fr, rr)
    g2, n2, a2 = run(do, fo, ro)
    out["clipped_grad"] = float((flat(g1) - flat(g2)).abs().max())
    out["grad_norms"] = float((a1.grad_norms - a2.grad_norms).abs().max())
    out["noise_realisation"] = float((flat(n1) - flat(n2)).abs().max())
    out["noise_std"] = float((flat(n2) - flat(g2)).std())

    fr_, fo_ = both("dpftrl")
    same = lambda a, b: [list(x) for x in a] == [list(x) for x in b]
    out["poisson_draws_equal"] = same(dr.PoissonSampler(range(200), 0.1, n_steps=6, key=rr.key(5)), do.PoissonSampler(range(200), 0.1, n_steps=6, key=ro.key(5)))
    out["random_allocation_draws_equal"] = same(dr.sampling.RandomAllocationSampler(range(50), num_bins=5, n_steps=10, key=rr.key(1)),
                                                 do.RandomAllocationSampler(range(50), 5, 10, key=ro.key(1)))
    out["balls_in_bins_draws_equal"] = same(fr_.BallsInBinsSampler(range(60), num_bins=5, n_steps=10, key=rr.key(2)),
                                             fo_.BallsInBinsSampler(range(60), num_bins=5, n_steps=10, key=ro.key(2)))

    orr, oo = both("optimizers")
    tr, to = both("types")
    torch.manual_seed(1)
    p = {"w": torch.randn(7), "b": torch.randn(3)}

    def steps(O, T):
        opt = O.adamw(1e-2, weight_decay=0.1, noise_bias_correction=True)
        st, q = opt.init(p), {k: v.clone() for k, v in p.items()}
        g = torch.Generator().manual_seed(3)
        for _ in range(4):
            grads = {k: torch.randn(v.shape, generator=g) for k, v in q.items()}
            u, st = opt.update(T.noised(grads, max_norm=1.0, noise_stddev=0.3), st, params=q)
            q = {k: q[k] + u[k] for k in q}            # the update is additive in both libraries
        return q
    q1, q2 = steps(orr, tr), steps(oo, to)
    out["adamw_bc"] = max(float((q1[k] - q2[k]).abs().max()) for k in q1)

    def steps_with(O, T, make):
        opt = make(O)
        st, q = opt.init(p), {k: v.clone() for k, v in p.items()}
        g = torch.Generator().manual_seed(3)
        for _ in range(5):
            grads = {k: torch.randn(v.shape, generator=g) for k, v in q.items()}
            u, st = opt.update(T.noised(grads, max_norm=1.0, noise_stddev=0.3), st, params=q)
            q = {k: q[k] + u[k] for k in q}
        return q
    worst = 0.0
    for make in (lambda O: O.sgd(1e-2, momentum=0.9, weight_decay=0.01), lambda O: O.sgd(1e-2, momentum=0.9, nesterov=True), lambda O: O.adam(1e-2),
                 lambda O: O.lion(1e-3, weight_decay=0.1), lambda O: O.adagrad(1e-2, noise_bias_correction=True),
                 lambda O: O.rmsprop(1e-2, noise_bias_correction=True), lambda O: O.radam(1e-2), lambda O: O.adadelta(1.0),
                 lambda O: O.ademamix(1e-2), lambda O: O.adamw(1e-2, update_rms_clip=1.0), lambda O: O.adafactor(1e-2),
                 lambda O: O.adafactor(1e-2, beta1=0.9, noise_bias_correction=True, weight_decay=0.01)):
        a, b = steps_with(orr, tr, make), steps_with(oo, to, make)
        worst = max(worst, max(float((a[k] - b[k]).abs().max()) for k in a))
    out["other_optimizers"] = worst

    def clip_variant(D, Fm, R, which):
        fmodel, params = Fm.make_functional(model, disable_autograd_tracking=True)
        loss = lambda p_, x, y: torch.nn.functional.cross_entropy(fmodel(p_, x[None]), y[None])
        common = dict(normalize_by=12.0, batch_argnums=(1, 2), return_aux=True)
        if which == "auto":
            gf, cs = D.auto_clipped_grad(loss, R=0.5, gamma=0.02, **common)
        elif which == "adaptive":
            gf, cs = D.adaptive_clipped_grad(loss, initial_clipping_norm=0.3, key=R.key(4), **common)
        else:
            gf, cs = D.clipped_grad(loss, clipping_norm=0.7, second_moment=True, **common)
        outs = []
        for _ in range(3):
            (g, _aux), cs = gf(params, X, Y, state=cs)
            outs.append(flat(g.grads) if hasattr(g, "grads") else flat(g))
        return torch.cat(outs)
    out["clipping_variants"] = max(float((clip_variant(dr, fr, rr, w) - clip_variant(do, fo, ro, w)).abs().max()) for w in ("auto", "adaptive", "second"))

    ref, ours = importlib.import_module("opaque.alignment.dpo.loss"), importlib.import_module("opaque_b200.alignment.dpo.loss")
    torch.manual_seed(0)
    c, r = torch.randn(9), torch.randn(9)
    lc, lr_ = -torch.rand(9) * 2 - 0.1, -torch.rand(9) * 2 - 0.1
    worst = 0.0
    for name in ("sigmoid_loss", "hinge_loss", "robust_loss", "ipo_loss", "discopop_loss", "apo_zero_loss", "apo_down_loss", "exo_loss",
                 "nca_loss", "bco_loss", "sppo_loss", "simpo_loss"):
        worst = max(worst, float((getattr(ref, name)(c, r, beta=0.3) - getattr(ours, name)(c, r, beta=0.3)).abs().max()))
    worst = max(worst, float((ref.odds_ratio_loss(lc, lr_) - ours.odds_ratio_loss(lc, lr_)).abs().max()),
                float((ref.chosen_nll_loss(lc) - ours.chosen_nll_loss(lc)).abs().max()))
    for kind in ("reverse_kl", "forward_kl", "js_divergence", "alpha_divergence"):
        for alpha in (0.3, 0.5):
            worst = max(worst, float((ref.f_divergence_logits(c, r, f_divergence_type=kind, alpha=alpha)
                                      - ours.f_divergence_logits(c, r, f_divergence_type=kind, alpha=alpha)).abs().max()),
                        float((ref.f_divergence_remap(c, f_divergence_type=kind, alpha=alpha)
                               - ours.f_divergence_remap(c, f_divergence_type=kind, alpha=alpha)).abs().max()))
    lp = -torch.rand(3, 6)
    m = torch.tensor([[0, 1, 1, 1, 0, 0], [1, 1, 1, 1, 1, 1], [0, 0, 0, 0, 0, 0]])
    logits, ids = torch.randn(2, 6, 11), torch.randint(0, 11, (2, 6))
    worst = max(worst, float((ref.wpo_weights(lp, m) - ours.wpo_weights(lp, m)).abs().max()),
                float((ref.ld_dpo_split(lp, m, 2, 0.3) - ours.ld_dpo_split(lp, m, 2, 0.3)).abs().max()),
                float((ref.sequence_logp(logits, ids, m[:2]) - ours.sequence_logp(logits, ids, m[:2])).abs().max()),
                float((ref.sequence_logp(logits, ids, m[:2], ld_alpha=0.4, shared_prefix_len=2)
                       - ours.sequence_logp(logits, ids, m[:2], ld_alpha=0.4, shared_prefix_len=2)).abs().max()),
                float((ref.mpo_combine({"a": c, "b": r}, {"a": 0.3, "b": 2.0}) - ours.mpo_combine({"a": c, "b": r}, {"a": 0.3, "b": 2.0})).abs().max()))
    out["preference_losses"] = worst

    # collators (factory form, unshifted labels) and the shift-inside SFT losses
    ra, oa = importlib.import_module("opaque.alignment"), importlib.import_module("opaque_b200.alignment")
    rows = [{"input_ids": [1, 2, 3, 4, 5], "completion_mask": [0, 0, 1, 1, 1]}, {"input_ids": [6, 7, 8], "completion_mask": [0, 1, 1]}]
    pairs = [{"chosen_input_ids": [1, 2, 3, 4, 5], "chosen_completion_mask": [0, 0, 0, 1, 1], "rejected_input_ids": [1, 2, 3, 6],
              "rejected_completion_mask": [0, 0, 0, 1], "ref_chosen_logps": -1.0, "ref_rejected_logps": -2.0},
             {"chosen_input_ids": [7, 8, 9, 10], "chosen_completion_mask": [0, 1, 1, 1], "rejected_input_ids": [7, 11, 12],
              "rejected_completion_mask": [0, 1, 1], "ref_chosen_logps": -1.5, "ref_rejected_logps": -2.5}]
    same_batch = lambda a, b: sorted(a) == sorted(b) and all(torch.equal(torch.as_tensor(a[k]), torch.as_tensor(b[k])) for k in a)
    ok = True
    for col in (True, False):
        for mult in (None, 4):
            kw = dict(completion_only_loss=col, pad_to_multiple_of=mult)
            ok &= same_batch(ra.sft.collator.language_modeling_collator(0, 4, **kw)(rows), oa.sft.collator.language_modeling_collator(0, 4, **kw)(rows))
    e1, e2 = ra.sft.collator.language_modeling_collator(0, 8)([]), oa.sft.collator.language_modeling_collator(0, 8)([])
    ok &= all(e1[k].shape == e2[k].shape for k in e1)
    for ml, mult in ((4, None), (16, 8)):
        ok &= same_batch(ra.dpo.collator.preference_collator(0, ml, pad_to_multiple_of=mult)(pairs),
                         oa.dpo.collator.preference_collator(0, ml, pad_to_multiple_of=mult)(pairs))
    out["collators_equal"] = bool(ok)
    torch.manual_seed(0)
    logits, hid, head = torch.randn(2, 5, 13), torch.randn(5, 6), torch.randn(13, 6)
    lab = ra.sft.collator.language_modeling_collator(0, 8, completion_only_loss=True)(rows)["labels"]
    worst = 0.0
    for name in ("nll_loss", "dft_loss"):
        worst = max(worst, float((getattr(ra.sft.loss, name)(logits, lab) - getattr(oa.sft.loss, name)(logits, lab)).abs().max()))
    for name in ("fused_nll_loss", "fused_dft_loss"):          # the reference's fused forms take ONE example
        worst = max(worst, float((getattr(ra.sft.loss, name)(hid, head, lab[0]) - getattr(oa.sft.loss, name)(hid[None], head, lab[:1])[0]).abs().max()))
    worst = max(worst, float((ra.metric.entropy_from_logits(logits, lab != -100) - oa.metric.entropy_from_logits(logits, lab != -100)).abs()),
                float((ra.metric.mean_token_accuracy(logits, lab.clamp_min(0), lab != -100) - oa.metric.mean_token_accuracy(logits, lab.clamp_min(0), lab != -100)).abs()))
    out["sft_losses_and_metrics"] = worst
    # ------------------------------------------------------------------ DP-FTRL: strategies and correlated noise
    import numpy as np
    fr, fo = both("dpftrl")
    lr = lambda t: 1.0 / (1 + t)
    worst = 0.0
    for n, kw in ((8, dict(bands=4)), (32, dict(bands=4, momentum=0.9)), (32, dict(bands=3, lr_schedule=lr))):
        a, b = fr.band_mf_strategy(**kw), fo.band_mf_strategy(**kw)
        worst = max(worst, float(np.abs(np.asarray(a.coefficients(n_steps=n)) - np.asarray(b.coefficients(n_steps=n))).max()))
    out["band_mf_coefficients"] = worst
    a, b = fr.bsr_strategy(bandwidth=4, alpha=1.0, beta=0.9), fo.bsr_strategy(bandwidth=4, alpha=1.0, beta=0.9)
    out["bsr_sensitivity"] = max(abs(float(a.sensitivity(n_steps=16, min_sep=ms, max_participations=mp))
                                     - float(b.sensitivity(n_steps=16, min_sep=ms, max_participations=mp)))
                                 for ms, mp in ((1, None), (4, None), (4, 2)))
    worst, spread = 0.0, 0.0
    for make in (lambda F: F.identity_strategy(), lambda F: F.band_mf_strategy(bands=4),
                 lambda F: F.bsr_strategy(bandwidth=4, alpha=1.0, beta=0.9),
                 lambda F: F.lambda_cgd_strategy(lambda_=0.5), lambda F: F.lambda_cgd_strategy(lambda_=0.5, normalized=False)):
        runs = []
        for F, T, R in ((fr, tr, rr), (fo, to, ro)):
            nf, ns = F.mf_gaussian_noise({"w": torch.zeros(6)}, make(F), n_steps=8, noise_multiplier=1.0, key=R.key(3))
            rows = []
            for _ in range(5):
                o, ns = nf(T.clipped({"w": torch.zeros(6)}, max_norm=1.0), ns)
                rows.append(torch.cat([o.pytree["w"], torch.tensor([float(o.noise_stddev)])]))
            runs.append(torch.stack(rows))
        worst = max(worst, float((runs[0] - runs[1]).abs().max()))
        spread = max(spread, float(runs[1].std()))
    out["mf_noise_realisation"], out["mf_noise_std"] = worst, spread
    # ------------------------------------------------------------------ auditing: order-statistics audits on the same scores
    import dataclasses
    ra_, oa_ = both("auditing")
    worst = 0.0
    for shift in (0.5, 2.0, 6.0):
        n = 200
        ca, cb = ra_.coin_flip(list(range(n)), num_canaries=n, key=rr.key(5)), oa_.coin_flip(list(range(n)), num_canaries=n, key=ro.key(5))
        member = np.zeros(n, bool)
        member[np.asarray(ca.in_indices)] = True
        values = np.where(member, shift, 0.0) + np.random.default_rng(1).normal(size=n)
        ea = ra_.one_run(ra_.canary_scores(values[np.asarray(ca.canary_indices)], canary_indices=ca.canary_indices), coin_flip=ca)
        eb = oa_.one_run(oa_.canary_scores(values[np.asarray(cb.canary_indices)], canary_indices=cb.canary_indices), coin_flip=cb)
        eb = dataclasses.replace(eb, in_scores=np.asarray(ea.in_scores), out_scores=np.asarray(ea.out_scores))   # the same split on both sides
        for d in (0.0, 1e-5, 0.05):
            worst = max(worst, abs(ea.eps_delta().epsilon_at(delta=d) - eb.eps_delta().epsilon_at(delta=d)),
                        abs(ea.eps_delta().epsilon_at(delta=d, threshold=shift / 2) - eb.eps_delta().epsilon_at(delta=d, threshold=shift / 2)))
        worst = max(worst, abs(ea.eps_delta().delta_at(epsilon=0.5) - eb.eps_delta().delta_at(epsilon=0.5)),
                    abs(ea.gdp(grid_size=2000).epsilon_at(delta=1e-5) - eb.gdp(grid_size=2000).epsilon_at(delta=1e-5)),
                    abs(ea.gdp(grid_size=2000).delta_at(epsilon=1.0) - eb.gdp(grid_size=2000).delta_at(epsilon=1.0)),
                    abs(ea.gdp(grid_size=2000).beta_at(alpha=0.1) - eb.gdp(grid_size=2000).beta_at(alpha=0.1)),
                    abs(ea.gdp(grid_size=2000).advantage() - eb.gdp(grid_size=2000).advantage()))
    out["order_statistics_audits"] = worst
    out["signature_checked"] = len(inspect.signature(ref.sigmoid_loss).parameters)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
