"""Building blocks added for import-path parity: preference-loss pieces, token metrics, reference helpers, fused DFT loss,
and the factory API for in-place family patches — each against its closed form."""
import math
import os

import pytest
import torch
import torch.nn.functional as F

from opaque_b200.alignment import dpo, metric, reference, sft


def test_preference_loss_pieces_match_their_closed_forms():
    torch.manual_seed(0)
    c, r = -torch.rand(7) * 3 - 0.05, -torch.rand(7) * 3 - 0.05          # length-normalised log-probabilities (< 0)
    odds = lambda lp: lp - torch.log1p(-lp.exp())
    assert torch.allclose(dpo.odds_ratio_loss(c, r), -F.logsigmoid(odds(c) - odds(r)), atol=1e-6)
    tiny = torch.tensor([-1e-9, -30.0])                                   # both ends of log(1 - e^x) stay finite
    assert torch.isfinite(dpo.odds_ratio_loss(tiny, tiny.flip(0))).all()
    x = torch.randn(9)
    assert torch.equal(dpo.f_divergence_remap(x), x)
    assert torch.allclose(dpo.f_divergence_remap(x, f_divergence_type="forward_kl"), 1 - torch.exp(-x))
    assert torch.allclose(dpo.f_divergence_remap(x, f_divergence_type="js_divergence"), math.log(2) + F.logsigmoid(x))
    assert torch.allclose(dpo.f_divergence_remap(x, f_divergence_type="alpha_divergence", alpha=0.5), (torch.exp(-0.5 * x) - 1) / -0.5)
    assert torch.equal(dpo.f_divergence_remap(x, f_divergence_type="alpha_divergence", alpha=1.0), x)
    assert torch.isfinite(dpo.f_divergence_remap(torch.tensor([-500.0]), f_divergence_type="forward_kl")).all()
    with pytest.raises(ValueError):
        dpo.f_divergence_remap(x, f_divergence_type="chi2")
    losses = {"sigmoid": torch.tensor([1.0, 2.0]), "sft": torch.tensor([3.0, 5.0]), "ipo": torch.tensor([9.0, 9.0])}
    assert torch.equal(dpo.mpo_combine(losses, {"sigmoid": 1.0, "sft": 0.5}), torch.tensor([2.5, 4.5]))
    with pytest.raises(KeyError):
        dpo.mpo_combine(losses, {"hinge": 1.0})
    lp = torch.tensor([[-0.5, -1.0, -2.0, -4.0], [-1.0, -1.0, -1.0, -1.0]], requires_grad=True)
    mask = torch.tensor([[0, 1, 1, 1], [0, 0, 0, 0]])
    w = dpo.wpo_weights(lp, mask)
    assert torch.allclose(w, torch.tensor([math.exp(-7 / 3), 1.0])) and not w.requires_grad
    # LD-DPO: the first 2 completion tokens weigh 1, later ones alpha
    got = dpo.ld_dpo_split(lp.detach(), mask, 2, 0.25)
    assert torch.allclose(got, torch.tensor([-1.0 - 2.0 - 0.25 * 4.0, 0.0]))
    assert torch.allclose(dpo.ld_dpo_split(lp.detach(), mask, torch.tensor([1, 3]), 0.0), torch.tensor([-1.0, 0.0]))
    assert torch.allclose(dpo.ld_dpo_split(lp.detach(), mask, 2, 1.0), (lp.detach() * mask).sum(-1))
    m = dpo.reward_metrics(torch.tensor([1.0, -1.0, 2.0]), torch.tensor([0.0, 0.0, 3.0]), beta=0.5)
    assert set(m) == {"rewards/chosen", "rewards/rejected", "rewards/accuracies", "rewards/margins"}
    assert float(m["rewards/accuracies"]) == pytest.approx(1 / 3) and float(m["rewards/margins"]) == pytest.approx(0.5 * (1 - 1 - 1) / 3)
    row = dpo.extract_prompt({"chosen": [1, 2, 3, 4], "rejected": [1, 2, 9], "id": 7})
    assert row == {"prompt": [1, 2], "chosen": [3, 4], "rejected": [9], "id": 7}
    same = {"prompt": [1], "chosen": [2], "rejected": [3]}
    assert dpo.extract_prompt(same) == same and dpo.extract_prompt({"prompt": "p", "completion": "c"}) == {"prompt": "p", "completion": "c"}
    msgs = dpo.extract_prompt({"chosen": [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "a"}],
                               "rejected": [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "b"}]})
    assert msgs["prompt"] == [{"role": "user", "content": "hi"}] and msgs["chosen"][0]["content"] == "a"


def test_token_metrics_shift_and_mask():
    torch.manual_seed(1)
    logits = torch.randn(2, 5, 11)
    labels = torch.randint(0, 11, (2, 5))
    mask = torch.tensor([[1, 1, 1, 0, 0], [0, 0, 1, 1, 1]])
    p = logits[:, :-1].softmax(-1)
    ent = -(p * p.log()).sum(-1)
    m = mask[:, 1:].float()
    assert float(metric.entropy_from_logits(logits, mask)) == pytest.approx(float((ent * m).sum() / m.sum()), rel=1e-5)
    hit = (logits[:, :-1].argmax(-1) == labels[:, 1:]).float()
    assert float(metric.mean_token_accuracy(logits, labels, mask)) == pytest.approx(float((hit * m).sum() / m.sum()))
    assert float(metric.mean_token_accuracy(logits, labels, torch.zeros_like(mask))) == 0.0
    assert float(metric.entropy_from_logits(logits, torch.zeros_like(mask))) == 0.0


def test_fused_dft_loss_equals_the_logits_form_with_gradients():
    torch.manual_seed(2)
    B, T, d, V = 3, 6, 16, 40
    hidden = torch.randn(B, T, d, requires_grad=True)
    head = torch.randn(V, d, requires_grad=True) * 0.3
    head.retain_grad()
    labels = torch.randint(0, V, (B, T))
    labels[0, :2] = -100
    labels[2, -1] = -100
    want = sft.dft_loss(hidden @ head.t(), labels)
    got = sft.fused_dft_loss(hidden, head, labels)
    assert torch.allclose(got, want, atol=1e-5)
    gw = torch.autograd.grad(want.sum(), hidden, retain_graph=True)[0]
    gg = torch.autograd.grad(got.sum(), hidden)[0]
    assert torch.allclose(gg, gw, atol=1e-5)


def test_reference_helpers(tmp_path):
    from opaque_b200.models import LlamaConfig, LlamaForCausalLM
    torch.manual_seed(3)
    model = LlamaForCausalLM(LlamaConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=2,
                                         num_key_value_heads=2, max_position_embeddings=32), dtype=torch.float32).eval()
    ids = torch.randint(0, 64, (2, 8))
    with torch.no_grad():
        base = model(ids)
    model.add_lora(4, 8.0, ("q_proj", "v_proj"))
    with torch.no_grad():
        for n, p in model.named_parameters():
            if n.endswith("lora_B"):
                p.normal_(0, 0.1)
        tuned = model(ids)
        assert not torch.allclose(tuned, base, atol=1e-4)
        with reference.with_disabled_adapter(model):
            assert torch.allclose(model(ids), base, atol=1e-6)
        with reference.null_ref_context(model):
            assert torch.allclose(model(ids), base, atol=1e-6)
        with reference.null_ref_context(model, ref_model=object()):          # a separate reference: the policy is left alone
            assert torch.allclose(model(ids), tuned, atol=1e-6)
        assert torch.allclose(model(ids), tuned, atol=1e-6)                   # restored

    class FakePeft:                                  # the PEFT calls that null_ref_context makes, recorded
        def __init__(self, adapters):
            self.peft_config, self.active_adapter, self.calls = {a: None for a in adapters}, "default", []

        def disable_adapter(self):
            import contextlib

            @contextlib.contextmanager
            def cm():
                self.calls.append("off")
                yield
                self.calls.append("on")
            return cm()

        def set_adapter(self, name):
            self.calls.append(f"set:{name}")
    plain, with_ref = FakePeft(["default"]), FakePeft(["default", "ref"])
    with reference.null_ref_context(plain):
        pass
    with reference.null_ref_context(with_ref):
        pass
    assert plain.calls == ["off", "on"] and with_ref.calls == ["set:ref", "set:default"]

    ref_p, pol_p = {"w": torch.zeros(3), "b": {"x": torch.ones(2)}}, {"w": torch.ones(3), "b": {"x": torch.zeros(2)}}
    out = reference.ema_update_reference(ref_p, pol_p, 0.25)
    assert torch.allclose(out["w"], torch.full((3,), 0.25)) and torch.allclose(out["b"]["x"], torch.full((2,), 0.75)) and float(ref_p["w"].sum()) == 0
    with pytest.raises(ValueError):
        reference.ema_update_reference(ref_p, pol_p, 1.5)

    rows = [{"v": float(i)} for i in range(11)]
    calls = []

    def ref_fn(batch):
        calls.append(len(batch["v"]))
        return {"ref_chosen_logps": batch["v"] * 2, "ref_rejected_logps": -batch["v"]}
    collate = lambda rs: {"v": torch.tensor([r["v"] for r in rs])}
    kw = dict(cache_identity={"model": "m", "step": 0}, batch_size=4, cache_dir=str(tmp_path / "cache"))
    out = reference.compute_ref_logprobs_for_dataset(rows, ref_fn, collate, ("ref_chosen_logps", "ref_rejected_logps"), **kw)
    assert [r["ref_chosen_logps"] for r in out] == [2.0 * i for i in range(11)] and out[3]["ref_rejected_logps"] == -3.0 and calls == [4, 4, 3]
    again = reference.compute_ref_logprobs_for_dataset(rows, ref_fn, collate, ("ref_chosen_logps", "ref_rejected_logps"), **kw)
    assert again == out and calls == [4, 4, 3]                                  # served from the cache
    files = os.listdir(tmp_path / "cache")
    assert len(files) == 1 and oct(os.stat(tmp_path / "cache" / files[0]).st_mode & 0o777) == "0o600"
    assert oct(os.stat(tmp_path / "cache").st_mode & 0o777) == "0o700"
    other = reference.compute_ref_logprobs_for_dataset(rows, ref_fn, collate, ("ref_chosen_logps", "ref_rejected_logps"),
                                                       **{**kw, "cache_identity": {"model": "m", "step": 1}})
    assert other == out and len(calls) == 6 and len(os.listdir(tmp_path / "cache")) == 2     # another identity: recomputed
    with pytest.raises(TypeError):
        reference.compute_ref_logprobs_for_dataset(rows, ref_fn, collate, ("ref_chosen_logps",), cache_identity=object(), cache_dir=str(tmp_path / "c2"))
    with pytest.raises(RuntimeError):
        reference.compute_ref_logprobs_for_dataset(rows, ref_fn, collate, ("ref_chosen_logps",), cache_identity=1, shard=True, use_cache=False)


def test_factory_api_patches_a_new_family_in_place():
    """A family described as data: class names per role and registered kinds; applied through ``apply_model_patches``."""
    from opaque_b200 import patches
    from opaque_b200.patches import inplace
    from opaque_b200.patches.transformers import make_apply_family_patches, make_apply_model_patches, register_family, register_rms_norm_kind

    class ToyNorm(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.weight = torch.nn.Parameter(torch.ones(8))

        def forward(self, x):
            return x * self.weight

    class ToyMLP(torch.nn.Module):
        def forward(self, x):
            return x + 1

    class Toy(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.config = {"model_type": "toy_family"}
            self.norm, self.norm2, self.mlp = ToyNorm(), ToyNorm(), ToyMLP()

        def forward(self, x):
            return self.mlp(self.norm2(self.norm(x)))
    seen = []
    register_rms_norm_kind("doubling", lambda original: (lambda x: 2 * original(x)))
    family_apply = make_apply_family_patches("toy_family", lambda: seen.append("runtime"))
    apply = make_apply_model_patches(family="toy_family", family_apply=family_apply, classes={"rms_norm": "ToyNorm", "mlp": "ToyMLP"},
                                     rms_norm_kind="doubling", activation_kind=lambda original: (lambda x: original(x) * 10))
    register_family("toy_family", apply)
    assert inplace.family_name(Toy()) == "toy_family"
    model, x = Toy(), torch.ones(8)
    assert float(model(x)[0]) == 2.0
    out = patches.apply_model_patches(model)
    assert out is model and float(model(x)[0]) == (2 * 2 * 1 + 1) * 10 and seen == ["runtime"]
    assert apply(model) == {"rms_norm": 2, "mlp": 1} and float(model(x)[0]) == 50.0 and seen == ["runtime"]      # idempotent, runtime once
    assert inplace.remove_factory_patches(model) == 3 and float(model(x)[0]) == 2.0
    assert apply(Toy(), mlp=False) == {"rms_norm": 2, "mlp": 0}
    with pytest.raises(ValueError, match="not registered"):
        make_apply_model_patches(family="t", classes={"rms_norm": "ToyNorm"}, rms_norm_kind="nope")


def test_auditing_dataset_forms_join_scores_by_identifier():
    """The dataset forms of ``loss_scores`` / ``gradient_scores`` (per-example loss as for ``clipped_grad``) against plain
    loops; scores carry the canaries' dataset indices, so a shuffled copy audits the same."""
    import numpy as np
    from opaque_b200 import auditing
    from opaque_b200.random import key
    torch.manual_seed(0)
    X, Y = torch.randn(60, 5), torch.randn(60)
    data = [(X[i], Y[i]) for i in range(60)]
    flips = auditing.coin_flip(data, num_canaries=20, key=key(1))
    kept = flips.kept_indices()
    w0, w = torch.zeros(5), torch.linalg.lstsq(X[kept], Y[kept].unsqueeze(1)).solution.squeeze(1)
    loss = lambda p, x, y: (x @ p - y) ** 2
    kw = dict(batch_argnums=(1, 2), coin_flip=flips, dataset=data, batch_size=7)
    ref = auditing.loss_scores(loss, w0, **kw)
    cur = auditing.loss_scores(loss, w, reference_scores=ref, **kw)
    want = np.array([float(loss(w0, *data[i]) - loss(w, *data[i])) for i in flips.canary_indices])
    assert np.allclose(cur.scores, want, atol=1e-5) and np.array_equal(cur.canary_indices, flips.canary_indices)
    grad = auditing.gradient_scores(loss, w, **kw)
    want_g = np.array([-float(((2 * (data[i][0] @ w - data[i][1]) * data[i][0]) ** 2).sum()) for i in flips.canary_indices])
    assert np.allclose(grad.scores, want_g, rtol=1e-4)
    shuffled = auditing.canary_scores(cur.scores[::-1].copy(), canary_indices=cur.canary_indices[::-1].copy())
    a, b = auditing.one_run(shuffled, coin_flip=flips), auditing.one_run(cur, coin_flip=flips)
    assert (a.num_correct, a.num_guesses, a.epsilon_lower_bound) == (b.num_correct, b.num_guesses, b.epsilon_lower_bound)
    legacy = auditing.loss_scores(lambda c: (c[0] @ w - c[1]) ** 2, [data[i] for i in flips.canary_indices])
    assert np.allclose(legacy.scores, -np.array([float(loss(w, *data[i])) for i in flips.canary_indices]), atol=1e-6)
    with pytest.raises(ValueError):
        auditing.gradient_scores(loss, w, batch_argnums=(0, 1), coin_flip=flips, dataset=data)
    with pytest.raises(TypeError):
        auditing.loss_scores(loss, w, reference_scores=legacy, **kw)
    with pytest.raises(ValueError):
        auditing.canary_scores([1.0, 2.0], canary_indices=[3, 3])
    with pytest.raises(ValueError):
        auditing.one_run(auditing.canary_scores(cur.scores, canary_indices=np.arange(20) + 1000), coin_flip=flips)


def test_completion_logp_shifts_and_matches_the_aligned_form():
    from opaque_b200.alignment.dpo.loss import fused_sequence_logp, sequence_logp
    torch.manual_seed(4)
    B, T, d, V = 2, 7, 8, 19
    hidden, head = torch.randn(B, T, d), torch.randn(V, d) * 0.4
    logits = hidden @ head.t()
    ids = torch.randint(0, V, (B, T))
    mask = torch.tensor([[0, 0, 1, 1, 1, 0, 0], [0, 1, 1, 1, 1, 1, 1]])
    labels = torch.full_like(ids, -100)
    labels[:, :-1] = torch.where(mask[:, 1:] != 0, ids[:, 1:], torch.full_like(ids[:, 1:], -100))
    want = sft.sequence_logp(logits, labels)
    assert torch.allclose(sequence_logp(logits, ids, mask), want, atol=1e-5)
    assert torch.allclose(sequence_logp(logits, ids, mask, length_normalized=True), sft.sequence_logp(logits, labels, average=True), atol=1e-5)
    assert torch.allclose(fused_sequence_logp(hidden, head, ids, mask), want, atol=1e-4)
    lp = torch.gather(logits[:, :-1].log_softmax(-1), -1, ids[:, 1:, None]).squeeze(-1)
    assert torch.allclose(sequence_logp(logits, ids, mask, ld_alpha=0.5, shared_prefix_len=2), dpo.ld_dpo_split(lp, mask[:, 1:], 2, 0.5), atol=1e-5)
    with pytest.raises(ValueError):
        sequence_logp(logits, ids, mask, ld_alpha=0.5)


def test_audit_estimate_answers_the_reference_questions():
    import numpy as np
    from opaque_b200 import auditing
    from opaque_b200.random import key
    data = list(range(400))
    flips = auditing.coin_flip(data, num_canaries=200, key=key(3))
    assert len(flips.in_indices) + len(flips.out_indices) == 200 and set(flips.in_indices).isdisjoint(flips.out_indices)
    assert len(flips.train_indices(400)) == 400 - len(flips.out_indices) == len(flips.train_subset(data))
    with pytest.raises(ValueError):
        flips.train_indices(399)
    scores = np.where(flips.included, 1.2, -1.2) + np.random.default_rng(0).normal(0, 1.0, 200)
    cs = auditing.canary_scores(scores, canary_indices=flips.canary_indices)
    ins, outs = flips.split_scores(cs)
    assert len(ins) == int(flips.included.sum()) and ins.mean() > outs.mean()
    est = auditing.one_run(cs, coin_flip=flips, delta=1e-5)
    assert est.epsilon_at(delta=1e-5) == pytest.approx(est.epsilon_lower_bound) and est.epsilon_at(delta=1e-5, significance=0.2) >= est.epsilon_lower_bound
    mu = est.gdp_mu()
    assert mu > 0 and 0 < est.delta_at(epsilon=0.5) < 1 and est.delta_at(epsilon=0.5) > est.delta_at(epsilon=2.0)
    assert 0 < est.beta_at(alpha=0.1) < 0.9 and 0 < est.advantage() < 1
    point, (lo, hi) = est.attack_auc(confidence=0.9, num_samples=200, key=key(1))
    assert 0.9 < lo <= point <= hi <= 1.0 and est.attack_auc() == point
    betas = est.attack_beta_at(alpha=np.array([0.0, 0.1, 1.0]))
    assert betas[0] >= betas[1] >= betas[2] == 0.0 and est.attack_beta_at(alpha=0.1) == betas[1]
    noise_only = auditing.one_run(auditing.canary_scores(np.random.default_rng(1).normal(size=200)), coin_flip=flips, delta=1e-5)
    assert noise_only.epsilon_at(delta=1e-5) == 0.0 and abs(noise_only.attack_auc() - 0.5) < 0.1 and noise_only.advantage() < 0.2


def test_order_statistics_audits_on_one_estimate():
    """``eps_delta()``: exact Binomial test on all canaries; ``gdp()``: the μ-GDP order-statistics test.  A strong attack
    certifies more than a weak one, more δ certifies less ε, μ-GDP certifies more than the assumption-free test, and the
    pieces (rank error probabilities, Chernoff tail) behave as their definitions say."""
    import dataclasses

    import numpy as np
    from scipy import stats

    from opaque_b200 import auditing as A
    from opaque_b200.random import key
    rng = np.random.default_rng(0)
    def estimate(shift, n=300):
        flips = A.coin_flip(list(range(n)), num_canaries=n, key=key(3))
        member = np.zeros(n, bool)
        member[np.asarray(flips.in_indices)] = True
        values = np.where(member, shift, 0.0) + rng.normal(size=n)
        ids = np.asarray(flips.canary_indices)
        return A.one_run(A.canary_scores(values[ids], canary_indices=ids), coin_flip=flips)
    weak, strong = estimate(0.5), estimate(3.0)
    ed = strong.eps_delta()
    r, u = ed.guesses_and_errors()
    assert r == 300 and u == min(ed.guesses_and_errors(t)[1] for t in np.r_[strong.in_scores, strong.out_scores])
    assert ed.epsilon_at() > weak.eps_delta().epsilon_at() >= 0.0
    assert ed.epsilon_at(delta=0.0) >= ed.epsilon_at(delta=0.1) and ed.epsilon_at(threshold=1.5) <= ed.epsilon_at() + 1e-9
    eps = ed.epsilon_at()
    assert ed.p_value(r, u, eps - 1e-3, 0.0) < 0.05 <= ed.p_value(r, u, eps + 1e-3, 0.0)
    assert ed.delta_at(epsilon=eps + 1.0) == 0.0 and ed.delta_at(epsilon=0.1) > 0.0
    g = strong.gdp()
    mu = g.mu_at()
    assert 1.5 < mu < 3.5 and weak.gdp().mu_at() < mu                      # the canaries are 3 standard deviations apart
    assert g.epsilon_at(delta=1e-5) > ed.epsilon_at(delta=1e-5)
    assert g.delta_at(epsilon=g.epsilon_at(delta=1e-3)) == pytest.approx(1e-3, rel=1e-3)
    assert 0 < g.beta_at(alpha=0.1) < 0.9 and 0 < g.advantage() < 1
    with pytest.raises(ValueError):
        g.epsilon_at(delta=0.0)
    with pytest.raises(ValueError):
        strong.gdp(grid_size=4)
    with pytest.raises(ValueError):
        dataclasses.replace(strong, in_scores=None).eps_delta()
    v = A.gdp_rank_error_probabilities(50, 50, 1.0)
    assert v.shape == (50,) and np.all(np.diff(v) <= 1e-12) and 0 < v[-1] < v[0] <= 0.5   # larger |loss| rank, fewer errors
    assert A.gdp_rank_error_probabilities(50, 50, 1e-6)[0] == pytest.approx(0.5, abs=1e-4)
    assert A.bernoulli_sum_lower_tail(np.full(40, 0.5), 0, 25) == 1.0
    exact = float(stats.binom.cdf(5, 40, 0.5))
    assert exact <= A.bernoulli_sum_lower_tail(np.full(40, 0.5), 0, 5) < 50 * exact            # a bound, and not a wild one
    assert A.bernoulli_sum_lower_tail(np.full(10, 0.5), 10, 0) == pytest.approx(0.5 ** 20)
    assert A.gdp_order_statistics_p_value(100, 100, 10, 0.0) == 1.0
