"""DPTrainer / SFTTrainer / DPOTrainer on a tiny causal LM (CPU, reference engine), checkpoint resume."""
import json
import math
import os

import pytest
import torch
from torch import nn

from opaque_b200.transformers import DPTrainer, TrainingArguments
from opaque_b200.transformers.trainer import TrainerCallback, list_checkpoints
from opaque_b200.transformers.trl import DPOConfig, DPOTrainer, SFTConfig, SFTTrainer


class TinyLM(nn.Module):
    def __init__(self, vocab=32, hidden=8):
        super().__init__()
        self.emb = nn.Embedding(vocab, hidden)
        self.mix = nn.Linear(hidden, hidden)
        self.head = nn.Linear(hidden, vocab)

    def forward(self, ids):
        h = self.emb(ids)
        h = h + torch.tanh(self.mix(torch.cumsum(h, dim=1) / (1 + torch.arange(ids.shape[1], device=ids.device))[None, :, None]))
        return self.head(h)


def _data(n=64, T=12, vocab=32, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [{"input_ids": torch.randint(0, vocab, (T,), generator=g).tolist()} for _ in range(n)]


def _args(tmp, **kw):
    base = dict(output_dir=str(tmp), per_device_train_batch_size=8, max_steps=6, learning_rate=1e-2, logging_steps=2,
                save_steps=3, privacy_noise_multiplier=1.0, clipping_norm=1.0, optim="adamw-bc", use_cpu=True,
                lr_scheduler="constant", seed=3)
    base.update(kw)
    return TrainingArguments(**base)


def test_training_arguments_validation_and_parsing():
    a = TrainingArguments(privacy_noise_mechanism="mf_band", privacy_noise_mechanism_kwargs="bands=4", privacy_noise_multiplier=1.0)
    assert a.sampling_mode == "b_min_sep" and a.privacy_noise_mechanism_kwargs == {"bands": 4}
    assert TrainingArguments(clipping_norm='{"emb": 0.5, "fallback": 1.0}', privacy_noise_multiplier=1.0).clipping_norm == {"emb": 0.5, "fallback": 1.0}
    assert TrainingArguments(optim="adamw_torch", privacy_noise_multiplier=1.0).optim == "adamw"
    with pytest.raises(ValueError):
        TrainingArguments(privacy_noise_mechanism="mf_blt", sampling_mode="poisson")
    with pytest.raises(ValueError):
        TrainingArguments(privacy_target_epsilon=3.0, privacy_noise_multiplier=1.0)
    with pytest.raises(ValueError):
        TrainingArguments.from_hf({"fsdp": "full_shard"})
    hf = TrainingArguments.from_hf({"learning_rate": 1e-3, "max_grad_norm": 0.5, "lr_scheduler_type": "cosine"}, privacy_noise_multiplier=1.0)
    assert hf.clipping_norm == 0.5 and hf.lr_scheduler == "cosine"


def test_hf_training_arguments_conversion_manifest():
    """Every field of the installed transformers.TrainingArguments is classified; the batch collapse keeps the
    privacy-relevant batch; refused and ignored fields behave as documented."""
    import dataclasses

    import transformers

    from opaque_b200.transformers import hf_convert
    own = {f.name for f in dataclasses.fields(TrainingArguments) if not f.name.startswith("_")}
    unknown = [f.name for f in dataclasses.fields(transformers.TrainingArguments) if hf_convert.classify(f.name, own) == "unknown"]
    assert not unknown, unknown
    # (a mapping with the Hugging Face field names: instantiating transformers.TrainingArguments itself needs accelerate)
    hf = dict(output_dir="x", per_device_train_batch_size=4, gradient_accumulation_steps=8, learning_rate=3e-4, max_grad_norm=0.7,
              optim="adamw_torch_fused", lr_scheduler_type="cosine", warmup_ratio=0.1, auto_find_batch_size=True, use_cpu=True,
              report_to="none", do_train=False, fsdp="", deepspeed=None)
    a = TrainingArguments.from_hf(hf, privacy_noise_multiplier=1.0)
    assert a.per_device_train_batch_size == 32 and a.microbatch_size == 4 and a.auto_find_microbatch_size
    assert a.clipping_norm == 0.7 and a.optim == "adamw" and a.lr_scheduler == "cosine" and a.warmup_steps == 0.1
    assert a.learning_rate == 3e-4 and a.privacy_noise_multiplier == 1.0
    assert TrainingArguments.from_hf({"max_grad_norm": 0.7}, clipping_norm=2.0, privacy_noise_multiplier=1.0).clipping_norm == 2.0
    for bad in ({"fsdp": "full_shard"}, {"deepspeed": "ds.json"}, {"optim": "paged_adamw_8bit"}, {"neftune_noise_alpha": 5.0}, {"fp16": True}):
        with pytest.raises(ValueError):
            TrainingArguments.from_hf(bad, privacy_noise_multiplier=1.0)
    with pytest.warns(RuntimeWarning, match="ddp_bucket_cap_mb"):
        TrainingArguments.from_hf({"ddp_bucket_cap_mb": 50}, privacy_noise_multiplier=1.0)


def test_dp_trainer_runs_logs_and_accounts(tmp_path):
    torch.manual_seed(0)
    tr = DPTrainer(model=TinyLM(), args=_args(tmp_path), train_dataset=_data(), eval_dataset=_data(16, seed=1))
    before = tr.evaluate()["eval_loss"] if False else None
    out = tr.train()
    assert out["global_step"] == 6 and math.isfinite(out["epsilon"]) and out["epsilon"] > 0
    from opaque_b200.dpsgd import accounting as d
    assert math.isclose(out["epsilon"], (d.poisson(d.gaussian(1.0), 8 / 64) * 6).epsilon_at(tr.target_delta), rel_tol=1e-9)
    assert any("loss" in h for h in tr.state.log_history) and tr.evaluate()["eval_loss"] > 0
    ck = list_checkpoints(str(tmp_path))
    assert [os.path.basename(c) for c in ck] == ["checkpoint-3", "checkpoint-6"]
    for f in ("model.safetensors", "dp_optimizer.pt", "dp_state.pt", "accountant.json", "trainer_state.json", "rng_state.pth"):
        assert os.path.exists(os.path.join(ck[-1], f)), f
    acct = json.load(open(os.path.join(ck[-1], "accountant.json")))
    assert acct["process"]["type"] == "Repeated" and acct["process"]["count"] == 6


def test_resume_is_equivalent_to_uninterrupted_run(tmp_path):
    def run(out, resume=None, steps=6):
        torch.manual_seed(0)
        tr = DPTrainer(model=TinyLM(), args=_args(out, max_steps=steps, save_steps=3), train_dataset=_data())
        tr.train(resume_from_checkpoint=resume)
        return tr
    full = run(tmp_path / "a")
    run(tmp_path / "b")                                   # writes checkpoint-3 and checkpoint-6
    resumed = run(tmp_path / "b", resume=str(tmp_path / "b" / "checkpoint-3"))
    assert resumed.state.global_step == 6
    for (n, p), (_, q) in zip(full.model.named_parameters(), resumed.model.named_parameters()):
        assert torch.allclose(p, q, atol=1e-6), n
    assert math.isclose(full.epsilon(), resumed.epsilon(), rel_tol=1e-9)
    with pytest.raises(ValueError):
        torch.manual_seed(0)
        DPTrainer(model=TinyLM(), args=_args(tmp_path / "b", clipping_norm=2.0), train_dataset=_data()).train(
            resume_from_checkpoint=str(tmp_path / "b" / "checkpoint-3"))


def test_calibrated_noise_hits_target_epsilon(tmp_path):
    args = _args(tmp_path, privacy_noise_multiplier=None, privacy_target_epsilon=4.0, privacy_target_delta=1e-5, max_steps=20, save_steps=0)
    tr = DPTrainer(model=TinyLM(), args=args, train_dataset=_data())
    out = tr.train()
    assert out["epsilon"] <= 4.0 and out["epsilon"] > 3.9


@pytest.mark.parametrize("mech,kw", [("mf_band", {"bands": 2}), ("mf_blt", {"max_buffers": 2}), ("mf_lambda_cgd", {"lambda_": 0.5})])
def test_dpftrl_mechanisms_train(tmp_path, mech, kw):
    args = _args(tmp_path, privacy_noise_mechanism=mech, privacy_noise_mechanism_kwargs=kw, max_steps=4, save_steps=0,
                 privacy_noise_multiplier=2.0)
    out = DPTrainer(model=TinyLM(), args=args, train_dataset=_data()).train()
    assert out["global_step"] == 4 and math.isfinite(out["epsilon"])


def test_adaptive_and_per_group_clipping(tmp_path):
    out = DPTrainer(model=TinyLM(), args=_args(tmp_path, clipping_mode="adaptive", clipping_norm=0.5, save_steps=0),
                    train_dataset=_data()).train()
    assert out["global_step"] == 6
    out = DPTrainer(model=TinyLM(), args=_args(tmp_path, clipping_norm={"emb": 0.5, "fallback": 1.0}, save_steps=0, optim="sgd"),
                    train_dataset=_data()).train()
    assert out["global_step"] == 6


def test_sft_trainer_completion_only_and_dft(tmp_path):
    rows = [{"input_ids": list(range(1, 9)), "completion_mask": [0, 0, 0, 0, 1, 1, 1, 1]} for _ in range(32)]
    cfg = SFTConfig(output_dir=str(tmp_path), per_device_train_batch_size=4, max_steps=3, privacy_noise_multiplier=1.0,
                    use_cpu=True, save_steps=0, loss_type="dft", learning_rate=1e-2)
    tr = SFTTrainer(model=TinyLM(), args=cfg, train_dataset=rows)
    batch = tr.data_collator(rows[:2])
    assert (batch["labels"][0] != -100).sum() == 4
    assert tr.train()["global_step"] == 3


def test_dpo_trainer_pairs(tmp_path):
    g = torch.Generator().manual_seed(0)
    rows = [{"prompt_input_ids": torch.randint(0, 32, (4,), generator=g).tolist(),
             "chosen_input_ids": torch.randint(0, 32, (5,), generator=g).tolist(),
             "rejected_input_ids": torch.randint(0, 32, (3,), generator=g).tolist()} for _ in range(24)]
    cfg = DPOConfig(output_dir=str(tmp_path), per_device_train_batch_size=4, max_steps=3, privacy_noise_multiplier=1.0,
                    use_cpu=True, save_steps=0, learning_rate=1e-2, loss_type=["sigmoid", "sft"], loss_weights=[1.0, 0.1])
    tr = DPOTrainer(model=TinyLM(), args=cfg, train_dataset=rows)
    assert "ref_chosen_logps" in tr.train_dataset[0]
    out = tr.train()
    assert out["global_step"] == 3 and math.isfinite(tr.state.log_history[-2].get("loss", 0.0))


def test_sigterm_writes_a_just_in_time_checkpoint_and_stops(tmp_path):
    import signal

    class Kill(TrainerCallback):
        def on_step_end(self, args, state, control, **kw):
            if state.global_step == 2:
                os.kill(os.getpid(), signal.SIGTERM)
    old = signal.getsignal(signal.SIGTERM)
    try:
        tr = DPTrainer(model=TinyLM(), args=_args(tmp_path, max_steps=6, save_steps=0, enable_jit_checkpoint=True),
                       train_dataset=_data(), callbacks=[Kill()])
        tr.train()
    finally:
        signal.signal(signal.SIGTERM, old)
    assert tr.state.global_step == 2
    assert [os.path.basename(c) for c in list_checkpoints(str(tmp_path))] == ["checkpoint-2"]


def test_report_to_jsonl_writes_metrics(tmp_path):
    tr = DPTrainer(model=TinyLM(), args=_args(tmp_path, max_steps=4, save_steps=0, report_to="jsonl"), train_dataset=_data())
    tr.train()
    rows = [json.loads(l) for l in open(os.path.join(str(tmp_path), "metrics.jsonl"))]
    assert rows and any("epsilon" in r for r in rows) and all("step" in r for r in rows)
    with pytest.raises(ValueError):
        DPTrainer(model=TinyLM(), args=_args(tmp_path, report_to="carrier-pigeon"), train_dataset=_data())


def test_out_of_memory_steps_the_microbatch_down_only_when_asked(tmp_path):
    """Host-injected failure: the model raises OutOfMemoryError on its first call."""
    class FlakyOnce(TinyLM):
        fired = 0

        def forward(self, ids):
            if not FlakyOnce.fired:
                FlakyOnce.fired += 1
                raise torch.OutOfMemoryError("simulated")
            return super().forward(ids)

    tr = DPTrainer(model=FlakyOnce(), args=_args(tmp_path / "a", save_steps=0, microbatch_size=8, auto_find_microbatch_size=True),
                   train_dataset=_data())
    out = tr.train()
    assert FlakyOnce.fired == 1 and out["global_step"] == 6 and tr._microbatch == 4
    FlakyOnce.fired = 0
    tr = DPTrainer(model=FlakyOnce(), args=_args(tmp_path / "b", save_steps=0, microbatch_size=8), train_dataset=_data())
    with pytest.raises(torch.OutOfMemoryError):
        tr.train()


def test_compatibility_arguments_are_applied_or_named(tmp_path):
    """Arguments taken over from Hugging Face either act (best-model reload, throughput fields, evaluation delay,
    loss-only prediction) or are listed by ``inert_arguments`` and warned about once."""
    torch.manual_seed(0)
    data, held_out = _data(), _data(16, seed=9)
    args = _args(tmp_path, eval_strategy="steps", eval_steps=2, save_steps=0, metric_for_best_model="loss",
                 greater_is_better=False, load_best_model_at_end=True, include_tokens_per_second=True,
                 include_num_input_tokens_seen=True, dataloader_num_workers=4, hub_model_id="x/y",
                 prediction_loss_only=True, tf32=True)
    tr = DPTrainer(model=TinyLM(), args=args, train_dataset=data, eval_dataset=held_out)
    assert set(tr.inert_arguments()) == {"dataloader_num_workers", "hub_model_id"}
    with pytest.warns(RuntimeWarning, match="dataloader_num_workers=4, hub_model_id='x/y'"):
        out = tr.train()
    assert out["train_tokens_per_second"] > 0 and out["num_input_tokens_seen"] > 0
    best = tr.state.best_model_checkpoint
    assert best and os.path.isdir(best) and tr.state.best_metric is not None
    evals = [r["eval_loss"] for r in tr.state.log_history if "eval_loss" in r]
    assert math.isclose(min(evals), tr.state.best_metric, rel_tol=1e-9)
    assert math.isclose(tr.evaluate(held_out)["eval_loss"], tr.state.best_metric, rel_tol=1e-5)   # the best weights are back
    pred = tr.predict(held_out)
    assert pred.predictions is None and "test_loss" in pred.metrics
    # a setting that would change what is trained if it were honoured is refused instead of ignored
    with pytest.raises(ValueError, match="torch_compile"):
        DPTrainer(model=TinyLM(), args=_args(tmp_path / "c", torch_compile=True, save_steps=0), train_dataset=data).train()
    # label smoothing: the trainer's default loss mixes in the uniform target (reference engine)
    from opaque_b200.transformers.trainer import default_per_example_loss
    model = TinyLM()
    ex = {"input_ids": torch.tensor(data[0]["input_ids"]), "labels": torch.tensor(data[0]["input_ids"][1:] + [-100])}
    plain, smooth = default_per_example_loss(model, ex), default_per_example_loss(model, ex, 0.1)
    logp = torch.log_softmax(model(ex["input_ids"][None])[0, :-1].float(), -1)
    want = 0.9 * float(plain) + 0.1 * float(-logp.mean())
    assert math.isclose(float(smooth), want, rel_tol=1e-5)
    out = DPTrainer(model=TinyLM(), args=_args(tmp_path / "ls", label_smoothing_factor=0.1, save_steps=0), train_dataset=data).train()
    assert out["global_step"] == 6


def test_cpo_head_is_reference_free_and_matches_its_closed_form(tmp_path):
    from opaque_b200.alignment import dpo
    c, r = torch.tensor([-3.0, -1.0]), torch.tensor([-2.0, -4.0])          # summed policy log-probabilities
    nll = torch.tensor([0.7, 0.2])                                        # per-token-mean chosen NLL
    got = dpo.dpo_loss("cpo", chosen_logratio=c, rejected_logratio=r, beta=0.5, chosen_nll=nll, chosen_logp=c,
                       rejected_logp=r, cpo_alpha=2.0)
    want = -torch.nn.functional.logsigmoid(0.5 * (c - r)) + 2.0 * nll
    assert torch.allclose(got, want, atol=1e-6)
    assert torch.allclose(dpo.dpo_loss("chosen_nll", chosen_logratio=c, rejected_logratio=r, chosen_nll=nll), nll)
    g = torch.Generator().manual_seed(0)
    rows = [{"prompt_input_ids": torch.randint(0, 32, (4,), generator=g).tolist(),
             "chosen_input_ids": torch.randint(0, 32, (5,), generator=g).tolist(),
             "rejected_input_ids": torch.randint(0, 32, (3,), generator=g).tolist()} for _ in range(16)]
    cfg = DPOConfig(output_dir=str(tmp_path), per_device_train_batch_size=4, max_steps=2, privacy_noise_multiplier=1.0,
                    use_cpu=True, save_steps=0, learning_rate=1e-2, loss_type="cpo", cpo_alpha=0.5)
    tr = DPOTrainer(model=TinyLM(), args=cfg, train_dataset=rows)
    assert tr.ref_model is None and "ref_chosen_logps" not in tr.train_dataset[0]      # no reference pass at all
    assert tr.train()["global_step"] == 2


def test_memory_options_on_the_reference_engine(tmp_path):
    """Offloading is refused (torch.func has no saved-tensor hooks); checkpointing works for the framework's models
    through ``functional_checkpoint`` and gives the same run as without it; foreign models are refused."""
    from opaque_b200.models import GPT2Config, GPT2LMHeadModel, LlamaConfig, LlamaForCausalLM, MoEConfig, MoEForCausalLM
    with pytest.raises(ValueError, match="fused engine"):
        DPTrainer(model=TinyLM(), args=_args(tmp_path, save_steps=0, activation_offloading=True), train_dataset=_data()).train()
    with pytest.raises(ValueError, match="opaque_b200.models"):
        DPTrainer(model=TinyLM(), args=_args(tmp_path, save_steps=0, gradient_checkpointing=True), train_dataset=_data()).train()
    rows = _data(48, 16, 200)
    for make in (lambda: LlamaForCausalLM(LlamaConfig.tiny(), dtype=torch.float32),
                 lambda: GPT2LMHeadModel(GPT2Config.tiny(), dtype=torch.float32),
                 lambda: MoEForCausalLM(MoEConfig.tiny(), dtype=torch.float32)):
        finals = []
        for ck in (False, True):
            torch.manual_seed(0)
            model = make()
            DPTrainer(model=model, args=_args(tmp_path / f"ck{ck}", save_steps=0, max_steps=2, gradient_checkpointing=ck),
                      train_dataset=rows).train()
            finals.append(torch.cat([p.detach().reshape(-1) for p in model.parameters()]))
        assert torch.allclose(finals[0], finals[1], atol=1e-6), type(model).__name__


def test_sft_and_dpo_trainers_accept_a_moe_model_on_the_reference_engine(tmp_path):
    """The experts' dense form and ``functional_checkpoint`` carry MoE models through ``vmap(grad)``."""
    from opaque_b200.models import MoEConfig, MoEForCausalLM
    g = torch.Generator().manual_seed(0)
    pairs = [{"prompt_input_ids": torch.randint(0, 500, (4,), generator=g).tolist(),
              "chosen_input_ids": torch.randint(0, 500, (5,), generator=g).tolist(),
              "rejected_input_ids": torch.randint(0, 500, (3,), generator=g).tolist()} for _ in range(16)]
    cfg = DPOConfig(output_dir=str(tmp_path / "dpo"), per_device_train_batch_size=4, max_steps=2, privacy_noise_multiplier=1.0,
                    use_cpu=True, save_steps=0, learning_rate=1e-3)
    assert DPOTrainer(model=MoEForCausalLM(MoEConfig.tiny(), dtype=torch.float32), args=cfg, train_dataset=pairs).train()["global_step"] == 2
    rows = [{"input_ids": torch.randint(0, 500, (16,), generator=g).tolist(), "completion_mask": [0] * 6 + [1] * 10} for _ in range(32)]
    scfg = SFTConfig(output_dir=str(tmp_path / "sft"), per_device_train_batch_size=4, max_steps=2, privacy_noise_multiplier=1.0,
                     use_cpu=True, save_steps=0, gradient_checkpointing=True)
    assert SFTTrainer(model=MoEForCausalLM(MoEConfig.tiny(), dtype=torch.float32), args=scfg, train_dataset=rows).train()["global_step"] == 2


def test_truncated_poisson_cap_reaches_the_accountant(tmp_path):
    """A cap on the Poisson batch changes the mechanism: epsilon with the cap is the truncated accountant's, and is at
    least the plain-Poisson epsilon; sampling modes that cannot truncate refuse the key."""
    from opaque_b200.dpsgd import accounting as d
    torch.manual_seed(0)
    plain = DPTrainer(model=TinyLM(), args=_args(tmp_path / "p", save_steps=100), train_dataset=_data()).train()["epsilon"]
    tr = DPTrainer(model=TinyLM(), args=_args(tmp_path / "t", save_steps=100, sampling_kwargs={"truncated_batch_size": 9}),
                   train_dataset=_data())
    capped = tr.train()["epsilon"]
    want = (d.poisson(d.gaussian(1.0), 8 / 64, truncated_batch_size=9, dataset_size=64) * 6).epsilon_at(tr.target_delta)
    assert math.isclose(capped, want, rel_tol=1e-9) and capped >= plain - 1e-12
    assert tr.sampler.truncated_batch_size == 9
    alias = DPTrainer(model=TinyLM(), args=_args(tmp_path / "a", save_steps=100, sampling_kwargs={"max_batch_size": 9}),
                      train_dataset=_data()).train()["epsilon"]
    assert math.isclose(alias, capped, rel_tol=1e-12)
    with pytest.raises(ValueError, match="Poisson sampling only"):
        DPTrainer(model=TinyLM(), args=_args(tmp_path / "r", sampling_mode="random_allocation",
                                             sampling_kwargs={"truncated_batch_size": 9}), train_dataset=_data()).train()


def test_dp_state_bundle_is_a_plain_dict_with_the_reference_field_names(tmp_path):
    """`dp_state.pt` is a torch.save of a dict (no class of this package is needed to read it); a bundle pickled as the
    reference's own dataclass instance loads too."""
    import pickle
    import sys
    import types

    from opaque_b200.transformers.trainer import DP_STATE_BUNDLE_VERSION, load_runtime_checkpoint
    torch.manual_seed(0)
    tr = DPTrainer(model=TinyLM(), args=_args(tmp_path, max_steps=3, save_steps=3), train_dataset=_data())
    tr.train()
    path = os.path.join(list_checkpoints(str(tmp_path))[-1], "dp_state.pt")
    raw = torch.load(path, weights_only=False)
    assert type(raw) is dict
    for k in ("version", "clip_state", "noise_state", "sampler_state", "sample_rate", "target_delta", "noise_multiplier",
              "expected_steps_per_epoch", "expected_batch_size", "total_steps", "mechanism_kind", "mf_n_steps", "mf_min_sep",
              "mf_max_participations", "lr_scheduler", "learning_rate", "warmup_steps", "lr_scheduler_kwargs"):
        assert k in raw, k
    assert raw["version"] == DP_STATE_BUNDLE_VERSION and raw["total_steps"] == 3 and raw["mechanism_kind"] == "gaussian"
    b = load_runtime_checkpoint(path)
    assert b.max_steps == 3 and b.extras["sampling_mode"] == "poisson"
    # a reference-shaped file: an instance of a dataclass living at the reference's module path
    mod_name = "opaque.api.transformers.trainer._checkpoint"
    import dataclasses as dc
    fake = types.ModuleType(mod_name)
    cls = dc.make_dataclass("RuntimeCheckpoint", [(k, object) for k in raw if k not in ("format", "extras")])
    cls.__module__ = mod_name
    fake.RuntimeCheckpoint = cls
    parents = ["opaque", "opaque.api", "opaque.api.transformers", "opaque.api.transformers.trainer"]
    added = [m for m in parents + [mod_name] if m not in sys.modules]
    for m in parents:
        sys.modules.setdefault(m, types.ModuleType(m))
    sys.modules[mod_name] = fake
    try:
        foreign = os.path.join(str(tmp_path), "foreign_dp_state.pt")
        torch.save(cls(**{k: v for k, v in raw.items() if k not in ("format", "extras")}), foreign)
    finally:
        for m in added:
            sys.modules.pop(m, None)
    got = load_runtime_checkpoint(foreign)                    # the reference's class is NOT importable here
    assert got.noise_multiplier == raw["noise_multiplier"] and got.sampler_state == raw["sampler_state"] and got.extras == {}


def test_prediction_accumulator_offload_cadence_padding_and_lists():
    from opaque_b200.transformers.evaluation import (EvalPrediction, PredictionAccumulator, speed_metrics, with_metric_prefix)
    g = torch.Generator().manual_seed(0)
    batches = [(torch.rand(3, generator=g), torch.randn(3, T, 5, generator=g), torch.randint(0, 5, (3, T), generator=g))
               for T in (4, 6, 6, 5, 4)]
    acc = PredictionAccumulator(eval_accumulation_steps=2, include_inputs=True, include_losses=True)
    for loss, logits, labels in batches:
        acc.add(loss, logits, labels, inputs=labels)
    assert acc.offloads == 2 and acc.num_samples == 15 and len(acc.logits.pending) == 1 and len(acc.logits.host) == 2
    losses, preds, labels, inputs = acc.finalize()
    assert preds.shape == (15, 6, 5) and labels.shape == (15, 6) and losses.shape == (15,)
    assert torch.equal(preds[:3, :4], batches[0][1]) and bool((preds[:3, 4:] == -100).all())       # ragged tails hold -100
    assert torch.equal(labels[9:12, :5], batches[3][2]) and bool((labels[9:12, 5:] == -100).all())
    assert torch.equal(losses, torch.cat([b[0] for b in batches]))
    ep = acc.eval_prediction()
    p, l, i, ls = ep                                    # unpacks in the Hugging Face order
    assert p is ep.predictions and l is ep.label_ids and torch.equal(i, labels) and len(ep) == 4
    # per-batch lists instead of one tensor; a scalar (mean-reduced) loss counts once per example
    acc = PredictionAccumulator(eval_do_concat_batches=False)
    for loss, logits, labels in batches:
        acc.add(loss.mean(), logits, labels)
    losses, preds, labels, _ = acc.finalize()
    assert isinstance(preds, list) and len(preds) == 5 and preds[1].shape == (3, 6, 5) and losses.shape == (15,)
    assert torch.allclose(losses[:3], batches[0][0].mean().repeat(3))
    # loss only: nothing else is kept
    acc = PredictionAccumulator(prediction_loss_only=True)
    acc.add(batches[0][0], batches[0][1], batches[0][2])
    assert acc.finalize()[1:] == (None, None, None) and not acc.logits.pending
    with pytest.raises(ValueError):
        PredictionAccumulator(eval_accumulation_steps=0)
    assert with_metric_prefix({"accuracy": 1.0, "eval_loss": 2.0, "epsilon": 3.0}, "eval") == {"eval_accuracy": 1.0, "eval_loss": 2.0, "epsilon": 3.0}
    import time
    sm = speed_metrics("eval", time.time() - 2.0, num_samples=10, num_steps=4)
    assert 4.5 < sm["eval_samples_per_second"] < 5.5 and "eval_steps_per_second" in sm and sm["eval_runtime"] >= 2.0


def test_evaluate_and_predict_feed_compute_metrics(tmp_path):
    """``compute_metrics`` sees all predictions of the evaluation set (whatever ``eval_accumulation_steps``), with inputs and
    per-example losses when ``include_for_metrics`` asks; results come back prefixed, with speed entries."""
    torch.manual_seed(0)
    data, held_out = _data(), _data(20, seed=9)
    seen = {}

    def metrics(ep):
        preds, labels = ep.predictions, ep.label_ids      # (a 2-tuple unpacking works only without inputs / losses, as in Hugging Face)
        seen.update(shape=tuple(preds.shape), inputs=ep.inputs, losses=ep.losses)
        pred_ids = preds.argmax(-1)[:, :-1]
        mask = labels[:, :-1] != -100 if labels.shape[1] == preds.shape[1] else torch.ones_like(pred_ids, dtype=torch.bool)
        return {"accuracy": float((pred_ids == labels[:, :pred_ids.shape[1]])[mask].float().mean()), "eval_custom": torch.tensor(2.0)}

    args = _args(tmp_path, save_steps=0, max_steps=2, per_device_eval_batch_size=6, eval_accumulation_steps=2,
                 include_for_metrics=["inputs", "loss"])
    tr = DPTrainer(model=TinyLM(), args=args, train_dataset=data, eval_dataset=held_out, compute_metrics=metrics)
    assert tr.inert_arguments() == {}
    tr.train()
    out = tr.evaluate()
    assert seen["shape"] == (20, 12, 32) and seen["inputs"].shape == (20, 12) and seen["losses"].shape == (20,)
    assert 0.0 <= out["eval_accuracy"] <= 1.0 and out["eval_custom"] == 2.0 and out["eval_samples"] == 20.0
    assert math.isclose(out["eval_loss"], float(seen["losses"].mean()), rel_tol=1e-5)
    assert out["eval_runtime"] >= 0 and "eval_samples_per_second" in out and "eval_steps_per_second" in out
    pred = tr.predict(held_out)
    assert pred.predictions.shape == (20, 12, 32) and pred.num_samples == 20 and "test_accuracy" in pred.metrics and "test_loss" in pred.metrics
    res = tr.evaluation_loop(held_out, prediction_loss_only=True)
    assert res.predictions is None and res.num_batches == 4 and res.offloads >= 2
    with pytest.raises(ValueError, match="include_for_metrics"):
        _args(tmp_path, include_for_metrics=["logits"])


def test_push_to_hub_uploads_the_model_folder_without_run_state(tmp_path):
    """``push_to_hub`` through a stand-in client: repository created once, ONE folder upload whose ignore list keeps every
    checkpoint folder and run-state file (noise / sampler keys) off the Hub; the model card carries the privacy line."""
    import fnmatch
    import types
    from opaque_b200.transformers import hub

    class FakeHub:
        def __init__(self):
            self.created, self.uploads = [], []

        def create_repo(self, repo_id, token=None, private=None, exist_ok=False):
            self.created.append((repo_id, token, private, exist_ok))
            return types.SimpleNamespace(repo_id=f"someone/{repo_id}" if "/" not in repo_id else repo_id)

        def upload_folder(self, **kw):
            sent = []
            for root, _dirs, files in os.walk(kw["folder_path"]):
                for f in files:
                    rel = os.path.relpath(os.path.join(root, f), kw["folder_path"])
                    if not any(fnmatch.fnmatch(rel, pat) for pat in kw["ignore_patterns"]):
                        sent.append(rel)
            self.uploads.append({**kw, "sent": sorted(sent)})
            return types.SimpleNamespace(commit_message=kw["commit_message"])

    torch.manual_seed(0)
    args = _args(tmp_path / "my-model", max_steps=4, save_steps=2, push_to_hub=True, hub_token="tok", hub_private_repo=True,
                 hub_revision="dev")
    tr = DPTrainer(model=TinyLM(), args=args, train_dataset=_data())
    tr.hub_client = FakeHub()
    assert tr.inert_arguments() == {}                       # with push_to_hub the hub_* fields act
    tr.train()                                              # pushes at the end
    api = tr.hub_client
    assert api.created == [("my-model", "tok", True, True)] and tr.hub_repo_id == "someone/my-model"
    up = api.uploads[-1]
    assert up["repo_id"] == "someone/my-model" and up["revision"] == "dev" and up["token"] == "tok" and up["run_as_future"] is False
    assert up["commit_message"] == "End of training"
    assert os.path.isdir(tmp_path / "my-model" / "checkpoint-4")                 # checkpoints exist locally ...
    assert not any(s.startswith("checkpoint-") or s.endswith((".pt", ".pth")) for s in up["sent"]), up["sent"]   # ... and stay there
    assert "README.md" in up["sent"] and any(s.endswith((".safetensors", ".bin")) for s in up["sent"])
    card = open(tmp_path / "my-model" / "README.md").read()
    assert "privacy guarantee" in card and "my-model" in card
    tr.push_to_hub("second push", blocking=False)
    assert len(api.created) == 1 and api.uploads[-1]["run_as_future"] is True and api.uploads[-1]["commit_message"] == "second push"
    assert set(hub.NEVER_UPLOADED) >= {"checkpoint-*", "dp_state.pt", "optimizer.pt", "rng_state*.pth"}
    assert hub.resolve_repo_id(types.SimpleNamespace(hub_model_id="org/name", output_dir="x")) == "org/name"


def test_sft_config_fields_of_trl_act(tmp_path):
    """``eos_token`` / ``chat_template_path`` reach the tokenizer, ``log_completion_metrics`` adds token statistics of the
    evaluation set, ``dataset_num_proc`` is accepted and reported as inert, DPO pads pairs to a multiple."""
    from opaque_b200.transformers.trl import DPOConfig, SFTConfig, SFTTrainer

    class Tok:
        pad_token_id, eos_token, chat_template = 0, "</s>", None

        def __call__(self, text, add_special_tokens=True):
            return {"input_ids": [1 + (ord(ch) % 30) for ch in text]}
    (tmp_path / "tpl").mkdir()
    (tmp_path / "tpl" / "chat_template.jinja").write_text("{% for m in messages %}{{ m['content'] }}{% endfor %}")
    tok = Tok()
    rows = [{"prompt": "ab", "completion": "cde"} for _ in range(32)]
    args = SFTConfig(output_dir=str(tmp_path / "o"), per_device_train_batch_size=8, max_steps=1, privacy_noise_multiplier=1.0, use_cpu=True,
                     save_steps=0, eos_token="<end>", chat_template_path=str(tmp_path / "tpl"), log_completion_metrics=True,
                     dataset_num_proc=4, max_length=16)
    tr = SFTTrainer(model=TinyLM(), args=args, train_dataset=rows, eval_dataset=rows[:8], processing_class=tok)
    assert tok.eos_token == "<end>" and "messages" in tok.chat_template
    assert set(tr.inert_arguments()) == {"dataset_num_proc"}
    out = tr.evaluate()
    assert 0.0 <= out["eval_mean_token_accuracy"] <= 1.0 and out["eval_entropy"] > 0 and out["eval_loss"] > 0
    cfg = DPOConfig(privacy_noise_multiplier=1.0, pad_to_multiple_of=8, dataset_num_proc=2, model_init_kwargs={"torch_dtype": "float32"})
    assert cfg.pad_to_multiple_of == 8 and cfg.trust_remote_code is False


def test_trl_configs_convert_with_from_trl():
    import warnings
    from opaque_b200.transformers.trl import DPOConfig, SFTConfig
    base = dict(output_dir="o", per_device_train_batch_size=4, gradient_accumulation_steps=8, learning_rate=3e-5, max_steps=10, max_grad_norm=0.7)
    c = SFTConfig.from_trl({**base, "max_length": 256, "completion_only_loss": True, "dataset_text_field": "body", "loss_type": "dft"},
                           privacy_noise_multiplier=1.0)
    assert (c.per_device_train_batch_size, c.microbatch_size, c.clipping_norm, c.max_length, c.loss_type, c.dataset_text_field) == (32, 4, 0.7, 256, "dft", "body")
    for bad in ({"packing": True}, {"padding_free": True}, {"shuffle_dataset": True}, {"truncation_mode": "keep_end"}, {"pad_token": "<pad>"}):
        with pytest.raises(ValueError):
            SFTConfig.from_trl({**base, **bad}, privacy_noise_multiplier=1.0)
    with warnings.catch_warnings(record=True) as seen:
        warnings.simplefilter("always")
        d = DPOConfig.from_trl({**base, "beta": 0.3, "loss_type": ["sigmoid", "sft"], "loss_weights": [1.0, 0.1], "max_prompt_length": 64},
                               privacy_noise_multiplier=1.0)
    assert d.beta == 0.3 and d.loss_type == ["sigmoid", "sft"] and any("max_prompt_length" in str(w.message) for w in seen)


def test_trainer_conveniences_of_the_hugging_face_surface(tmp_path, capsys):
    torch.manual_seed(0)
    held_out = _data(10, seed=4)
    tr = DPTrainer(model=TinyLM(), args=_args(tmp_path, max_steps=2, save_steps=0, per_device_eval_batch_size=4), train_dataset=_data(),
                   eval_dataset=held_out)
    out = tr.train()
    assert out.global_step == 2 and out.training_loss > 0 and out.metrics["global_step"] == 2 and out["epsilon"] > 0
    loader = tr.get_eval_dataloader()
    batches = list(loader)
    assert len(loader) == len(batches) == 3 and batches[0]["input_ids"].shape[0] == 4 and batches[-1]["input_ids"].shape[0] == 2
    loss, logits, labels = tr.prediction_step(tr.model, batches[0], prediction_loss_only=False)
    assert loss > 0 and logits.shape[:2] == labels.shape and tr.prediction_step(tr.model, batches[0], True)[1] is None
    metrics = tr.evaluate()
    tr.log_metrics("eval", metrics)
    assert "***** eval metrics *****" in capsys.readouterr().out
    tr.save_metrics("eval", metrics)
    tr.save_metrics("train", dict(out))
    tr.save_state()
    path = tr.save_accountant()
    merged = json.load(open(tmp_path / "all_results.json"))
    assert "eval_loss" in merged and "train_runtime" in merged and os.path.exists(tmp_path / "eval_results.json")
    assert json.load(open(tmp_path / "trainer_state.json"))["global_step"] == 2 and os.path.exists(path)
    assert tr.callback_handler.callbacks is tr.callbacks and callable(tr.create_scheduler(10)) and tr.create_optimizer() is not None
    loss1, extra = tr.compute_per_example_loss_and_metrics(tr.model, {"input_ids": batches[0]["input_ids"][0], "labels": batches[0]["labels"][0]})
    assert extra == {} and loss1 > 0
