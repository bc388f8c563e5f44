"""DPTrainer on the fused engine (B200): steps, metrics, checkpoint and resume, graph replay, DP-FTRL mechanism."""
import math
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rows(n=96, T=64, vocab=256, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [{"input_ids": torch.randint(0, vocab, (T,), generator=g).tolist()} for _ in range(n)]


def _model(lora=True):
    from opaque_b200.models import LlamaConfig, LlamaForCausalLM
    torch.manual_seed(0)
    m = LlamaForCausalLM(LlamaConfig.tiny(), device=torch.device("cuda", 0))
    if lora:
        m.add_lora(16, 32.0)
    return m


def _args(tmp, **kw):
    from opaque_b200.transformers import TrainingArguments
    base = dict(output_dir=str(tmp), per_device_train_batch_size=8, max_steps=4, learning_rate=1e-3, logging_steps=2, save_steps=2,
                privacy_noise_multiplier=1.0, clipping_norm=1.0, optim="adamw-bc", lr_scheduler="constant", seed=3, dp_engine="fused",
                bf16=True)
    base.update(kw)
    return TrainingArguments(**base)


def test_fused_trainer_steps_checkpoints_and_resumes(tmp_path):
    from opaque_b200.transformers import DPTrainer
    from opaque_b200.transformers.trainer import list_checkpoints
    tr = DPTrainer(model=_model(), args=_args(tmp_path / "a"), train_dataset=_rows())
    out = tr.train()
    assert tr.engine_kind == "fused" and out["global_step"] == 4 and math.isfinite(out["epsilon"]) and out["epsilon"] > 0
    ck = list_checkpoints(str(tmp_path / "a"))
    assert [os.path.basename(c) for c in ck] == ["checkpoint-2", "checkpoint-4"]
    for f in ("adapter_model.safetensors", "dp_optimizer.pt", "dp_state.pt", "accountant.json", "trainer_state.json"):   # LoRA: adapter only
        assert os.path.exists(os.path.join(ck[-1], f)), f
    full = {n: p.detach().float().clone() for n, p in tr.model.named_parameters() if p.requires_grad}
    resumed = DPTrainer(model=_model(), args=_args(tmp_path / "a"), train_dataset=_rows())
    resumed.train(resume_from_checkpoint=ck[0])
    assert resumed.state.global_step == 4 and math.isclose(resumed.epsilon(), tr.epsilon(), rel_tol=1e-9)
    for n, p in resumed.model.named_parameters():
        if p.requires_grad:          # same noise stream and data order; fp32 atomics may reorder sums
            assert float((p.detach().float() - full[n]).abs().max()) < 5e-2 * float(full[n].abs().max()) + 1e-3, n


@pytest.mark.parametrize("kw", [dict(dp_cuda_graph=True), dict(privacy_noise_mechanism="mf_blt", privacy_noise_mechanism_kwargs={"max_buffers": 2},
                                                              sampling_mode="sequential"),
                                dict(clipping_mode="adaptive", clipping_norm=0.5), dict(clipping_mode="auto"),
                                dict(privacy_noise_mechanism="mf_band"), dict(privacy_noise_mechanism="mf_bsr"),
                                dict(privacy_noise_mechanism="mf_bisr"), dict(privacy_noise_mechanism="mf_lambda_cgd"),
                                dict(privacy_noise_mechanism="mf_identity"),
                                dict(optim="sgd", optim_args={"momentum": 0.9}), dict(optim="sgd", optim_args={"momentum": 0.9, "nesterov": True}),
                                dict(optim="lion", learning_rate=1e-4), dict(optim="adam"), dict(optim="adamw")])
def test_fused_trainer_options(tmp_path, kw):
    from opaque_b200.transformers import DPTrainer
    tr = DPTrainer(model=_model(lora=kw.get("privacy_noise_mechanism") is None), args=_args(tmp_path, save_steps=0, **kw), train_dataset=_rows())
    out = tr.train()
    assert tr.engine_kind == "fused" and out["global_step"] == 4 and math.isfinite(tr.state.log_history[-2]["loss"])


def test_fused_trainer_evaluates_and_predicts_on_the_gpu(tmp_path):
    """Evaluation on the device: per-example losses from the fused head, predictions offloaded every two batches,
    ``compute_metrics`` on the gathered tensors."""
    from opaque_b200.transformers import DPTrainer
    seen = {}

    def metrics(ep):
        seen["shape"] = tuple(ep.predictions.shape)
        keep = ep.label_ids != -100
        return {"labelled": int(keep.sum()), "mean_loss": float(ep.losses.mean())}

    held_out = _rows(20, seed=5)
    args = _args(tmp_path, save_steps=0, max_steps=2, per_device_eval_batch_size=6, eval_accumulation_steps=2, include_for_metrics=["loss"])
    tr = DPTrainer(model=_model(), args=args, train_dataset=_rows(), eval_dataset=held_out, compute_metrics=metrics)
    tr.train()
    out = tr.evaluate()
    assert seen["shape"][:2] == (20, 64) and out["eval_samples"] == 20.0 and out["eval_labelled"] == 20 * 63
    assert math.isfinite(out["eval_loss"]) and abs(out["eval_loss"] - out["eval_mean_loss"]) < 1e-3
    pred = tr.predict(held_out[:7])
    assert pred.num_samples == 7 and pred.predictions.shape[0] == 7 and "test_loss" in pred.metrics
    tr.compute_metrics = None
    assert tr.evaluate()["eval_loss"] == pytest.approx(out["eval_loss"], rel=1e-3)        # loss-only path


def test_fused_trainer_logs_sync_times_when_asked(tmp_path):
    from opaque_b200.transformers import DPTrainer
    tr = DPTrainer(model=_model(), args=_args(tmp_path, save_steps=0, include_sync_metrics=True, logging_steps=1), train_dataset=_rows())
    tr.train()
    rows = [r for r in tr.state.log_history if "sync/shard_step_ms" in r]
    assert rows and all(r["sync/shard_step_ms"] > 0 and r["sync/exposed_wait_ms"] >= 0 for r in rows)


def test_fused_trainer_steps_down_after_a_simulated_oom(tmp_path):
    """The failure is injected on the host: the loss raises OutOfMemoryError once for a microbatch of more than 4 rows."""
    from opaque_b200.transformers import DPTrainer
    model = _model()
    inner, fired = model.per_example_loss, []

    def flaky(input_ids, labels, **kw):
        if input_ids.shape[0] > 4 and not fired:
            fired.append(1)
            raise torch.OutOfMemoryError("simulated")
        return inner(input_ids, labels, **kw)
    model.per_example_loss = flaky
    tr = DPTrainer(model=model, args=_args(tmp_path, save_steps=0, per_device_train_batch_size=16, microbatch_size=8,
                                       auto_find_microbatch_size=True), train_dataset=_rows())
    out = tr.train()
    assert fired and out["global_step"] == 4 and tr._fused.microbatch_size == 4
    assert float(tr._fused.space.grad.local.abs().max()) == 0.0          # consumed by the last step, nothing left over


def _pairs(n=48, vocab=256, seed=0):
    g = torch.Generator().manual_seed(seed)
    rows = []
    for _ in range(n):
        lp, lc, lr = (int(torch.randint(8, 20, (1,), generator=g)) for _ in range(3))
        rows.append({"prompt_input_ids": torch.randint(0, vocab, (lp,), generator=g).tolist(),
                     "chosen_input_ids": torch.randint(0, vocab, (lc,), generator=g).tolist(),
                     "rejected_input_ids": torch.randint(0, vocab, (lr,), generator=g).tolist()})
    return rows


@pytest.mark.parametrize("loss_type", ["sigmoid", "ipo", "simpo", "orpo"])
def test_dpo_runs_on_the_fused_engine_and_matches_the_reference_engine(tmp_path, loss_type):
    """One preference pair = one privacy unit on the fused engine ([B, 2, T] batches, rows of a pair clipped together);
    first-step loss and mean per-pair gradient norm equal those of the vmap engine on the same batch."""
    from opaque_b200.transformers.trl import DPOConfig, DPOTrainer

    def run(engine, out):
        torch.manual_seed(0)
        model = _model()
        with torch.no_grad():                       # LoRA B starts at zero: move off the saddle so both factors get gradients
            for n, p in model.named_parameters():
                if n.endswith("lora_B"):
                    p.copy_(torch.randn_like(p) * 0.05)
        args = DPOConfig(output_dir=str(out), per_device_train_batch_size=8, max_steps=2, learning_rate=1e-4, logging_steps=1,
                         save_steps=0, privacy_noise_multiplier=1.0, clipping_norm=1.0, optim="adamw-bc", lr_scheduler="constant",
                         seed=3, dp_engine=engine, bf16=True, loss_type=loss_type, beta=0.5, microbatch_size=4)
        tr = DPOTrainer(model=model, args=args, train_dataset=_pairs())
        tr.train()
        first = next(h for h in tr.state.log_history if "loss" in h)
        return tr, first
    fused, f = run("fused", tmp_path / "f")
    ref, r = run("reference", tmp_path / "r")
    assert fused.engine_kind == "fused" and ref.engine_kind == "reference"
    assert fused.ref_model is None                    # adapter-disabled policy, no copy of the weights
    assert math.isfinite(f["loss"]) and abs(f["loss"] - r["loss"]) < 3e-2 * max(1.0, abs(r["loss"]))
    assert abs(f["grad_norm"] - r["grad_norm"]) < 8e-2 * max(r["grad_norm"], 1e-3)
    if loss_type not in ("simpo", "orpo"):           # reference-based heads: the cached table exists and is reused
        files = [x for x in os.listdir(tmp_path / "f") if x.startswith("ref_logps_train_")]
        assert len(files) == 1
