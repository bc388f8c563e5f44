"""Functional DP-DPO: one privacy unit = one preference pair; any of the library's preference heads.

The explicit functional loop (what ``DPOTrainer`` does internally): reference log-probabilities are computed once from the
initial policy (for LoRA that is the adapter-free base model), each pair's loss is written for ONE pair and mapped over
the batch by ``clipped_grad``, so both responses of a pair are clipped as one gradient.

  python examples/train_dpo.py --steps 20 --loss_type sigmoid                       # toy model, synthetic pairs, CPU
  python examples/train_dpo.py --loss_type ipo --beta 0.2
  python examples/train_dpo.py --model small --lora-r 8 --dataset prefs.jsonl --loss_type simpo --target-epsilon 8

Data (``--dataset file.jsonl``): rows ``{"prompt": ..., "chosen": ..., "rejected": ...}`` (field names configurable),
tokenised with a local Hugging Face tokenizer or as bytes.  ``--loss_type`` takes one head or a comma-separated mixture
with ``--loss-weights``; reference-free heads (``simpo``, ``orpo``, ``cpo``, ``sft``) skip the reference pass.

Parity: examples/train_dpo.py of the reference (pair collation, reference log-probs, per-pair clipping, loss table).
"""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from _presets import add_preset_argument, apply_preset  # noqa: E402

import torch

import opaque_b200.accounting as acc
from opaque_b200 import optimizers
from opaque_b200.alignment import data as adata
from opaque_b200.alignment import dpo, sft
from opaque_b200.distributed import sum_gradients_, sync
from opaque_b200.dpsgd import PoissonSampler, clipped_grad, gaussian_noise
from opaque_b200.dpsgd import accounting as dacc
from opaque_b200.pytree import tree_map
from opaque_b200.random import key

import _lm_common as C  # noqa: E402


def load_pairs(a: argparse.Namespace, tok: C.Tokens | None) -> tuple[list[dict], int, int]:
    if a.dataset == "synthetic":
        g = torch.Generator().manual_seed(a.seed)
        toks = lambda n: torch.randint(1, 64, (n,), generator=g).tolist()
        rows = []
        for _ in range(a.n + a.eval_n):
            prompt = toks(6)
            chosen = [(t + 1) % 63 + 1 for t in prompt]                 # "chosen" follows a rule, "rejected" is noise
            rows.append({"prompt_input_ids": prompt, "chosen_input_ids": chosen, "rejected_input_ids": toks(5)})
        return rows, 64, 0
    rows = []
    half = max(a.max_seq_len // 2, 1)
    for r in C.read_jsonl(a.dataset, a.n + a.eval_n):
        p, c, j = (tok.encode(str(r[f])) for f in (a.prompt_field, a.chosen_field, a.rejected_field))
        p, c, j = p[-half:], c[:half], j[:half]                        # keep the END of a long prompt, the start of responses
        if p and c and j:
            rows.append({"prompt_input_ids": p, "chosen_input_ids": c, "rejected_input_ids": j})
    if len(rows) < a.n + a.eval_n:
        C.fail(f"{a.dataset}: {len(rows)} usable pairs, need --n + --eval-n = {a.n + a.eval_n}")
    return rows, tok.vocab, tok.pad


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    add_preset_argument(ap, "train_dpo")
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--n", type=int, default=512, help="training pairs")
    ap.add_argument("--eval-n", type=int, default=0, help="held-out pairs: reward accuracy and margin at the end")
    ap.add_argument("--batch", type=int, default=16, help="expected number of pairs per step (Poisson)")
    g = ap.add_argument_group("preference loss")
    g.add_argument("--loss_type", "--loss-type", dest="loss_type", default="sigmoid", help=f"one of {', '.join(dpo.ALL_LOSS_TYPES)}; or a comma-separated mixture")
    g.add_argument("--loss-weights", default=None, help="comma-separated weights of a mixture")
    g.add_argument("--beta", type=float, default=0.1)
    g.add_argument("--label-smoothing", type=float, default=0.0)
    g.add_argument("--simpo-gamma", type=float, default=0.5)
    g.add_argument("--cpo-alpha", type=float, default=1.0)
    g = ap.add_argument_group("data")
    g.add_argument("--dataset", default="synthetic", help="synthetic | file.jsonl")
    g.add_argument("--prompt-field", default="prompt")
    g.add_argument("--chosen-field", default="chosen")
    g.add_argument("--rejected-field", default="rejected")
    C.add_model_arguments(ap)
    C.add_optimizer_arguments(ap, lr=1e-2)
    C.add_privacy_arguments(ap)
    a = apply_preset(ap, ap.parse_args(), "train_dpo")
    heads = a.loss_type.split(",")
    unknown = [h for h in heads if h not in dpo.ALL_LOSS_TYPES]
    if unknown:
        ap.error(f"unknown loss type(s) {unknown}; known: {', '.join(dpo.ALL_LOSS_TYPES)}")
    weights = [float(w) for w in a.loss_weights.split(",")] if a.loss_weights else None
    loss_type = heads if len(heads) > 1 else heads[0]
    needs_reference = any(h not in dpo.REFERENCE_FREE for h in heads)

    device = torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
    tok = C.Tokens(a.tokenizer) if a.dataset != "synthetic" else None
    rows, vocab, pad = load_pairs(a, tok)
    train, held_out = rows[:a.n], rows[a.n:a.n + a.eval_n]
    model = C.build_model(a, vocab, device)
    logits_of, params, write_back = C.functional(model)
    ref_params = tree_map(lambda v: v.clone(), params)        # the initial policy; with LoRA (B = 0) that is the base model

    def seq_stats(p, ids, labels):
        """Summed and per-token-mean log-probability of the response tokens of ONE sequence."""
        logits = logits_of(p, ids[None])[0].float()
        return sft.sequence_logp(logits, labels), sft.sequence_logp(logits, labels, average=True)

    def loss_fn(p, ex):                      # ONE pair; clipped_grad maps it over the batch
        c_sum, c_avg = seq_stats(p, ex["chosen_input_ids"], ex["chosen_labels"])
        r_sum, r_avg = seq_stats(p, ex["rejected_input_ids"], ex["rejected_labels"])
        return dpo.dpo_loss(loss_type, chosen_logratio=c_sum - ex["ref_chosen_logps"], rejected_logratio=r_sum - ex["ref_rejected_logps"],
                            beta=a.beta, label_smoothing=a.label_smoothing, loss_weights=weights, chosen_nll=-c_avg,
                            chosen_avg_logp=c_avg, rejected_avg_logp=r_avg, chosen_logp=c_sum, rejected_logp=r_sum,
                            simpo_gamma=a.simpo_gamma, cpo_alpha=a.cpo_alpha)

    def collate(batch_rows):
        b = adata.preference_collator(batch_rows, pad_token_id=pad)
        b = {k: v.to(device) for k, v in b.items() if not k.endswith("attention_mask")}
        n = b["chosen_input_ids"].shape[0]
        if needs_reference:
            with torch.no_grad(), C.plain_ops():
                b["ref_chosen_logps"] = torch.stack([seq_stats(ref_params, i, l)[0] for i, l in zip(b["chosen_input_ids"], b["chosen_labels"])])
                b["ref_rejected_logps"] = torch.stack([seq_stats(ref_params, i, l)[0] for i, l in zip(b["rejected_input_ids"], b["rejected_labels"])])
        else:
            b["ref_chosen_logps"] = b["ref_rejected_logps"] = torch.zeros(n, device=device)
        return b

    q = a.batch / a.n
    sigma = C.noise_multiplier(a, lambda s: dacc.poisson(dacc.gaussian(s), q) * a.steps)
    sampler = PoissonSampler(range(a.n), q, n_steps=a.steps, key=key(a.seed + 1))
    grad_fn, clip_state = clipped_grad(loss_fn, clipping_norm=a.clip, normalize_by=float(a.batch), batch_argnums=1, return_aux=True,
                                       microbatch_size=a.microbatch)
    noise_fn, noise_state = gaussian_noise(noise_multiplier=sigma, key=key(a.seed + 2))
    schedule, opt = C.schedule_and_optimizer(a, a.steps)
    opt_state = opt.init(params)
    accountant = acc.Accountant()
    step_process = dacc.poisson(dacc.gaussian(sigma), q)
    losses = []
    for step, idx in zip(range(a.steps), sampler):
        accountant |= step_process
        if not idx:
            continue
        with C.plain_ops():
            (grads, aux), clip_state = grad_fn(params, collate([train[i] for i in idx]), state=clip_state)
        grads, aux = sum_gradients_(grads), sync(aux)
        noisy, noise_state = noise_fn(grads, noise_state)
        updates, opt_state = opt.update(noisy, opt_state, params=params)
        params = optimizers.apply_updates(params, updates)
        losses.append(float(aux.loss_values.mean()))
    write_back(params)
    summary = {"loss_type": a.loss_type, "steps": len(losses), "first_loss": losses[0], "last_loss": losses[-1], "noise_multiplier": sigma,
               "epsilon": accountant.epsilon_at(a.delta), "delta": a.delta}
    if held_out:
        with torch.no_grad(), C.plain_ops():
            b = collate(held_out)
            c = torch.stack([seq_stats(params, i, l)[0] for i, l in zip(b["chosen_input_ids"], b["chosen_labels"])]) - b["ref_chosen_logps"]
            r = torch.stack([seq_stats(params, i, l)[0] for i, l in zip(b["rejected_input_ids"], b["rejected_labels"])]) - b["ref_rejected_logps"]
        summary["eval_reward_accuracy"] = float((c > r).float().mean())
        summary["eval_reward_margin"] = float(a.beta * (c - r).mean())
    C.emit(summary)


if __name__ == "__main__":
    main()
