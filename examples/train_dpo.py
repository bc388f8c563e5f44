"""Functional DP-DPO: one privacy unit = one preference pair; any of the library's preference heads.

Reference log-probabilities come from the frozen initial parameters.  The explicit functional loop on a tiny LM:

  python examples/train_dpo.py --steps 20 --loss_type sigmoid
  python examples/train_dpo.py --loss_type ipo --beta 0.2

Parity: examples/train_dpo.py of the reference (pair collation, reference log-probs, per-pair clipping).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from _presets import add_preset_argument, apply_preset  # noqa: E402

import torch
from torch import nn

import opaque_b200.accounting as acc
from opaque_b200 import optimizers
from opaque_b200.alignment import data as adata
from opaque_b200.alignment import dpo, sft
from opaque_b200.distributed import sum_gradients_, sync
from opaque_b200.dpsgd import PoissonSampler, clipped_grad, gaussian_noise
from opaque_b200.dpsgd import accounting as dacc
from opaque_b200.functional import make_functional
from opaque_b200.pytree import tree_map
from opaque_b200.random import key


class TinyLM(nn.Module):
    def __init__(self, vocab=64, hidden=32):
        super().__init__()
        self.emb = nn.Embedding(vocab, hidden)
        self.mix = nn.Linear(hidden, hidden)
        self.head = nn.Linear(hidden, vocab)

    def forward(self, ids):
        h = self.emb(ids)
        pos = 1 + torch.arange(ids.shape[-1], device=ids.device)
        return self.head(h + torch.tanh(self.mix(torch.cumsum(h, dim=-2) / pos[:, None])))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--n", type=int, default=512)
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--sigma", type=float, default=1.0)
    ap.add_argument("--clip", type=float, default=1.0)
    ap.add_argument("--beta", type=float, default=0.1)
    ap.add_argument("--loss_type", default="sigmoid")
    ap.add_argument("--lr", type=float, default=1e-2)
    ap.add_argument("--delta", type=float, default=1e-5)
    add_preset_argument(ap, "train_dpo")
    a = apply_preset(ap, ap.parse_args(), "train_dpo")

    g = torch.Generator().manual_seed(0)
    toks = lambda n: torch.randint(0, 64, (n,), generator=g).tolist()
    rows = [{"prompt_input_ids": toks(6), "chosen_input_ids": toks(6), "rejected_input_ids": toks(5)} for _ in range(a.n)]
    torch.manual_seed(0)
    fmodel, params = make_functional(TinyLM(), disable_autograd_tracking=True)
    ref_params = tree_map(lambda v: v.clone(), params)

    def logp(p, ids, labels):
        return sft.sequence_logp(fmodel(p, ids), labels)

    def loss_fn(p, ex):                      # ONE pair; vmapped by clipped_grad
        c = logp(p, ex["chosen_input_ids"], ex["chosen_labels"]) - ex["ref_chosen_logps"]
        r = logp(p, ex["rejected_input_ids"], ex["rejected_labels"]) - ex["ref_rejected_logps"]
        return dpo.dpo_loss(a.loss_type, chosen_logratio=c, rejected_logratio=r, beta=a.beta)

    sampler = PoissonSampler(range(a.n), a.batch / a.n, key=key(1))
    grad_fn, clip_state = clipped_grad(loss_fn, clipping_norm=a.clip, normalize_by=float(a.batch), batch_argnums=1, return_aux=True)
    noise_fn, noise_state = gaussian_noise(noise_multiplier=a.sigma, key=key(2))
    opt = optimizers.adamw(lr=a.lr, noise_bias_correction=True)
    opt_state = opt.init(params)
    accountant = acc.Accountant()
    step_process = dacc.poisson(dacc.gaussian(a.sigma), a.batch / a.n)
    losses, margins = [], []
    for step, idx in zip(range(a.steps), sampler):
        if not idx:
            continue
        batch = adata.preference_collator([rows[i] for i in idx], pad_token_id=0)
        with torch.no_grad():
            batch["ref_chosen_logps"] = torch.stack([logp(ref_params, i, l) for i, l in zip(batch["chosen_input_ids"], batch["chosen_labels"])])
            batch["ref_rejected_logps"] = torch.stack([logp(ref_params, i, l) for i, l in zip(batch["rejected_input_ids"], batch["rejected_labels"])])
        payload = {k: v for k, v in batch.items() if not k.endswith("attention_mask")}
        (grads, aux), clip_state = grad_fn(params, payload, state=clip_state)
        grads, aux = sum_gradients_(grads), sync(aux)
        noisy, noise_state = noise_fn(grads, noise_state)
        updates, opt_state = opt.update(noisy, opt_state, params=params)
        params = optimizers.apply_updates(params, updates)
        accountant |= step_process
        losses.append(float(aux.loss_values.mean()))
    print(json.dumps({"loss_type": a.loss_type, "steps": len(losses), "first_loss": losses[0], "last_loss": losses[-1],
                      "epsilon": accountant.epsilon_at(a.delta), "delta": a.delta}))


if __name__ == "__main__":
    main()
