"""Functional DP-SFT: per-example completion-only NLL (or DFT) loss, clipped_grad → gaussian_noise → AdamW-BC.

The explicit loop of the functional API (what ``SFTTrainer`` does internally), on a tiny causal LM so it runs on CPU:

  python examples/train_sft.py --steps 20 --loss dft

Parity: examples/train_sft.py of the reference (completion masks, one privacy unit = one conversation).
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
from opaque_b200.alignment import sft
from opaque_b200.distributed import sum_gradients_, sync
from opaque_b200.dpsgd import PoissonSampler, clipped_grad, gaussian_noise
from opaque_b200.dpsgd import accounting as dacc
from opaque_b200.functional import make_functional
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
    ap.add_argument("--n", type=int, default=1024)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--sigma", type=float, default=1.0)
    ap.add_argument("--clip", type=float, default=1.0)
    ap.add_argument("--lr", type=float, default=1e-2)
    ap.add_argument("--loss", default="nll", choices=["nll", "dft"])
    ap.add_argument("--delta", type=float, default=1e-5)
    add_preset_argument(ap, "train_sft")
    a = apply_preset(ap, ap.parse_args(), "train_sft")

    g = torch.Generator().manual_seed(0)
    rows = []
    for _ in range(a.n):
        prompt = torch.randint(0, 64, (int(torch.randint(4, 9, (1,), generator=g)),), generator=g).tolist()
        completion = torch.randint(0, 64, (int(torch.randint(4, 9, (1,), generator=g)),), generator=g).tolist()
        rows.append({"input_ids": prompt + completion, "completion_mask": adata.completion_mask(len(prompt) + len(completion), len(prompt))})
    torch.manual_seed(0)
    fmodel, params = make_functional(TinyLM(), disable_autograd_tracking=True)
    loss_of = sft.dft_loss if a.loss == "dft" else sft.nll_loss

    def loss_fn(p, ex):                      # ONE record; vmapped by clipped_grad
        logits = fmodel(p, ex["input_ids"])
        return loss_of(logits, ex["labels"])            # the collator already shifted the labels

    sampler = PoissonSampler(range(a.n), a.batch / a.n, key=key(1))
    grad_fn, clip_state = clipped_grad(loss_fn, clipping_norm=a.clip, normalize_by=float(a.batch), batch_argnums=1, return_aux=True)
    noise_fn, noise_state = gaussian_noise(noise_multiplier=a.sigma, key=key(2))
    opt = optimizers.adamw(lr=a.lr, noise_bias_correction=True)          # AdamW-BC
    opt_state = opt.init(params)
    accountant = acc.Accountant()
    step_process = dacc.poisson(dacc.gaussian(a.sigma), a.batch / a.n)
    losses = []
    for step, idx in zip(range(a.steps), sampler):
        batch = adata.language_modeling_collator([rows[i] for i in idx], pad_token_id=0, completion_only=True) if idx else None
        if batch is None:
            continue
        payload = {"input_ids": batch["input_ids"], "labels": batch["labels"]}
        (grads, aux), clip_state = grad_fn(params, payload, state=clip_state)
        grads, aux = sum_gradients_(grads), sync(aux)
        noisy, noise_state = noise_fn(grads, noise_state)
        updates, opt_state = opt.update(noisy, opt_state, params=params)
        params = optimizers.apply_updates(params, updates)
        accountant |= step_process
        losses.append(float(aux.loss_values.mean()))
    print(json.dumps({"loss": a.loss, "steps": len(losses), "first_loss": losses[0], "last_loss": losses[-1],
                      "epsilon": accountant.epsilon_at(a.delta), "delta": a.delta}))


if __name__ == "__main__":
    main()
