"""Functional DP-FTRL (matrix-factorisation noise) on a tiny causal LM; runs on CPU, one process or gloo ranks.

Every strategy of the library can be selected (``--strategy identity|band_mf|blt|bsr|bisr|lambda_cgd``), with the
matching participation scheme (``--sampler sequential|cyclic_poisson|b_min_sep|balls_in_bins``) and its accountant.

  python examples/train_dpftrl.py --strategy blt --buffers 4 --steps 64
  python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/train_dpftrl.py --strategy band_mf

Parity: examples/train_dpftrl.py of the reference (strategy construction, streaming noise state, amplified
accounting); docs/mechanisms of the reference for the sensitivity conventions (σ = noise_multiplier · max column
norm; the accountant divides by the sensitivity).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from _presets import add_preset_argument, apply_preset  # noqa: E402

import torch
import torch.distributed as dist
from torch import nn

import opaque_b200.accounting as acc
from opaque_b200 import dpftrl, optimizers
from opaque_b200.distributed import get_rank, get_world_size, local_shard, sum_gradients_, sync
from opaque_b200.dpftrl import accounting as facc
from opaque_b200.dpftrl.sampling import (BallsInBinsSampler, BMinSepSampler, CyclicPoissonSampler,
                                         SequentialBatchSampler)
from opaque_b200.dpsgd import clipped_grad
from opaque_b200.functional import make_functional
from opaque_b200.random import fold_in, key
from opaque_b200.types import clipped


class TinyLM(nn.Module):
    def __init__(self, vocab=64, hidden=32):
        super().__init__()
        self.emb = nn.Embedding(vocab, hidden)
        self.mix = nn.Linear(hidden, hidden)
        self.head = nn.Linear(hidden, vocab)

    def forward(self, ids):
        h = self.emb(ids)
        pos = 1 + torch.arange(ids.shape[-1], device=ids.device)
        h = h + torch.tanh(self.mix(torch.cumsum(h, dim=-2) / pos[:, None]))
        return self.head(h)


def build_strategy(a):
    if a.strategy == "identity":
        return dpftrl.identity_strategy()
    if a.strategy == "band_mf":
        return dpftrl.band_mf_strategy(bands=a.bands)
    if a.strategy == "blt":
        return dpftrl.blt_strategy(max_buffers=a.buffers)
    if a.strategy == "bsr":
        return dpftrl.bsr_strategy(bandwidth=a.bands)
    if a.strategy == "bisr":
        return dpftrl.bisr_strategy(bandwidth=a.bands)
    return dpftrl.lambda_cgd_strategy(lambda_=a.lambda_)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--strategy", default="blt", choices=["identity", "band_mf", "blt", "bsr", "bisr", "lambda_cgd"])
    ap.add_argument("--sampler", default="sequential", choices=["sequential", "cyclic_poisson", "b_min_sep", "balls_in_bins"])
    ap.add_argument("--bands", type=int, default=4)
    ap.add_argument("--buffers", type=int, default=4)
    ap.add_argument("--lambda_", type=float, default=0.5)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--n", type=int, default=2048)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--seq", type=int, default=16)
    ap.add_argument("--clip", type=float, default=1.0)
    ap.add_argument("--sigma", type=float, default=2.0)
    ap.add_argument("--lr", type=float, default=0.05)
    ap.add_argument("--delta", type=float, default=1e-5)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--backend", default=None)
    add_preset_argument(ap, "train_dpftrl")
    a = apply_preset(ap, ap.parse_args(), "train_dpftrl")

    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group(a.backend or "gloo")
    rank, world = get_rank(), get_world_size()

    gen = torch.Generator().manual_seed(a.seed)
    data = torch.randint(0, 64, (a.n, a.seq), generator=gen)
    torch.manual_seed(a.seed)
    model = TinyLM()
    fmodel, params = make_functional(model, disable_autograd_tracking=True)

    def loss_fn(p, ids):
        logits = fmodel(p, ids[:-1])
        return nn.functional.cross_entropy(logits, ids[1:])

    shard = local_shard(range(a.n))
    per_rank = max(a.batch // world, 1)
    skey = fold_in(key(a.seed + 1), rank)
    strategy = build_strategy(a)
    min_sep, max_part = 1, None
    if a.sampler == "sequential":
        sampler = SequentialBatchSampler(shard, per_rank, n_steps=a.steps)
        epochs = -(-a.steps * per_rank // len(shard))
        min_sep, max_part = len(shard) // per_rank, epochs
        process = facc.mf_gaussian(a.sigma, strategy, n_steps=a.steps, min_sep=min_sep, max_participations=max_part)
    elif a.sampler == "cyclic_poisson":
        sampler = CyclicPoissonSampler(shard, min(1.0, per_rank * a.bands / len(shard)), bands=a.bands, n_steps=a.steps, key=skey)
        min_sep = a.bands
        inner = facc.mf_gaussian(a.sigma, strategy, n_steps=a.steps, min_sep=min_sep)
        process = facc.poisson(inner, sampler.sample_rate if hasattr(sampler, "sample_rate") else min(1.0, per_rank * a.bands / len(shard)), n_steps=a.steps)
    elif a.sampler == "b_min_sep":
        sampler = BMinSepSampler(shard, a.bands, min(1.0, per_rank * a.bands / len(shard)), a.steps, key=skey)
        min_sep = a.bands
        process = facc.b_min_sep(facc.mf_gaussian(a.sigma, strategy, n_steps=a.steps, min_sep=min_sep), bands=a.bands, n_steps=a.steps)
    else:
        bins = max(len(shard) // per_rank, 1)
        sampler = BallsInBinsSampler(shard, bins, n_steps=a.steps, key=skey)
        min_sep = bins
        process = facc.balls_in_bins(facc.mf_gaussian(a.sigma, strategy, n_steps=a.steps, min_sep=bins), num_bins=bins, n_steps=a.steps)

    grad_fn, clip_state = clipped_grad(loss_fn, clipping_norm=a.clip, normalize_by=float(a.batch), batch_argnums=1,
                                       return_aux=True)
    noise_fn, noise_state = dpftrl.mf_gaussian_noise(clipped(params, 1.0), strategy, n_steps=a.steps, min_sep=min_sep,
                                                     max_participations=max_part, noise_multiplier=a.sigma, key=key(a.seed + 2))
    opt = optimizers.sgd(lr=a.lr)
    opt_state = opt.init(params)

    t0 = time.perf_counter()
    losses = []
    for step, idx in enumerate(sampler):
        batch = data[torch.as_tensor(list(idx), dtype=torch.long)]
        (grads, aux), clip_state = grad_fn(params, batch, state=clip_state)
        grads = sum_gradients_(grads)
        aux = sync(aux)
        noisy, noise_state = noise_fn(grads, noise_state)
        updates, opt_state = opt.update(noisy, opt_state, params=params)
        params = optimizers.apply_updates(params, updates)
        if aux.batch_size:
            losses.append(float(aux.loss_values.mean()))
    dt = time.perf_counter() - t0

    accountant = acc.Accountant()
    accountant |= process
    if rank == 0:
        print(json.dumps({"strategy": a.strategy, "sampler": a.sampler, "steps": a.steps, "world": world,
                          "sensitivity": strategy.sensitivity(a.steps, min_sep, max_part),
                          "epsilon": accountant.epsilon_at(a.delta), "delta": a.delta,
                          "first_loss": losses[0] if losses else None, "last_loss": losses[-1] if losses else None,
                          "steps_per_s": a.steps / dt}))
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
