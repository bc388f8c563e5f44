"""Functional DP-SGD on a small MLP (runs on CPU; one process or several gloo ranks).

Default = the CPU reference configuration: fp32 784→256→10 ReLU MLP, N = 60 000 synthetic points
(x ~ N(0, 1), uniform labels), Poisson sampling q = 256/60000, C = 1.0, σ = 1.0, SGD lr 0.1, 200 steps,
ε reported at δ = 1e-5 from the PLD accountant.

  python examples/train_dpsgd.py
  python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/train_dpsgd.py --backend gloo

Parity: examples/train_dpsgd.py (loop at :1884-1915) and docs/user-guide/distributed.md:36-106 of the reference.
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
from opaque_b200 import optimizers
from opaque_b200.distributed import get_rank, get_world_size, local_shard, sum_gradients_, sync
from opaque_b200.dpsgd import PoissonSampler, clipped_grad, gaussian_noise
from opaque_b200.dpsgd import accounting as dacc
from opaque_b200.functional import make_functional
from opaque_b200.random import fold_in, key


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--n", type=int, default=60000)
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--clip", type=float, default=1.0)
    ap.add_argument("--sigma", type=float, default=1.0)
    ap.add_argument("--lr", type=float, default=0.1)
    ap.add_argument("--delta", type=float, default=1e-5)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--backend", default=None)
    ap.add_argument("--microbatch", type=int, default=None)
    add_preset_argument(ap, "train_dpsgd")
    args = apply_preset(ap, ap.parse_args(), "train_dpsgd")

    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group(args.backend or "gloo")
    rank, world = get_rank(), get_world_size()

    gen = torch.Generator().manual_seed(args.seed)
    X = torch.randn(args.n, 784, generator=gen)
    Y = torch.randint(0, 10, (args.n,), generator=gen)
    torch.manual_seed(args.seed)
    model = nn.Sequential(nn.Linear(784, 256), nn.ReLU(), nn.Linear(256, 10))
    fmodel, params = make_functional(model, disable_autograd_tracking=True)

    def loss_fn(p, x, y):
        return nn.functional.cross_entropy(fmodel(p, x.unsqueeze(0)), y.unsqueeze(0))

    per = args.n // world
    shard = local_shard(range(per * world), rank=rank, world_size=world)
    q = args.batch / args.n                                     # every record is sampled at rate q by its own rank
    sampler = PoissonSampler(shard, q, n_steps=args.steps, key=fold_in(key(args.seed), rank))
    grad_fn, clip_state = clipped_grad(loss_fn, clipping_norm=args.clip, normalize_by=float(args.batch),
                                       batch_argnums=(1, 2), return_aux=True, microbatch_size=args.microbatch)
    noise_fn, noise_state = gaussian_noise(noise_multiplier=args.sigma, key=key(args.seed + 1))   # same key on all ranks
    opt = optimizers.sgd(lr=args.lr)
    opt_state = opt.init(params)
    accountant = acc.Accountant()
    step_process = dacc.poisson(dacc.gaussian(args.sigma), q)

    t0 = time.perf_counter()
    losses = []
    for idx in sampler:
        gi = torch.as_tensor([shard[i] for i in idx], dtype=torch.long)
        accountant |= step_process
        (grads, aux), clip_state = grad_fn(params, X[gi], Y[gi], state=clip_state)
        clip_state, aux = sync(clip_state, aux)
        grads = sum_gradients_(grads)
        noisy, noise_state = noise_fn(grads, noise_state)
        noise_state = sync(noise_state)
        updates, opt_state = opt.update(noisy, opt_state, params=params)
        params = optimizers.apply_updates(params, updates)
        if aux.batch_size:
            losses.append(float(aux.loss_values.mean()))
    dt = time.perf_counter() - t0
    if rank == 0:
        print(json.dumps({"steps": args.steps, "world_size": world, "steps_per_s": args.steps / dt,
                          "final_loss": losses[-1] if losses else None, "epsilon": accountant.epsilon_at(args.delta),
                          "delta": args.delta, "param_checksum": float(sum(p.double().sum() for p in params))}))
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
