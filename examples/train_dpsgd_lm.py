"""Functional DP-SGD fine-tuning of a causal language model: the explicit loop, with every knob on the command line.

What the script does, in the order of a step: draw a batch (Poisson, fixed-size without replacement, or random
allocation) → per-example gradients, clipped (fixed bound, automatic ``R/(‖g‖+γ)``, adaptive quantile, per-group bounds)
→ summed over ranks → Gaussian noise → optimizer (SGD, AdamW, AdamW with noise bias correction, Lion) under a warm-up +
decay schedule → accountant.  Around the loop: calibration of the noise multiplier to a target (ε, δ), periodic
evaluation on held-out text, JSON-lines logging, an optional one-run privacy audit with canaries, and — on a B200 —
``--engine fused``, which runs the same step on the CUDA kernels (ghost norms, clip-weighted gradients, fused noise +
optimizer).

Data: ``--dataset synthetic`` (default; a small Markov source, so the loss can go down), a ``.jsonl`` file with
``--text-field``, or a ``.txt`` file with one document per line.  Tokens: a local Hugging Face tokenizer directory
(``--tokenizer``) or bytes.  Model: a built-in random-init Llama configuration (``--model tiny|small|base``) or a local
Hugging Face checkpoint directory, converted with ``patches.apply_model_patches``; ``--lora-r`` freezes it and trains
adapters.

  python examples/train_dpsgd_lm.py --preset smoke
  python examples/train_dpsgd_lm.py --model small --lora-r 8 --target-epsilon 8 --steps 200 --eval-steps 50
  python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/train_dpsgd_lm.py --preset smoke

Parity: examples/train_dpsgd.py of the reference (argument groups :357-819, presets :845-900, training loop :1884-1915,
audit section :776-800).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from _presets import add_preset_argument, apply_preset  # noqa: E402

import torch
import torch.distributed as dist

import opaque_b200.accounting as acc
from opaque_b200 import auditing, optimizers, scheduling
from opaque_b200.distributed import get_rank, get_world_size, reduce_scalar, sum_gradients_, sync
from opaque_b200.dpsgd import (KOutOfTSampler, PoissonSampler, RandomAllocationSampler, adaptive_clipped_grad, auto_clipped_grad,
                               clipped_grad, gaussian_noise, per_group)
from opaque_b200.dpsgd import accounting as dacc
from opaque_b200.functional import make_functional
from opaque_b200.models import LlamaConfig, LlamaForCausalLM
from opaque_b200.random import fold_in, key

MODELS = {      # random-init configurations (no download); vocabulary is set from the tokenizer
    "tiny": dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2),
    "small": dict(hidden_size=256, intermediate_size=704, num_hidden_layers=4, num_attention_heads=8, num_key_value_heads=4),
    "base": dict(hidden_size=768, intermediate_size=2048, num_hidden_layers=12, num_attention_heads=12, num_key_value_heads=4),
}


def parse_args() -> argparse.Namespace:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    add_preset_argument(ap, "train_dpsgd_lm")
    g = ap.add_argument_group("model")
    g.add_argument("--model", default="tiny", help="tiny | small | base (random init) or a local Hugging Face checkpoint directory")
    g.add_argument("--dtype", default="float32", choices=["float32", "bfloat16"])
    g.add_argument("--engine", default="reference", choices=["reference", "fused"],
                   help="reference: vmap per-example gradients (any device); fused: the CUDA kernels (B200)")
    g.add_argument("--gradient-checkpointing", action="store_true")
    g = ap.add_argument_group("LoRA")
    g.add_argument("--lora-r", type=int, default=0, help="0 trains the whole model")
    g.add_argument("--lora-alpha", type=float, default=None, help="default 2 r")
    g.add_argument("--lora-modules", default="q_proj,k_proj,v_proj,o_proj")
    g = ap.add_argument_group("data")
    g.add_argument("--dataset", default="synthetic", help="synthetic | file.jsonl | file.txt")
    g.add_argument("--text-field", default="text")
    g.add_argument("--tokenizer", default=None, help="local Hugging Face tokenizer directory (default: bytes)")
    g.add_argument("--num-train-samples", type=int, default=2048)
    g.add_argument("--num-eval-samples", type=int, default=128)
    g.add_argument("--max-seq-len", type=int, default=64)
    g = ap.add_argument_group("training")
    g.add_argument("--batch-size", type=int, default=64, help="expected (Poisson) or exact (fixed) GLOBAL batch size")
    g.add_argument("--eval-batch-size", type=int, default=32)
    g.add_argument("--microbatch-size", type=int, default=None)
    g.add_argument("--steps", type=int, default=None)
    g.add_argument("--num-epochs", type=float, default=1.0, help="used when --steps is not given")
    g.add_argument("--learning-rate", type=float, default=2e-3)
    g.add_argument("--lr-schedule", default="cosine", choices=["constant", "cosine", "linear"])
    g.add_argument("--lr-min-ratio", type=float, default=0.1)
    g.add_argument("--lr-warmup-steps", type=int, default=0)
    g.add_argument("--optimizer", default="adamw-bc", choices=["sgd", "adamw", "adamw-bc", "lion"])
    g.add_argument("--weight-decay", type=float, default=0.0)
    g.add_argument("--log-steps", type=int, default=10)
    g.add_argument("--eval-steps", type=int, default=0, help="0: evaluate only at the end")
    g.add_argument("--stop-at-step", type=int, default=None, help="leave the loop early (the schedule keeps its full length)")
    g.add_argument("--seed", type=int, default=42)
    g.add_argument("--output", default=None, help="JSON-lines log file")
    g = ap.add_argument_group("differential privacy")
    g.add_argument("--sampler", default="poisson", choices=["poisson", "fixed", "random-allocation"])
    g.add_argument("--truncated-batch-size", type=int, default=None, help="Poisson only: cap on the realised batch")
    g.add_argument("--clipping-mode", default="fixed", choices=["fixed", "auto", "adaptive"])
    g.add_argument("--clipping-norm", type=float, default=1.0)
    g.add_argument("--auto-clipping-gamma", type=float, default=0.01)
    g.add_argument("--target-clipping-rate", type=float, default=0.5, help="adaptive: quantile of norms the bound tracks")
    g.add_argument("--clipping-norm-max", type=float, default=100.0)
    g.add_argument("--per-group-clipping", default=None,
                   help="JSON {name pattern: bound}, e.g. '{\"embed\": 0.5, \"fallback\": 1.0}' (fixed mode)")
    g.add_argument("--noise-multiplier", type=float, default=None)
    g.add_argument("--target-epsilon", type=float, default=None)
    g.add_argument("--target-delta", type=float, default=1e-5)
    g.add_argument("--calibration-min", type=float, default=0.3)
    g.add_argument("--calibration-max", type=float, default=50.0)
    g.add_argument("--calibration-tolerance", type=float, default=1e-3)
    g = ap.add_argument_group("audit")
    g.add_argument("--audit", action="store_true", help="one-run audit: random canaries, each included with probability 1/2")
    g.add_argument("--audit-canaries", type=int, default=64)
    g = ap.add_argument_group("tracking")
    g.add_argument("--wandb-project", default=None, help="log to Weights & Biases when the package is installed")
    args = apply_preset(ap, ap.parse_args(), "train_dpsgd_lm")
    given = {name for name in ("--noise-multiplier", "--target-epsilon") if any(a.split("=")[0] == name for a in sys.argv[1:])}
    if args.noise_multiplier is not None and args.target_epsilon is not None and len(given) == 1:
        # one came from the preset, the other from the command line: the command line wins
        if "--target-epsilon" in given:
            args.noise_multiplier = None
        else:
            args.target_epsilon = None
    if (args.noise_multiplier is None) == (args.target_epsilon is None):
        ap.error("give exactly one of --noise-multiplier and --target-epsilon")
    return args


# ------------------------------------------------------------------------------------------------ data

def load_texts(args: argparse.Namespace) -> list[str] | None:
    if args.dataset == "synthetic":
        return None
    need = args.num_train_samples + args.num_eval_samples
    rows: list[str] = []
    with open(args.dataset, encoding="utf-8") as f:
        for line in f:
            line = line.strip()
            if not line:
                continue
            rows.append(str(json.loads(line)[args.text_field]) if args.dataset.endswith(".jsonl") else line)
            if len(rows) >= need:
                break
    if len(rows) < need:
        raise SystemExit(f"{args.dataset} holds {len(rows)} documents; --num-train-samples + --num-eval-samples = {need}")
    return rows


def tokenize(args: argparse.Namespace, texts: list[str] | None) -> tuple[list[list[int]], int]:
    """Token-id lists (each at most ``max_seq_len`` long, at least 2) and the vocabulary size."""
    T = args.max_seq_len
    if texts is None:
        # order-1 Markov chain over 61 symbols with a sparse transition table: learnable, so the loss moves
        gen = torch.Generator().manual_seed(args.seed)
        V = 64
        nxt = torch.randint(3, V, (V, 4), generator=gen)
        n = args.num_train_samples + args.num_eval_samples
        lens = torch.randint(max(T // 2, 2), T + 1, (n,), generator=gen)
        out = []
        for i in range(n):
            seq = [int(torch.randint(3, V, (1,), generator=gen))]
            pick = torch.randint(0, 4, (int(lens[i]) - 1,), generator=gen)
            for j in pick.tolist():
                seq.append(int(nxt[seq[-1], j]))
            out.append(seq)
        return out, V
    if args.tokenizer:
        from transformers import AutoTokenizer
        tok = AutoTokenizer.from_pretrained(args.tokenizer, local_files_only=True)
        ids = [tok(t, truncation=True, max_length=T)["input_ids"] for t in texts]
        return [x if len(x) >= 2 else x + [tok.eos_token_id or 0] * (2 - len(x)) for x in ids], len(tok)
    ids = [list(t.encode("utf-8"))[:T] for t in texts]                      # bytes; 256 = padding
    return [x if len(x) >= 2 else x + [10] * (2 - len(x)) for x in ids], 257


def collate(rows: list[list[int]], pad: int) -> dict[str, torch.Tensor]:
    """Right-padded ids and next-token labels (−100 on padding and on the last position)."""
    T = max(len(r) for r in rows)
    ids = torch.full((len(rows), T), pad, dtype=torch.long)
    labels = torch.full((len(rows), T), -100, dtype=torch.long)
    for i, r in enumerate(rows):
        ids[i, :len(r)] = torch.tensor(r)
        labels[i, :len(r) - 1] = torch.tensor(r[1:])
    return {"input_ids": ids, "labels": labels}


# ------------------------------------------------------------------------------------------------ model

def build_model(args: argparse.Namespace, vocab: int, device: torch.device) -> LlamaForCausalLM:
    dtype = getattr(torch, args.dtype)
    if args.model in MODELS:
        cfg = LlamaConfig(vocab_size=(vocab + 63) // 64 * 64, max_position_embeddings=max(args.max_seq_len, 64), **MODELS[args.model])
        torch.manual_seed(args.seed)
        model = LlamaForCausalLM(cfg, device=device, dtype=dtype)
    else:
        import transformers
        from opaque_b200 import patches
        hf = transformers.AutoModelForCausalLM.from_pretrained(args.model, local_files_only=True)
        model = patches.apply_model_patches(hf, dtype=dtype, device=device)
    if args.lora_r > 0:
        model.add_lora(args.lora_r, args.lora_alpha or 2.0 * args.lora_r, tuple(args.lora_modules.split(",")))
    if args.gradient_checkpointing:
        model.activation_checkpointing = True
    return model


def lr_schedule(args: argparse.Namespace, steps: int):
    lr, lo = args.learning_rate, args.learning_rate * args.lr_min_ratio
    decay = max(steps - args.lr_warmup_steps, 1)
    base = {"constant": lambda: scheduling.constant_schedule(lr), "cosine": lambda: scheduling.cosine_schedule(lr, lo, decay),
            "linear": lambda: scheduling.linear_schedule(lr, lo, decay)}[args.lr_schedule]()
    return scheduling.with_warmup(base, args.lr_warmup_steps) if args.lr_warmup_steps > 0 else base


def build_optimizer(args: argparse.Namespace, schedule):
    if args.optimizer == "sgd":
        return optimizers.sgd(schedule, weight_decay=args.weight_decay)
    if args.optimizer == "lion":
        return optimizers.lion(schedule, weight_decay=args.weight_decay)
    return optimizers.adamw(schedule, weight_decay=args.weight_decay, noise_bias_correction=args.optimizer == "adamw-bc")


# ------------------------------------------------------------------------------------------------ privacy

def step_process(args: argparse.Namespace, sigma: float, n: int, steps: int):
    """The DP process of ONE step for the chosen sampler (composed ``steps`` times by the caller)."""
    mech = dacc.gaussian(sigma)
    if args.sampler == "poisson":
        return dacc.poisson(mech, args.batch_size / n)
    if args.sampler == "fixed":
        return dacc.k_out_of_t(mech, args.batch_size, n)
    return None       # random allocation is accounted over the whole run, see below


def run_process(args: argparse.Namespace, sigma: float, n: int, steps: int):
    if args.sampler == "random-allocation":
        return dacc.random_allocation(dacc.gaussian(sigma), steps)
    return step_process(args, sigma, n, steps) * steps


def make_sampler(args: argparse.Namespace, shard, n: int, steps: int, rank: int, world: int):
    k = fold_in(key(args.seed), f"sampler/{rank}")
    if args.sampler == "poisson":
        cap = None if args.truncated_batch_size is None else max(args.truncated_batch_size // world, 1)
        return PoissonSampler(shard, args.batch_size / n, n_steps=steps, truncated_batch_size=cap, key=k)
    if args.sampler == "fixed":
        return KOutOfTSampler(shard, max(args.batch_size // world, 1), len(shard), n_steps=steps, key=k)
    return RandomAllocationSampler(shard, steps, n_steps=steps, key=k)


# ------------------------------------------------------------------------------------------------ main

def main() -> None:
    args = parse_args()
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl" if torch.cuda.is_available() and args.engine == "fused" else "gloo")
    rank, world = get_rank(), get_world_size()
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0))) if torch.cuda.is_available() else torch.device("cpu")
    if device.type == "cuda":
        torch.cuda.set_device(device)
    if args.engine == "fused" and device.type != "cuda":
        raise SystemExit("--engine fused needs a CUDA device (B200)")

    rows, vocab = tokenize(args, load_texts(args))
    pad = vocab - 1 if args.dataset != "synthetic" and not args.tokenizer else 0
    train_rows, eval_rows = rows[:args.num_train_samples], rows[args.num_train_samples:args.num_train_samples + args.num_eval_samples]

    # one-run audit: canaries are random token sequences appended to the training set; a fair keyed coin decides which
    # of them are really trained on
    flip = None
    if args.audit:
        gen = torch.Generator().manual_seed(args.seed + 7)
        canaries = [torch.randint(3, min(vocab, 256), (args.max_seq_len,), generator=gen).tolist() for _ in range(args.audit_canaries)]
        first = len(train_rows)
        train_rows = train_rows + canaries
        picked = auditing.coin_flip(range(args.audit_canaries), num_canaries=args.audit_canaries, key=key(args.seed + 8))
        flip = auditing.CoinFlip(picked.canary_indices + first, picked.included, len(train_rows))
        train_rows = [train_rows[i] for i in flip.kept_indices()]
        canary_rows = canaries
    n = len(train_rows)
    steps = args.steps or max(int(math.ceil(args.num_epochs * n / args.batch_size)), 1)

    sigma = args.noise_multiplier
    if sigma is None:
        budget = acc.epsilon_budget(args.target_epsilon, args.target_delta)
        sigma = float(acc.calibrate(budget, lambda s: run_process(args, s, n, steps), args.calibration_min, args.calibration_max,
                                    tolerance=args.calibration_tolerance).param)
    accountant = acc.Accountant()
    per_step = step_process(args, sigma, n, steps)
    if per_step is None:
        accountant |= run_process(args, sigma, n, steps)        # the whole run is one process

    model = build_model(args, vocab, device)
    per = n // world
    shard = range(rank * per, n if rank == world - 1 else (rank + 1) * per)
    sampler = make_sampler(args, shard, n, steps, rank, world)
    schedule = lr_schedule(args, steps)
    trainable = sum(p.numel() for p in model.parameters() if p.requires_grad)

    def to_dev(batch):
        return {k: v.to(device, non_blocking=True) for k, v in batch.items()}

    @torch.no_grad()
    def evaluate() -> dict[str, float]:
        model.eval()
        tot, cnt = 0.0, 0
        mine = eval_rows[rank::world]
        for lo in range(0, len(mine), args.eval_batch_size):
            b = to_dev(collate(mine[lo:lo + args.eval_batch_size], pad))
            tokens = (b["labels"] != -100).sum(1)
            tot += float((model.per_example_loss(b["input_ids"], b["labels"]).float() * tokens).sum())
            cnt += int(tokens.sum())
        model.train()
        tot, cnt = float(reduce_scalar(tot, "sum")), int(reduce_scalar(cnt, "sum"))
        nll = tot / max(cnt, 1)
        return {"eval_nll": nll, "eval_ppl": math.exp(min(nll, 30.0))}

    # ---- the two engines ------------------------------------------------------------------------------
    if args.engine == "fused":
        from opaque_b200.engine.fused import FusedDPEngine
        from opaque_b200.parallel.sharded import DPStepConfig
        if args.clipping_mode == "adaptive" or args.per_group_clipping:
            raise SystemExit("--engine fused: use --clipping-mode fixed|auto with one bound (or the trainer, which supports more)")
        opt_name = {"adamw": "adam", "adamw-bc": "adam", "sgd": "sgd", "lion": "lion"}[args.optimizer]
        cfg = DPStepConfig(lr=schedule, weight_decay=args.weight_decay, noise_bias_correction=args.optimizer == "adamw-bc",
                           optimizer=opt_name, decoupled_weight_decay=args.optimizer != "sgd")
        engine = FusedDPEngine(model, clipping_norm=args.clipping_norm, noise_multiplier=sigma, normalize_by=float(args.batch_size),
                               key=key(args.seed + 1), step_config=cfg, microbatch_size=args.microbatch_size or 8,
                               clipping_mode="auto" if args.clipping_mode == "auto" else "clip", gamma=args.auto_clipping_gamma)

        def train_step(batch):
            res = engine.step(model.per_example_loss, to_dev(batch))
            return {"loss": res.loss, "grad_norm": res.grad_norm_mean, "clip_rate": res.clip_rate, "batch_size": res.batch_size}
    else:
        from opaque_b200.ops.functional import plain_torch_ops
        fmodel, params, frozen = make_functional(model, disable_autograd_tracking=True, partition_trainable=True)

        def loss_fn(p, ex):                       # ONE record; clipped_grad maps it over the batch
            return _one_loss(fmodel, {**frozen, **p}, ex)

        common = dict(normalize_by=float(args.batch_size), batch_argnums=1, return_aux=True, microbatch_size=args.microbatch_size)
        bound = args.clipping_norm
        if args.per_group_clipping:
            spec = json.loads(args.per_group_clipping)
            bound = per_group(params, {k: float(v) for k, v in spec.items() if k != "fallback"}, fallback=spec.get("fallback"))
        if args.clipping_mode == "fixed":
            grad_fn, clip_state = clipped_grad(loss_fn, clipping_norm=bound, **common)
        elif args.clipping_mode == "auto":
            grad_fn, clip_state = auto_clipped_grad(loss_fn, R=bound, gamma=args.auto_clipping_gamma, **common)
        else:
            grad_fn, clip_state = adaptive_clipped_grad(loss_fn, initial_clipping_norm=bound, target_quantile=args.target_clipping_rate,
                                                        clipping_norm_max=args.clipping_norm_max, key=key(args.seed + 2), **common)
        noise_fn, noise_state = gaussian_noise(noise_multiplier=sigma, key=key(args.seed + 1))      # same key on every rank
        opt = build_optimizer(args, schedule)
        opt_state = opt.init(params)
        state = {"params": params, "clip": clip_state, "noise": noise_state, "opt": opt_state}

        def train_step(batch):
            with plain_torch_ops():
                (grads, aux), clip = grad_fn(state["params"], to_dev(batch), state=state["clip"])
            state["clip"], aux = sync(clip, aux)
            grads = sum_gradients_(grads)
            noisy, noise = noise_fn(grads, state["noise"])
            state["noise"] = sync(noise)
            updates, state["opt"] = opt.update(noisy, state["opt"], params=state["params"])
            state["params"] = optimizers.apply_updates(state["params"], updates)
            nb = aux.batch_size
            return {"loss": float(aux.loss_values.mean()) if nb else 0.0, "grad_norm": float(aux.grad_norms.mean()) if nb else 0.0,
                    "clip_rate": float(aux.clipping_rate) if isinstance(aux.clipping_rate, (int, float)) else 0.0, "batch_size": nb}

        def write_back():
            named = dict(model.named_parameters())
            with torch.no_grad():
                for name, v in state["params"].items():
                    named[name].copy_(v)

    # ---- logging ----------------------------------------------------------------------------------------
    log_file = open(args.output, "a") if args.output and rank == 0 else None
    run = None
    if args.wandb_project and rank == 0:
        try:
            import wandb
            run = wandb.init(project=args.wandb_project, config=vars(args))
        except ImportError:
            print("wandb is not installed: logging to stdout / --output only", file=sys.stderr)

    def log(row: dict) -> None:
        if rank != 0:
            return
        line = json.dumps(row)
        print(line, flush=True)
        if log_file:
            log_file.write(line + "\n")
            log_file.flush()
        if run is not None:
            run.log(row)

    log({"event": "start", "world_size": world, "engine": args.engine, "train_records": n, "steps": steps, "noise_multiplier": sigma,
         "trainable_parameters": trainable, "sampler": args.sampler, "clipping_mode": args.clipping_mode, "vocab": vocab})
    baseline = None
    if flip is not None:                                   # canary losses before training: the audit scores are differences
        if args.engine == "reference":
            write_back()
        with torch.no_grad():
            baseline = [float(model.per_example_loss(**to_dev(collate([c], pad)))) for c in canary_rows]

    # ---- the loop ------------------------------------------------------------------------------------------
    t0, window, tokens_seen = time.perf_counter(), [], 0
    last = {}
    for step, idx in enumerate(sampler, start=1):
        batch_rows = [train_rows[i] for i in idx]
        if per_step is not None:
            accountant |= per_step
        if batch_rows or world > 1:
            batch = collate(batch_rows, pad) if batch_rows else {"input_ids": torch.zeros(0, 2, dtype=torch.long), "labels": torch.zeros(0, 2, dtype=torch.long)}
            tokens_seen += int((batch["labels"] != -100).sum())
            last = train_step(batch)
            if last["batch_size"]:
                window.append(last)
        if step % args.log_steps == 0 and window:
            log({"step": step, "loss": sum(w["loss"] for w in window) / len(window), "grad_norm": sum(w["grad_norm"] for w in window) / len(window),
                 "clip_rate": sum(w["clip_rate"] for w in window) / len(window), "lr": float(schedule(step - 1)),
                 "epsilon": accountant.epsilon_at(args.target_delta)})
            window = []
        if args.eval_steps and step % args.eval_steps == 0:
            if args.engine == "reference":
                write_back()
            log({"step": step, **evaluate()})
        if step >= steps or (args.stop_at_step and step >= args.stop_at_step):
            break
    if args.engine == "reference":
        write_back()
    dt = time.perf_counter() - t0
    summary = {"event": "end", "steps": step, "seconds": round(dt, 2), "tokens_per_second": float(reduce_scalar(tokens_seen, "sum")) / max(dt, 1e-9),
               "final_loss": last.get("loss"), **evaluate(), "epsilon": accountant.epsilon_at(args.target_delta), "delta": args.target_delta,
               "noise_multiplier": sigma}
    if flip is not None:
        scores = auditing.loss_scores(lambda c: model.per_example_loss(**to_dev(collate([c], pad))), canary_rows, baseline_losses=baseline)
        est = auditing.one_run(scores, coin_flip=flip, delta=args.target_delta)
        summary["audit_epsilon_lower_bound"] = float(est.epsilon_lower_bound)
        summary["audit_guess_accuracy"] = float(est.accuracy)
        summary["audit_canaries_included"] = int(flip.included.sum())
    log(summary)
    if log_file:
        log_file.close()
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


def _one_loss(fmodel, params, ex):
    """Mean next-token NLL of one record through the functional model (plain PyTorch ops, so ``vmap`` can batch it)."""
    logits = fmodel(params, ex["input_ids"][None])[0].float()
    labels = ex["labels"]
    keep = labels != -100
    nll = torch.nn.functional.cross_entropy(logits, labels.clamp_min(0), reduction="none")
    return (nll * keep).sum() / keep.sum().clamp_min(1)


if __name__ == "__main__":
    main()
