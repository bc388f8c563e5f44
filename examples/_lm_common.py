"""Pieces shared by the functional SFT / DPO examples: models, tokenisation, the functional model call, calibration, logging.

The language-model fine-tuning example (``train_dpsgd_lm.py``) defines the model table, the schedule and the optimizer
factory; they are re-used from there.
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import Any, Callable

import torch
from torch import nn

import opaque_b200.accounting as acc
from opaque_b200.functional import make_functional
from train_dpsgd_lm import MODELS, build_model as build_llama, build_optimizer, lr_schedule  # noqa: F401  (re-exported)


class TinyLM(nn.Module):
    """A few thousand parameters: embedding, one causal mixing layer, head.  Fast enough for CPU smoke runs."""

    def __init__(self, vocab: int = 64, hidden: int = 32):
        super().__init__()
        self.emb = nn.Embedding(vocab, hidden)
        self.mix = nn.Linear(hidden, hidden)
        self.head = nn.Linear(hidden, vocab)

    def forward(self, ids):
        h = self.emb(ids)
        pos = 1 + torch.arange(ids.shape[-1], device=ids.device)
        return self.head(h + torch.tanh(self.mix(torch.cumsum(h, dim=-2) / pos[:, None])))


def add_model_arguments(ap: argparse.ArgumentParser) -> None:
    g = ap.add_argument_group("model")
    g.add_argument("--model", default="tinylm", help="tinylm (toy) | tiny | small | base (random-init Llama) | local Hugging Face checkpoint directory")
    g.add_argument("--dtype", default="float32", choices=["float32", "bfloat16"])
    g.add_argument("--gradient-checkpointing", action="store_true")
    g.add_argument("--lora-r", type=int, default=0, help="0 trains the whole model")
    g.add_argument("--lora-alpha", type=float, default=None)
    g.add_argument("--lora-modules", default="q_proj,k_proj,v_proj,o_proj")
    g.add_argument("--tokenizer", default=None, help="local Hugging Face tokenizer directory (default: bytes; synthetic data needs none)")
    g.add_argument("--max-seq-len", type=int, default=64)
    g.add_argument("--seed", type=int, default=0)


def add_optimizer_arguments(ap: argparse.ArgumentParser, lr: float) -> None:
    g = ap.add_argument_group("optimizer")
    g.add_argument("--lr", "--learning-rate", dest="lr", type=float, default=lr)
    g.add_argument("--optimizer", default="adamw-bc", choices=["sgd", "adamw", "adamw-bc", "lion"])
    g.add_argument("--weight-decay", type=float, default=0.0)
    g.add_argument("--lr-schedule", default="constant", choices=["constant", "cosine", "linear"])
    g.add_argument("--lr-min-ratio", type=float, default=0.1)
    g.add_argument("--lr-warmup-steps", type=int, default=0)


def add_privacy_arguments(ap: argparse.ArgumentParser) -> None:
    g = ap.add_argument_group("differential privacy")
    g.add_argument("--sigma", "--noise-multiplier", dest="sigma", type=float, default=1.0)
    g.add_argument("--target-epsilon", type=float, default=None, help="calibrate sigma to this epsilon instead")
    g.add_argument("--delta", "--target-delta", dest="delta", type=float, default=1e-5)
    g.add_argument("--clip", "--clipping-norm", dest="clip", type=float, default=1.0)
    g.add_argument("--microbatch", type=int, default=None)


class Tokens:
    """``encode(text) -> ids`` and the ids reserved for padding: a local Hugging Face tokenizer, or bytes (pad = 256)."""

    def __init__(self, path: str | None):
        self.hf = None
        if path:
            from transformers import AutoTokenizer
            self.hf = AutoTokenizer.from_pretrained(path, local_files_only=True)
            self.vocab = len(self.hf)
            self.pad = self.hf.pad_token_id if self.hf.pad_token_id is not None else (self.hf.eos_token_id or 0)
        else:
            self.vocab, self.pad = 257, 256

    def encode(self, text: str) -> list[int]:
        if self.hf is not None:
            return list(self.hf(text, add_special_tokens=False)["input_ids"])
        return list(text.encode("utf-8"))


def build_model(args: argparse.Namespace, vocab: int, device: torch.device) -> nn.Module:
    if args.model == "tinylm":
        if args.lora_r:
            raise SystemExit("--lora-r needs a Llama model (--model tiny | small | base | <directory>)")
        torch.manual_seed(args.seed)
        return TinyLM(vocab=(vocab + 7) // 8 * 8).to(device)
    return build_llama(args, vocab, device)


def functional(model: nn.Module) -> tuple[Callable, dict, Callable[[dict], None]]:
    """``(logits_of(trainable, ids), trainable, write_back)``: the model as a pure function of its TRAINABLE parameters
    (frozen ones are closed over), and a function that copies trained values back into the module."""
    fmodel, trainable, frozen = make_functional(model, disable_autograd_tracking=True, partition_trainable=True)

    def logits_of(p, ids):
        out = fmodel({**frozen, **p}, ids)
        return getattr(out, "logits", out)

    def write_back(p):
        named = dict(model.named_parameters())
        with torch.no_grad():
            for name, v in p.items():
                named[name].copy_(v)
    return logits_of, trainable, write_back


def plain_ops():
    """Context in which this package's layers use plain PyTorch ops, so ``vmap`` can batch them (no-op for other models)."""
    from opaque_b200.ops.functional import plain_torch_ops
    return plain_torch_ops()


def schedule_and_optimizer(args: argparse.Namespace, steps: int):
    args.learning_rate = args.lr
    schedule = lr_schedule(args, steps)
    return schedule, build_optimizer(args, schedule)


def noise_multiplier(args: argparse.Namespace, process_of_sigma: Callable[[float], Any]) -> float:
    """``--sigma``, or the smallest multiplier whose whole-run process meets ``--target-epsilon`` at ``--delta``."""
    if args.target_epsilon is None:
        return float(args.sigma)
    budget = acc.epsilon_budget(args.target_epsilon, args.delta)
    return float(acc.calibrate(budget, process_of_sigma, 0.3, 50.0, tolerance=1e-3).param)


def read_jsonl(path: str, limit: int) -> list[dict]:
    rows = []
    with open(path, encoding="utf-8") as f:
        for line in f:
            if line.strip():
                rows.append(json.loads(line))
                if len(rows) >= limit:
                    break
    return rows


def emit(row: dict, rank: int = 0) -> None:
    if rank == 0:
        print(json.dumps(row), flush=True)


def fail(msg: str) -> None:
    print(msg, file=sys.stderr)
    raise SystemExit(2)
