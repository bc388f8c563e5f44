"""Named argument presets shared by the example scripts: ``--preset NAME`` fills in a documented configuration, explicit
command-line flags still win.

Parity: the ``--preset`` tables of the reference's examples (examples/train_dpsgd.py:845-900: ``smoke``,
``mellum-kstack`` …); the presets here name this repository's benchmark configurations (synthetic data, no downloads).
"""
from __future__ import annotations

import argparse
import sys

PRESETS: dict[str, dict[str, dict]] = {
    "train_dpsgd": {
        "smoke": dict(steps=10, n=2048, batch=64, sigma=1.0, lr=0.1),
        "mlp-60k": dict(steps=200, n=60000, batch=256, clip=1.0, sigma=1.0, lr=0.1, delta=1e-5),     # benchmark config 1
    },
    "train_dpsgd_lm": {
        "smoke": dict(model="tiny", num_train_samples=256, num_eval_samples=32, max_seq_len=16, batch_size=32, steps=4,
                      noise_multiplier=1.0, log_steps=2, microbatch_size=16),
        "lora-eps8": dict(model="small", lora_r=8, num_train_samples=4096, max_seq_len=128, batch_size=256, num_epochs=3.0,
                          target_epsilon=8.0, target_delta=1e-5, learning_rate=1e-3, lr_warmup_steps=5, eval_steps=16),
        "full-auto-clip": dict(model="small", num_train_samples=4096, max_seq_len=128, batch_size=256, num_epochs=2.0,
                               clipping_mode="auto", noise_multiplier=0.8, optimizer="adamw-bc", learning_rate=5e-4),
        "b200-fused": dict(model="base", engine="fused", dtype="bfloat16", lora_r=16, num_train_samples=16384, max_seq_len=512,
                           batch_size=512, microbatch_size=8, steps=50, target_epsilon=8.0, eval_steps=25),
    },
    "train_dpftrl": {
        "smoke": dict(steps=8, n=512, batch=16, seq=8),
        "blt-4": dict(strategy="blt", buffers=4, sampler="sequential", steps=64, batch=32, sigma=2.0),
        "band-16": dict(strategy="band_mf", bands=16, sampler="b_min_sep", steps=64, batch=32, sigma=2.0),
        "lambda-cgd": dict(strategy="lambda_cgd", lambda_=0.5, sampler="balls_in_bins", steps=64, batch=32, sigma=2.0),
    },
    "train_sft": {
        "smoke": dict(steps=5, n=256, batch=16),
        "dft": dict(steps=40, n=2048, batch=64, loss="dft", sigma=0.8, lr=5e-3),
        "llama-lora-eps8": dict(model="small", lora_r=8, steps=60, n=4096, eval_n=256, batch=128, microbatch=16, target_epsilon=8.0,
                                lr=2e-3, lr_schedule="cosine", lr_warmup_steps=5),
    },
    "train_dpo": {
        "smoke": dict(steps=5, n=128, batch=8),
        "ipo": dict(steps=40, n=1024, batch=32, loss_type="ipo", beta=0.1, sigma=0.8),
        "simpo": dict(steps=40, n=1024, batch=32, loss_type="simpo", beta=2.0, sigma=0.8),
        "llama-lora-eps8": dict(model="small", lora_r=8, steps=60, n=2048, eval_n=128, batch=64, microbatch=8, target_epsilon=8.0,
                                lr=1e-3, loss_type="sigmoid", beta=0.1),
    },
}


def add_preset_argument(ap: argparse.ArgumentParser, script: str) -> None:
    names = sorted(PRESETS[script])
    ap.add_argument("--preset", default=None, choices=names, help="named configuration; explicit flags override it")


def apply_preset(ap: argparse.ArgumentParser, args: argparse.Namespace, script: str, argv: list[str] | None = None) -> argparse.Namespace:
    """Fill ``args`` from the chosen preset, except for options that were given explicitly on the command line."""
    if not getattr(args, "preset", None):
        return args
    argv = sys.argv[1:] if argv is None else argv
    given = set()
    for action in ap._actions:
        if any(tok == opt or tok.startswith(opt + "=") for opt in action.option_strings for tok in argv):
            given.add(action.dest)
    for key, value in PRESETS[script][args.preset].items():
        if not hasattr(args, key):
            raise KeyError(f"preset {args.preset!r} sets unknown option {key!r}")
        if key not in given:
            setattr(args, key, value)
    return args
