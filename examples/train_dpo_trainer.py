"""Differentially private preference optimisation (DPO and its variants) through ``DPOTrainer``.

Reference log-probabilities are precomputed once with the initial model; one privacy unit is one preference pair.

  python examples/train_dpo_trainer.py --max_steps 10 --loss_type sigmoid
  python examples/train_dpo_trainer.py --loss_type ipo --beta 0.2

Parity: examples/train_dpo_trainer.py of the reference (DPOConfig surface: beta, loss_type, loss_weights, ld_alpha).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

from opaque_b200.models import LlamaConfig, LlamaForCausalLM
from opaque_b200.transformers.trl import DPOConfig, DPOTrainer


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--n", type=int, default=512)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--max_steps", type=int, default=10)
    ap.add_argument("--beta", type=float, default=0.1)
    ap.add_argument("--loss_type", default="sigmoid")
    ap.add_argument("--noise_multiplier", type=float, default=1.0)
    ap.add_argument("--output_dir", default="")
    a = ap.parse_args()

    device = torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
    cfg = LlamaConfig.tiny()
    torch.manual_seed(0)
    model = LlamaForCausalLM(cfg, device=device, dtype=torch.float32)
    g = torch.Generator().manual_seed(1)

    def toks(n):
        return torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist()
    rows = [{"prompt_input_ids": toks(12), "chosen_input_ids": toks(10), "rejected_input_ids": toks(8)} for _ in range(a.n)]
    args = DPOConfig(output_dir=a.output_dir, per_device_train_batch_size=a.batch, max_steps=a.max_steps, learning_rate=1e-4,
                     privacy_noise_multiplier=a.noise_multiplier, clipping_norm=1.0, beta=a.beta, loss_type=a.loss_type,
                     save_steps=0, logging_steps=max(a.max_steps // 5, 1), use_cpu=device.type == "cpu", dp_engine="reference")
    trainer = DPOTrainer(model=model, args=args, train_dataset=rows)
    out = trainer.train()
    print(json.dumps({"global_step": out["global_step"], "epsilon": out["epsilon"]}))


if __name__ == "__main__":
    main()
