"""Differentially private supervised fine-tuning (prompt/completion rows, completion-only loss) through ``SFTTrainer``.

  python examples/train_sft_trainer.py --max_steps 10                         # tiny Llama, CPU or GPU
  python examples/train_sft_trainer.py --model llama3-8b --lora 16 --seq 1024 --batch 64 --target_epsilon 8

Parity: examples/train_sft_trainer.py of the reference (SFTConfig surface: completion_only_loss, loss_type nll/dft).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

from opaque_b200.models import LlamaConfig, LlamaForCausalLM
from opaque_b200.transformers.trl import SFTConfig, SFTTrainer


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-tiny", choices=["llama-tiny", "llama3.2-1b", "llama3-8b"])
    ap.add_argument("--lora", type=int, default=16)
    ap.add_argument("--seq", type=int, default=64)
    ap.add_argument("--n", type=int, default=1024)
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--max_steps", type=int, default=10)
    ap.add_argument("--loss_type", default="nll", choices=["nll", "dft", "chunked_nll"])
    ap.add_argument("--noise_multiplier", type=float, default=None)
    ap.add_argument("--target_epsilon", type=float, default=None)
    ap.add_argument("--output_dir", default="")
    a = ap.parse_args()

    device = torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
    cfg = {"llama-tiny": LlamaConfig.tiny, "llama3.2-1b": LlamaConfig.llama32_1b, "llama3-8b": LlamaConfig.llama3_8b}[a.model]()
    torch.manual_seed(0)
    model = LlamaForCausalLM(cfg, device=device, dtype=torch.bfloat16 if device.type == "cuda" else torch.float32)
    if a.lora:
        model.add_lora(a.lora, 2.0 * a.lora)
    g = torch.Generator().manual_seed(1)
    half = a.seq // 2
    rows = [{"input_ids": torch.randint(0, cfg.vocab_size, (a.seq,), generator=g).tolist(),
             "completion_mask": [0] * half + [1] * (a.seq - half)} for _ in range(a.n)]
    if a.noise_multiplier is None and a.target_epsilon is None:
        a.noise_multiplier = 0.7
    args = SFTConfig(output_dir=a.output_dir, per_device_train_batch_size=a.batch, max_steps=a.max_steps, learning_rate=2e-4,
                     privacy_noise_multiplier=a.noise_multiplier, privacy_target_epsilon=a.target_epsilon, clipping_norm=1.0,
                     optim="adamw-bc", loss_type=a.loss_type, completion_only_loss=True, save_steps=0,
                     logging_steps=max(a.max_steps // 5, 1), use_cpu=device.type == "cpu", bf16=device.type == "cuda",
                     max_length=a.seq)
    trainer = SFTTrainer(model=model, args=args, train_dataset=rows)
    out = trainer.train()
    print(json.dumps({"global_step": out["global_step"], "epsilon": out["epsilon"], "engine": trainer.engine_kind}))


if __name__ == "__main__":
    main()
