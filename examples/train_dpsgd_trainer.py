"""DP-SGD / DP-FTRL fine-tuning of a causal LM through ``DPTrainer``.

On a B200 the trainer picks the fused engine (tcgen05 ghost-norm / clip-GEMM kernels, sharded Philox + AdamW-BC step);
on CPU it falls back to the reference engine, so the same script is a smoke test without a GPU.

  python examples/train_dpsgd_trainer.py --model llama-tiny --max_steps 10                 # CPU or GPU
  python examples/train_dpsgd_trainer.py --model llama3-8b --lora 16 --seq 1024 --batch 64 --target_epsilon 8
  python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 examples/train_dpsgd_trainer.py --model gpt2

Parity: examples/train_dpsgd_trainer.py of the reference (argument surface: privacy_*, clipping_*, sampling_mode).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

from opaque_b200.models import GPT2Config, GPT2LMHeadModel, LlamaConfig, LlamaForCausalLM
from opaque_b200.transformers import DPTrainer, TrainingArguments


# Named configurations (the benchmark configurations of this repository, per GPU; launch with torchrun for several GPUs).
# Parity: the presets of examples/train_dpsgd_trainer.py:755-763 of the reference (there: one H200).
PRESETS = {
    "llama3-8b-lora-b200": dict(model="llama3-8b", lora=16, seq=1024, batch=64, noise_multiplier=0.7, clipping_norm=1.0, lr=2e-4),
    "gpt2-full-b200": dict(model="gpt2", lora=0, seq=512, batch=128, noise_multiplier=0.8, clipping_norm=1.0, lr=1e-4),
    "llama3.2-1b-blt-b200": dict(model="llama3.2-1b", lora=0, seq=1024, batch=32, target_epsilon=8.0, clipping_norm=1.0, lr=1e-4,
                                 mechanism="mf_blt", sampling_mode="sequential"),
    "tiny-cpu": dict(model="llama-tiny", lora=8, seq=64, batch=16, noise_multiplier=1.0),
}


def build_model(name: str, lora: int, device):
    dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    if name == "gpt2":
        return GPT2LMHeadModel(GPT2Config.small(), device=device, dtype=dtype), 50257
    cfg = {"llama-tiny": LlamaConfig.tiny, "llama3.2-1b": LlamaConfig.llama32_1b, "llama3-8b": LlamaConfig.llama3_8b}[name]()
    model = LlamaForCausalLM(cfg, device=device, dtype=dtype)
    if lora:
        model.add_lora(lora, 2.0 * lora)
    return model, cfg.vocab_size


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-tiny", choices=["llama-tiny", "gpt2", "llama3.2-1b", "llama3-8b"])
    ap.add_argument("--lora", type=int, default=0)
    ap.add_argument("--seq", type=int, default=64)
    ap.add_argument("--n", type=int, default=4096, help="synthetic dataset size")
    ap.add_argument("--batch", type=int, default=16, help="expected per-device batch")
    ap.add_argument("--max_steps", type=int, default=10)
    ap.add_argument("--noise_multiplier", type=float, default=None)
    ap.add_argument("--target_epsilon", type=float, default=None)
    ap.add_argument("--clipping_norm", type=float, default=1.0)
    ap.add_argument("--clipping_mode", default="fixed", choices=["fixed", "auto", "adaptive"])
    ap.add_argument("--mechanism", default="gaussian")
    ap.add_argument("--sampling_mode", default=None)
    ap.add_argument("--lr", type=float, default=2e-4)
    ap.add_argument("--output_dir", default="")
    ap.add_argument("--preset", default=None, choices=sorted(PRESETS), help="a named configuration; explicit flags still override")
    a = ap.parse_args()
    if a.preset:
        given = {act.dest for act in ap._actions for opt in act.option_strings if opt in sys.argv}
        for k, v in PRESETS[a.preset].items():
            if k not in given:
                setattr(a, k, v)

    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if torch.cuda.is_available():
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        torch.distributed.init_process_group("nccl" if torch.cuda.is_available() else "gloo")
    device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    torch.manual_seed(0)
    model, vocab = build_model(a.model, a.lora, device)
    g = torch.Generator().manual_seed(1)
    rows = [{"input_ids": torch.randint(0, vocab, (a.seq,), generator=g).tolist()} for _ in range(a.n)]
    if a.noise_multiplier is None and a.target_epsilon is None:
        a.noise_multiplier = 1.0
    args = TrainingArguments(
        output_dir=a.output_dir, per_device_train_batch_size=a.batch, max_steps=a.max_steps, learning_rate=a.lr,
        privacy_noise_multiplier=a.noise_multiplier, privacy_target_epsilon=a.target_epsilon,
        privacy_noise_mechanism=a.mechanism, clipping_norm=a.clipping_norm, clipping_mode=a.clipping_mode,
        sampling_mode=a.sampling_mode or ("poisson" if a.mechanism == "gaussian" else "sequential"),
        optim="adamw-bc", logging_steps=max(a.max_steps // 5, 1), save_steps=0, use_cpu=device.type == "cpu",
        bf16=device.type == "cuda")
    trainer = DPTrainer(model=model, args=args, train_dataset=rows)
    out = trainer.train()
    if trainer.is_world_process_zero():
        print(json.dumps({k: out[k] for k in ("global_step", "epsilon", "train_runtime") if k in out} |
                         {"engine": trainer.engine_kind, "noise_multiplier": trainer.noise_multiplier}))
    if torch.distributed.is_initialized():
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
