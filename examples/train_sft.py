"""Functional DP-SFT: per-example completion-only NLL (or DFT) loss, clipped_grad → gaussian_noise → optimizer.

The explicit loop of the functional API (what ``SFTTrainer`` does internally).  One privacy unit = one conversation:
all of its tokens are clipped as one gradient.

  python examples/train_sft.py --steps 20 --loss dft                                   # toy model, synthetic pairs, CPU
  python examples/train_sft.py --model small --lora-r 8 --dataset chats.jsonl --format messages --target-epsilon 8
  python examples/train_sft.py --dataset pairs.jsonl --format prompt-completion --tokenizer ./tok --no-completion-only

Data formats (``--dataset file.jsonl``): ``prompt-completion`` rows ``{"prompt": ..., "completion": ...}``; ``messages``
rows ``{"messages": [{"role": ..., "content": ...}, ...]}`` (everything up to the last assistant turn is the prompt,
rendered with the tokenizer's chat template or a plain ``<|role|>`` fallback); ``text`` rows ``{"text": ...}`` (loss on
every token).  With ``--completion-only`` (default) prompt tokens carry no loss.

Parity: examples/train_sft.py of the reference (completion masks, chat templates, one privacy unit = one conversation).
"""
from __future__ import annotations

import argparse
import math
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from _presets import add_preset_argument, apply_preset  # noqa: E402

import torch

import opaque_b200.accounting as acc
from opaque_b200 import optimizers
from opaque_b200.alignment import data as adata
from opaque_b200.alignment import sft
from opaque_b200.distributed import sum_gradients_, sync
from opaque_b200.dpsgd import PoissonSampler, clipped_grad, gaussian_noise
from opaque_b200.dpsgd import accounting as dacc
from opaque_b200.random import key

import _lm_common as C  # noqa: E402


def load_rows(a: argparse.Namespace, tok: C.Tokens) -> tuple[list[dict], int, int]:
    """Rows ``{"input_ids", "completion_mask"}``, the vocabulary size and the padding id."""
    T = a.max_seq_len
    if a.dataset == "synthetic":
        g = torch.Generator().manual_seed(a.seed)
        rows = []
        for _ in range(a.n + a.eval_n):
            lp, lc = int(torch.randint(4, 9, (1,), generator=g)), int(torch.randint(4, 9, (1,), generator=g))
            prompt = torch.randint(1, 64, (lp,), generator=g).tolist()
            completion = [(prompt[i % lp] + 1 + i) % 63 + 1 for i in range(lc)]            # a function of the prompt: learnable
            rows.append({"input_ids": prompt + completion, "completion_mask": adata.completion_mask(lp + lc, lp)})
        return rows, 64, 0
    rows = []
    for r in C.read_jsonl(a.dataset, a.n + a.eval_n):
        if a.format == "messages":
            prompt_msgs, completion_msgs = adata.split_prompt_completion(r[a.messages_field])
            prompt = adata.apply_chat_template(prompt_msgs, tok.hf, add_generation_prompt=True)
            full = adata.apply_chat_template(prompt_msgs + completion_msgs, tok.hf)
            p_ids, ids = tok.encode(prompt), tok.encode(full)
        elif a.format == "prompt-completion":
            p_ids = tok.encode(str(r[a.prompt_field]))
            ids = p_ids + tok.encode(str(r[a.completion_field]))
        else:
            p_ids, ids = [], tok.encode(str(r[a.text_field]))
        ids = ids[:T]
        lp = min(len(p_ids), max(len(ids) - 1, 0))
        if len(ids) < 2:
            continue
        rows.append({"input_ids": ids, "completion_mask": adata.completion_mask(len(ids), lp if a.completion_only else 0)})
    if len(rows) < a.n + a.eval_n:
        C.fail(f"{a.dataset}: {len(rows)} usable rows, need --n + --eval-n = {a.n + a.eval_n}")
    return rows, tok.vocab, tok.pad


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    add_preset_argument(ap, "train_sft")
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--n", type=int, default=1024, help="training conversations")
    ap.add_argument("--eval-n", type=int, default=0, help="held-out conversations evaluated at the end")
    ap.add_argument("--batch", type=int, default=32, help="expected batch size (Poisson)")
    ap.add_argument("--loss", default="nll", choices=["nll", "dft"])
    g = ap.add_argument_group("data")
    g.add_argument("--dataset", default="synthetic", help="synthetic | file.jsonl")
    g.add_argument("--format", default="prompt-completion", choices=["prompt-completion", "messages", "text"])
    g.add_argument("--prompt-field", default="prompt")
    g.add_argument("--completion-field", default="completion")
    g.add_argument("--messages-field", default="messages")
    g.add_argument("--text-field", default="text")
    g.add_argument("--completion-only", action=argparse.BooleanOptionalAction, default=True)
    C.add_model_arguments(ap)
    C.add_optimizer_arguments(ap, lr=1e-2)
    C.add_privacy_arguments(ap)
    a = apply_preset(ap, ap.parse_args(), "train_sft")

    device = torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
    tok = C.Tokens(a.tokenizer) if a.dataset != "synthetic" else None
    rows, vocab, pad = load_rows(a, tok)
    train, held_out = rows[:a.n], rows[a.n:a.n + a.eval_n]
    model = C.build_model(a, vocab, device)
    logits_of, params, write_back = C.functional(model)
    loss_of = sft.dft_loss if a.loss == "dft" else sft.nll_loss

    def loss_fn(p, ex):                      # ONE conversation; clipped_grad maps it over the batch
        return loss_of(logits_of(p, ex["input_ids"][None])[0].float(), ex["labels"])      # the collator already shifted the labels

    q = a.batch / a.n
    sigma = C.noise_multiplier(a, lambda s: dacc.poisson(dacc.gaussian(s), q) * a.steps)
    sampler = PoissonSampler(range(a.n), q, n_steps=a.steps, key=key(a.seed + 1))
    grad_fn, clip_state = clipped_grad(loss_fn, clipping_norm=a.clip, normalize_by=float(a.batch), batch_argnums=1, return_aux=True,
                                       microbatch_size=a.microbatch)
    noise_fn, noise_state = gaussian_noise(noise_multiplier=sigma, key=key(a.seed + 2))
    schedule, opt = C.schedule_and_optimizer(a, a.steps)
    opt_state = opt.init(params)
    accountant = acc.Accountant()
    step_process = dacc.poisson(dacc.gaussian(sigma), q)

    def collate(batch_rows):
        b = adata.language_modeling_collator(batch_rows, pad_token_id=pad, completion_only=True)
        return {"input_ids": b["input_ids"].to(device), "labels": b["labels"].to(device)}

    losses = []
    for step, idx in zip(range(a.steps), sampler):
        accountant |= step_process                      # an empty draw is still a step of the mechanism
        if not idx:
            continue
        with C.plain_ops():
            (grads, aux), clip_state = grad_fn(params, collate([train[i] for i in idx]), state=clip_state)
        grads, aux = sum_gradients_(grads), sync(aux)
        noisy, noise_state = noise_fn(grads, noise_state)
        updates, opt_state = opt.update(noisy, opt_state, params=params)
        params = optimizers.apply_updates(params, updates)
        losses.append(float(aux.loss_values.mean()))
    write_back(params)
    summary = {"loss": a.loss, "steps": len(losses), "first_loss": losses[0], "last_loss": losses[-1], "noise_multiplier": sigma,
               "epsilon": accountant.epsilon_at(a.delta), "delta": a.delta}
    if held_out:
        model.eval()
        tot = cnt = hit = 0.0
        with torch.no_grad():
            for lo in range(0, len(held_out), 32):
                b = collate(held_out[lo:lo + 32])
                out = model(b["input_ids"])
                logits = getattr(out, "logits", out).float()
                keep = b["labels"] != -100
                tot += float(sum(sft.nll_loss(lg, lb) * k.sum() for lg, lb, k in zip(logits, b["labels"], keep)))
                hit += float(sum(sft.token_accuracy(lg, lb) * k.sum() for lg, lb, k in zip(logits, b["labels"], keep)))
                cnt += float(keep.sum())
        summary.update(eval_nll=tot / max(cnt, 1), eval_ppl=math.exp(min(tot / max(cnt, 1), 30.0)), eval_token_accuracy=hit / max(cnt, 1))
    C.emit(summary)


if __name__ == "__main__":
    main()
