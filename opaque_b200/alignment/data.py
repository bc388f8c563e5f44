"""Collators, completion masks and chat-template helpers for SFT / preference data.

Batches are padded on the right; labels are the inputs shifted left by one with ``−100`` on every position that
must not be scored (padding, prompt tokens when ``completion_only``), so model code never shifts again.

Parity: packages/opaque-alignment/src/opaque/api/alignment/{sft,dpo}/collator/*.py, data/{_chat_template,
_completion_mask,_prompt}.py.
"""
from __future__ import annotations

from collections.abc import Mapping, Sequence
from typing import Any

import torch

IGNORE_INDEX = -100


def completion_mask(input_len: int, prompt_len: int) -> list[int]:
    """1 on completion tokens, 0 on prompt tokens."""
    return [0] * min(prompt_len, input_len) + [1] * max(0, input_len - prompt_len)


def shift_labels(input_ids: torch.Tensor, score_mask: torch.Tensor | None = None, attention_mask: torch.Tensor | None = None):
    """``labels[t] = input_ids[t+1]`` where token ``t+1`` is scored, else ``−100``."""
    labels = torch.full_like(input_ids, IGNORE_INDEX)
    labels[..., :-1] = input_ids[..., 1:]
    keep = torch.ones_like(input_ids, dtype=torch.bool)
    if attention_mask is not None:
        keep &= attention_mask.bool()
    if score_mask is not None:
        keep &= score_mask.bool()
    nxt = torch.zeros_like(keep)
    nxt[..., :-1] = keep[..., 1:]
    return labels.masked_fill(~nxt, IGNORE_INDEX)


def _pad(seqs: Sequence[Sequence[int]], value: int, multiple: int | None, max_length: int | None) -> torch.Tensor:
    n = max((len(s) for s in seqs), default=0)
    if max_length is not None:
        n = min(n, max_length)
    if multiple:
        n = (n + multiple - 1) // multiple * multiple
    out = torch.full((len(seqs), n), value, dtype=torch.long)
    for i, s in enumerate(seqs):
        s = list(s)[:n]
        out[i, :len(s)] = torch.as_tensor(s, dtype=torch.long)
    return out


def language_modeling_collator(examples: Sequence[Mapping[str, Any]], *, pad_token_id: int = 0,
                               completion_only: bool = False, pad_to_multiple_of: int | None = None,
                               max_length: int | None = None, completion_only_loss: bool | None = None) -> dict[str, torch.Tensor]:
    """Collate ``{"input_ids", ["completion_mask"]}`` rows; an empty list gives zero-length tensors (empty Poisson batch).
    ``completion_only_loss`` is the same switch as ``completion_only`` under its TRL name."""
    if completion_only_loss is not None:
        completion_only = bool(completion_only_loss)
    if len(examples) == 0:
        z = torch.zeros((0, pad_to_multiple_of or 1), dtype=torch.long)
        return {"input_ids": z, "attention_mask": z.clone(), "labels": z.clone()}
    ids = _pad([e["input_ids"] for e in examples], pad_token_id, pad_to_multiple_of, max_length)
    att = _pad([[1] * len(e["input_ids"]) for e in examples], 0, pad_to_multiple_of, max_length)
    score = None
    if completion_only:
        if any("completion_mask" not in e for e in examples):
            raise ValueError("completion_only needs a completion_mask on every example")
        score = _pad([e["completion_mask"] for e in examples], 0, pad_to_multiple_of, max_length)
    return {"input_ids": ids, "attention_mask": att, "labels": shift_labels(ids, score, att)}


def preference_collator(examples: Sequence[Mapping[str, Any]], *, pad_token_id: int = 0,
                        pad_to_multiple_of: int | None = None, max_length: int | None = None) -> dict[str, torch.Tensor]:
    """Collate ``{"prompt_input_ids", "chosen_input_ids", "rejected_input_ids"}`` rows into paired sequences.

    One row = one preference pair (the privacy unit): both completions of example i sit at batch index i.
    """
    out: dict[str, torch.Tensor] = {}
    for side in ("chosen", "rejected"):
        seqs = [list(e["prompt_input_ids"]) + list(e[f"{side}_input_ids"]) for e in examples]
        masks = [completion_mask(len(s), len(e["prompt_input_ids"])) for s, e in zip(seqs, examples)]
        ids = _pad(seqs, pad_token_id, pad_to_multiple_of, max_length)
        att = _pad([[1] * len(s) for s in seqs], 0, pad_to_multiple_of, max_length)
        sc = _pad(masks, 0, pad_to_multiple_of, max_length)
        out[f"{side}_input_ids"], out[f"{side}_attention_mask"] = ids, att
        out[f"{side}_labels"] = shift_labels(ids, sc, att) if len(examples) else ids.clone()
    for k in ("ref_chosen_logps", "ref_rejected_logps"):
        if examples and all(k in e for e in examples):
            out[k] = torch.tensor([float(e[k]) for e in examples])
    return out


def apply_chat_template(messages: Sequence[Mapping[str, str]], tokenizer: Any = None, *, add_generation_prompt: bool = False) -> str:
    """Render a conversation with the tokenizer's template, or a plain ``<|role|>`` fallback."""
    if tokenizer is not None and getattr(tokenizer, "chat_template", None):
        return tokenizer.apply_chat_template(messages, tokenize=False, add_generation_prompt=add_generation_prompt)
    text = "".join(f"<|{m['role']}|>\n{m['content']}\n" for m in messages)
    return text + ("<|assistant|>\n" if add_generation_prompt else "")


def split_prompt_completion(messages: Sequence[Mapping[str, str]]):
    """Everything up to the last assistant turn is the prompt."""
    last = max((i for i, m in enumerate(messages) if m["role"] == "assistant"), default=len(messages) - 1)
    return list(messages[:last]), list(messages[last:])


from .chat_template import apply_chat_template_with_mask, clone_chat_template, get_training_chat_template  # noqa: E402

__all__ = ["IGNORE_INDEX", "apply_chat_template", "apply_chat_template_with_mask", "clone_chat_template", "completion_mask",
           "get_training_chat_template", "language_modeling_collator",
           "preference_collator", "shift_labels", "split_prompt_completion"]
