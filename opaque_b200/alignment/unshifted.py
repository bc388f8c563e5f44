"""Collators and SFT losses in the reference library's batch layout: UNSHIFTED labels, the shift inside the loss.

This package's own pipeline aligns labels in the collator (``labels[t]`` is the token that position ``t`` predicts) so that
the fused head + cross-entropy kernel reads them as they are.  The reference does it the other way round: its collators
are FACTORIES (``collate = language_modeling_collator(pad_token_id, max_length, ...)``) whose batches carry
``labels = input_ids`` with −100 on unscored positions plus the ``completion_mask``, and its losses shift
``logits[..., :-1, :]`` against ``labels[..., 1:]``.  Both give the same numbers; code written against the reference finds
its forms here — they are what ``opaque_b200.alignment.sft.collator`` / ``.sft.loss`` / ``.dpo.collator`` export.

Parity: packages/opaque-alignment/src/opaque/api/alignment/sft/collator/_language_modeling.py,
sft/loss/{_nll,_dft}.py, dpo/collator/_preference.py.
"""
from __future__ import annotations

from collections.abc import Callable, Mapping, Sequence
from typing import Any

import torch

from . import sft as _aligned

IGNORE_INDEX = -100


def _round_up(n: int, multiple: int | None) -> int:
    return n if not multiple else (n + multiple - 1) // multiple * multiple


def _pad_rows(rows: Sequence[Sequence[int]], value: int, length: int) -> torch.Tensor:
    out = torch.full((len(rows), length), value, dtype=torch.long)
    for i, r in enumerate(rows):
        if len(r):
            out[i, :len(r)] = torch.as_tensor(list(r), dtype=torch.long)
    return out


def language_modeling_collator(pad_token_id: int, max_length: int, *, completion_only_loss: bool = False,
                               pad_to_multiple_of: int | None = None) -> Callable[[list], dict[str, torch.Tensor]]:
    """``collate(examples) -> {"input_ids", "attention_mask", "labels", ["completion_mask"]}``: rows truncated to
    ``max_length`` from the right, right-padded to the batch maximum (rounded up to ``pad_to_multiple_of``); ``labels`` are
    the input ids with −100 on padding and — with ``completion_only_loss`` — on positions whose ``completion_mask`` is 0.
    An empty list gives ``(0, 0)`` tensors."""
    def collate(examples: list[Mapping[str, Any]]) -> dict[str, torch.Tensor]:
        if len(examples) == 0:
            z = torch.zeros((0, 0), dtype=torch.long)
            return {"input_ids": z, "attention_mask": z.clone(), "labels": z.clone()}
        ids = [list(e["input_ids"])[:max_length] for e in examples]
        length = _round_up(max(len(r) for r in ids), pad_to_multiple_of)
        input_ids = _pad_rows(ids, pad_token_id, length)
        attention = _pad_rows([[1] * len(r) for r in ids], 0, length)
        labels = torch.where(attention.bool(), input_ids, torch.full_like(input_ids, IGNORE_INDEX))
        batch = {"input_ids": input_ids, "attention_mask": attention, "labels": labels}
        if all("completion_mask" in e for e in examples):
            cmask = _pad_rows([list(e["completion_mask"])[:max_length] for e in examples], 0, length)
            batch["completion_mask"] = cmask
            if completion_only_loss:
                batch["labels"] = torch.where(cmask.bool(), labels, torch.full_like(labels, IGNORE_INDEX))
        elif completion_only_loss:
            raise ValueError("completion_only_loss needs a completion_mask on every example")
        return batch
    return collate


def preference_collator(pad_token_id: int, max_length: int, *, pad_to_multiple_of: int | None = None) -> Callable[[list], dict[str, torch.Tensor]]:
    """``collate(pairs)`` in the ``(B, …)`` layout (pair ``i`` at index ``i`` on both sides): ``{side}_input_ids``,
    ``{side}_attention_mask``, ``{side}_completion_mask`` for ``chosen`` and ``rejected`` (each side padded to its own
    maximum), and ``ref_{side}_logps`` when every pair carries them.  A pair is either the reference's row
    (``{side}_input_ids`` = prompt + response with ``{side}_completion_mask``) or this package's
    (``prompt_input_ids`` + response-only ``{side}_input_ids``)."""
    def side(examples, name):
        ids, masks = [], []
        for e in examples:
            if f"{name}_completion_mask" in e:
                full, m = list(e[f"{name}_input_ids"]), list(e[f"{name}_completion_mask"])
            else:
                prompt, resp = list(e["prompt_input_ids"]), list(e[f"{name}_input_ids"])
                full, m = prompt + resp, [0] * len(prompt) + [1] * len(resp)
            ids.append(full[:max_length])
            masks.append(m[:max_length])
        length = _round_up(max((len(r) for r in ids), default=0), pad_to_multiple_of)
        return {f"{name}_input_ids": _pad_rows(ids, pad_token_id, length),
                f"{name}_attention_mask": _pad_rows([[1] * len(r) for r in ids], 0, length),
                f"{name}_completion_mask": _pad_rows(masks, 0, length)}

    def collate(examples: list[Mapping[str, Any]]) -> dict[str, torch.Tensor]:
        batch = {**side(examples, "chosen"), **side(examples, "rejected")}
        for key in ("ref_chosen_logps", "ref_rejected_logps"):
            if examples and all(key in e for e in examples):
                batch[key] = torch.tensor([float(e[key]) for e in examples], dtype=torch.float32)
        return batch
    return collate


def _shift(labels: torch.Tensor) -> torch.Tensor:
    """Aligned labels for the logits at positions ``0 … T−2`` (the last position predicts nothing)."""
    return labels[..., 1:]


def nll_loss(logits: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    """Per-example mean NLL with the causal shift inside: ``logits[..., :-1, :]`` against ``labels[..., 1:]`` (−100 ignored;
    the divisor is the example's own number of scored tokens)."""
    return _aligned.nll_loss(logits[..., :-1, :], _shift(labels))


def dft_loss(logits: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    """Dynamic fine-tuning loss with the causal shift inside (see :func:`opaque_b200.alignment.sft.dft_loss`)."""
    return _aligned.dft_loss(logits[..., :-1, :], _shift(labels))


def _aligned_labels(labels: torch.Tensor) -> torch.Tensor:
    out = torch.full_like(labels, IGNORE_INDEX)
    out[..., :-1] = labels[..., 1:]
    return out


def fused_nll_loss(hidden_states: torch.Tensor, lm_head_weight: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    """:func:`nll_loss` from final hidden states and the output head, without keeping logits."""
    return _aligned.fused_nll_loss(hidden_states, lm_head_weight, _aligned_labels(labels))


def fused_dft_loss(hidden_states: torch.Tensor, lm_head_weight: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    """:func:`dft_loss` from final hidden states and the output head, without keeping logits."""
    return _aligned.fused_dft_loss(hidden_states, lm_head_weight, _aligned_labels(labels))


__all__ = ["dft_loss", "fused_dft_loss", "fused_nll_loss", "language_modeling_collator", "nll_loss", "preference_collator"]
