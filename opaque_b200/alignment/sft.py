"""Per-example SFT losses and log-probability helpers.

``nll_loss`` averages over EACH example's own scored tokens (never over the batch), which is what makes the
loss a sum of per-record terms that DP clipping can bound.  ``dft_loss`` is the token-scaled variant (each
token's NLL weighted by its own detached probability).  The ``fused_*`` forms take the final hidden states and the
output-head weight and never materialise ``[T, V]`` logits for unscored tokens.

Parity: packages/opaque-alignment/src/opaque/api/alignment/sft/loss/{_nll,_dft}.py, logprob/{_gather,_sequence}.py,
_fused_lce.py.
"""
from __future__ import annotations

import torch

from .. import ops
from ..models.layers import linear_cross_entropy, per_example_token_weights

IGNORE_INDEX = -100


def selective_log_softmax(logits: torch.Tensor, index: torch.Tensor) -> torch.Tensor:
    """``log_softmax(logits, -1).gather(-1, index)`` without materialising the softmax."""
    flat = logits.reshape(-1, logits.shape[-1])
    return (-ops.cross_entropy(flat, index.reshape(-1), ignore_index=-(2 ** 62))).view(index.shape)


def token_logps(logits: torch.Tensor, labels: torch.Tensor, ignore_index: int = IGNORE_INDEX):
    """Log-probability of each label token (0 where ignored) and the scoring mask."""
    mask = labels != ignore_index
    safe = labels.masked_fill(~mask, 0)
    return selective_log_softmax(logits, safe) * mask, mask


def sequence_logp(logits: torch.Tensor, labels: torch.Tensor, *, average: bool = False, ignore_index: int = IGNORE_INDEX,
                  length_normalized: bool | None = None):
    """Sum (or mean: ``average`` / ``length_normalized``) of label log-probabilities over each sequence's scored tokens."""
    average = bool(length_normalized) if length_normalized is not None else average
    lp, mask = token_logps(logits, labels, ignore_index)
    total = lp.sum(-1)
    return total / mask.sum(-1).clamp_min(1) if average else total


def nll_loss(logits: torch.Tensor, labels: torch.Tensor, ignore_index: int = IGNORE_INDEX) -> torch.Tensor:
    """Mean NLL over each example's own scored tokens; ``logits [..., T, V]``, ``labels [..., T]`` already aligned."""
    return -sequence_logp(logits, labels, average=True, ignore_index=ignore_index)


def dft_loss(logits: torch.Tensor, labels: torch.Tensor, ignore_index: int = IGNORE_INDEX) -> torch.Tensor:
    """Dynamic fine-tuning: ``−Σ sg(p_t)·log p_t / count``."""
    lp, mask = token_logps(logits, labels, ignore_index)
    return -(lp.detach().exp() * lp).sum(-1) / mask.sum(-1).clamp_min(1)


def fused_nll_loss(hidden_states: torch.Tensor, lm_head_weight: torch.Tensor, labels: torch.Tensor,
                   ignore_index: int = IGNORE_INDEX, chunk: int = 8192) -> torch.Tensor:
    """``nll_loss`` from final hidden states ``[B, T, d]`` and the output head, through the fused linear-CE node."""
    hidden, head_weight = hidden_states, lm_head_weight
    B, T = labels.shape
    w = per_example_token_weights(labels, ignore_index).reshape(-1)
    rows = linear_cross_entropy(hidden.reshape(B * T, -1), head_weight, labels.reshape(-1), w, chunk=chunk,
                                ignore_index=ignore_index)
    return rows.view(B, T).sum(1)


def fused_dft_loss(hidden_states: torch.Tensor, lm_head_weight: torch.Tensor, labels: torch.Tensor,
                   ignore_index: int = IGNORE_INDEX, chunk: int = 8192) -> torch.Tensor:
    """``dft_loss`` from final hidden states ``[B, T, d]`` and the output head without keeping logits: one pass without
    gradients gives every token's probability (the detached weight), a second pass the weighted NLL."""
    hidden, head_weight = hidden_states, lm_head_weight
    B, T = labels.shape
    mask = labels != ignore_index
    h2, l1 = hidden.reshape(B * T, -1), labels.reshape(-1)
    with torch.no_grad():
        nll = linear_cross_entropy(h2, head_weight, l1, mask.float().reshape(-1), chunk=chunk, ignore_index=ignore_index)
        prob = torch.exp(-nll.float()).view(B, T) * mask
    w = prob / mask.sum(1, keepdim=True).clamp_min(1)
    rows = linear_cross_entropy(h2, head_weight, l1, w.reshape(-1).to(torch.float32), chunk=chunk, ignore_index=ignore_index)
    return rows.view(B, T).sum(1)


def fused_sequence_logp(hidden_states, lm_head_weight, labels, *, average: bool = False, ignore_index: int = IGNORE_INDEX,
                        chunk: int = 8192, length_normalized: bool | None = None):
    """Per-sequence (sum or mean) log-probability of the labels from hidden states and the head weight, without keeping logits."""
    hidden, head_weight = hidden_states, lm_head_weight
    average = bool(length_normalized) if length_normalized is not None else average
    B, T = labels.shape
    mask = labels != ignore_index
    w = per_example_token_weights(labels, ignore_index) if average else mask.float()
    rows = linear_cross_entropy(hidden.reshape(B * T, -1), head_weight, labels.reshape(-1), w.reshape(-1), chunk=chunk,
                                ignore_index=ignore_index)
    return -rows.view(B, T).sum(1)


def token_accuracy(logits: torch.Tensor, labels: torch.Tensor, ignore_index: int = IGNORE_INDEX) -> torch.Tensor:
    """Fraction of scored tokens whose arg-max prediction equals the label."""
    mask = labels != ignore_index
    return ((logits.argmax(-1) == labels) & mask).sum().float() / mask.sum().clamp_min(1)


__all__ = ["IGNORE_INDEX", "dft_loss", "fused_dft_loss", "fused_nll_loss", "fused_sequence_logp", "nll_loss", "selective_log_softmax",
           "sequence_logp", "token_accuracy", "token_logps"]
