"""Token-level logging metrics for causal language models (detached scalars; not part of any loss).

Both functions take FULL-length logits / labels / mask and shift them here: position ``t`` predicts the token at ``t + 1``.
Under differential privacy these are statistics of the private batch: log them for public / evaluation data, or treat
their release as part of the privacy analysis.

Parity: packages/opaque-alignment/src/opaque/api/alignment/metric/_token.py.
"""
from __future__ import annotations

import torch


def entropy_from_logits(logits: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """Mean Shannon entropy of the predictive distribution over the positions whose (shifted) ``mask`` is set; ``logits``
    ``(..., T, V)``, ``mask`` ``(..., T)``.  Zero when nothing is unmasked."""
    z = logits[..., :-1, :].float()
    m = mask[..., 1:].to(z.dtype)
    logp = z.log_softmax(-1)
    ent = -(logp.exp() * logp).sum(-1)
    return ((ent * m).sum() / m.sum().clamp(min=1)).detach()


def mean_token_accuracy(logits: torch.Tensor, labels: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """Fraction of unmasked (shifted) positions whose arg-max prediction equals the next token.  Zero when nothing is
    unmasked."""
    pred = logits[..., :-1, :].argmax(-1)
    m = mask[..., 1:].bool()
    hit = ((pred == labels[..., 1:]) & m).sum()
    return (hit / m.sum().clamp(min=1)).float().detach()


__all__ = ["entropy_from_logits", "mean_token_accuracy"]
