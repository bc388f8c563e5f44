"""Functional dynamic loss scaling for fp16 runs (a stateless GradScaler).

``loss_scaler(...)`` returns ``(LossScaler, LossScalerState)``.  The three
members are pure functions; the caller threads the frozen state.  The unscale
step is meant to be bound as ``pre_clipping_transform`` of ``clipped_grad`` so
that per-example gradients are divided by the scale *before* their norm is
taken.  An overflow never suppresses the noised update or its accounting: the
loop always applies noise and only uses ``stats.all_finite`` to back the scale
off.

Parity: packages/opaque-engine/src/opaque/api/engine/precision/_loss_scaler.py:123.
"""
from __future__ import annotations

import dataclasses
import math
from collections.abc import Callable
from typing import Any, NamedTuple

import torch

from ..pytree import tree_leaves, tree_map
from ..types import ClippedPytree, SecondMomentClippingOutput


@dataclasses.dataclass(frozen=True)
class LossScalerState:
    scale: float
    growth_tracker: int


class LossScaler(NamedTuple):
    scale_loss: Callable[[torch.Tensor, LossScalerState], torch.Tensor]
    unscale_grads: Callable[[Any, LossScalerState], Any]
    update: Callable[[LossScalerState, bool], LossScalerState]


def _scalable(x: Any) -> bool:
    return isinstance(x, torch.Tensor) and (x.is_floating_point() or x.is_complex())


def loss_scaler(*, init_scale: float = 2.0 ** 16, growth_factor: float = 2.0,
                backoff_factor: float = 0.5, growth_interval: int = 2000,
                enabled: bool = True) -> tuple[LossScaler, LossScalerState]:
    """Functional dynamic loss scaler for fp16: returns ``(LossScaler, LossScalerState)``."""
    if not math.isfinite(init_scale) or init_scale <= 0.0:
        raise ValueError(f"init_scale must be finite and > 0, got {init_scale}")
    if not math.isfinite(growth_factor) or growth_factor <= 1.0:
        raise ValueError(f"growth_factor must be finite and > 1.0, got {growth_factor}")
    if not 0.0 < backoff_factor < 1.0:
        raise ValueError(f"backoff_factor must be in (0, 1), got {backoff_factor}")
    if growth_interval <= 0:
        raise ValueError(f"growth_interval must be > 0, got {growth_interval}")

    def scale_loss(loss, state):
        return loss * state.scale if enabled else loss

    def unscale_grads(grads, state):
        if not enabled:
            return grads
        inv = state.scale
        return tree_map(lambda g: g / inv if _scalable(g) else g, grads)

    def update(state, grads_were_finite):
        if not enabled:
            return state
        if not grads_were_finite:
            return LossScalerState(state.scale * backoff_factor, 0)
        streak = state.growth_tracker + 1
        if streak >= growth_interval:
            return LossScalerState(state.scale * growth_factor, 0)
        return LossScalerState(state.scale, streak)

    return LossScaler(scale_loss, unscale_grads, update), LossScalerState(float(init_scale), 0)


def all_finite(updates: Any) -> bool:
    """True iff every floating or complex tensor leaf is finite (wrappers are opened)."""
    pending = [updates]
    while pending:
        node = pending.pop()
        if isinstance(node, SecondMomentClippingOutput):
            pending += [node.grads, node.squared_grads]
        elif isinstance(node, ClippedPytree):
            pending.append(node.pytree)
        elif isinstance(node, torch.Tensor):
            if _scalable(node) and not bool(torch.isfinite(node).all()):
                return False
        else:
            leaves = tree_leaves(node)
            if len(leaves) == 1 and leaves[0] is node:
                continue
            pending += leaves
    return True


__all__ = ["LossScaler", "LossScalerState", "all_finite", "loss_scaler"]
