"""Minimal stand-in for the third-party ``torchopt`` package (only what the reference arm calls)."""
from __future__ import annotations

from typing import Any

import optree
import torch

from . import alias, base, transform
from .base import GradientTransformation, chain

__version__ = "0.0-standin"


def apply_updates(params: Any, updates: Any, *, inplace: bool = True) -> Any:
    """``params + updates`` leaf by leaf (in place by default, as in torchopt)."""
    if inplace:
        def f(p, u):
            if u is not None and p is not None:
                p.data.add_(u)
            return p
        return optree.tree_map(f, params, updates)
    return optree.tree_map(lambda p, u: p if u is None else p + u, params, updates)


def sgd(lr, momentum: float = 0.0, dampening: float = 0.0, weight_decay: float = 0.0, nesterov: bool = False, *,
        moment_requires_grad: bool = False, maximize: bool = False) -> GradientTransformation:
    """Functional SGD with optional (Nesterov) momentum and L2 weight decay."""
    if callable(lr):
        schedule = lr
    else:
        def schedule(_count, _lr=float(lr)):
            return _lr

    def init_fn(params):
        trace = optree.tree_map(lambda p: torch.zeros_like(p, requires_grad=moment_requires_grad), params) if momentum else None
        return {"trace": trace, "count": 0, "first": True}

    def update_fn(updates, state, *, params=None, inplace: bool = True):
        sign = 1.0 if maximize else -1.0
        if weight_decay:
            updates = optree.tree_map(lambda g, p: g + weight_decay * p, updates, params)
        trace, first = state["trace"], state["first"]
        if momentum:
            if first:
                trace = optree.tree_map(lambda g: g.clone(), updates)
            else:
                trace = optree.tree_map(lambda t, g: t * momentum + (1.0 - dampening) * g, trace, updates)
            updates = optree.tree_map(lambda g, t: g + momentum * t, updates, trace) if nesterov else trace
        step_lr = schedule(state["count"])
        out = optree.tree_map(lambda g: g * (sign * step_lr), updates)
        return out, {"trace": trace, "count": state["count"] + 1, "first": False}

    return GradientTransformation(init_fn, update_fn)
