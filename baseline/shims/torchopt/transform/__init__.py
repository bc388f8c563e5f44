"""``add_decayed_weights``: ``updates + weight_decay * params``."""
from __future__ import annotations

import optree

from ..base import GradientTransformation


def add_decayed_weights(weight_decay: float = 0.0, mask=None) -> GradientTransformation:
    def init_fn(params):
        return ()

    def update_fn(updates, state, *, params=None, inplace: bool = True):
        if weight_decay == 0.0:
            return updates, state
        if params is None:
            raise ValueError("add_decayed_weights needs params")
        if inplace:
            return optree.tree_map(lambda g, p: g.add_(p, alpha=weight_decay), updates, params), state
        return optree.tree_map(lambda g, p: g + weight_decay * p, updates, params), state
    return GradientTransformation(init_fn, update_fn)
