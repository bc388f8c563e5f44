"""``scale_by_neg_lr``: multiply updates by ``-lr`` (a float or a schedule of the step count)."""
from __future__ import annotations

import optree

from ..base import GradientTransformation


def scale_by_neg_lr(lr) -> GradientTransformation:
    if callable(lr):
        def init_fn(params):
            return {"count": 0}

        def update_fn(updates, state, *, params=None, inplace: bool = True):
            step = -lr(state["count"])
            return optree.tree_map(lambda g: g * step, updates), {"count": state["count"] + 1}
        return GradientTransformation(init_fn, update_fn)

    neg = -float(lr)

    def init_fn(params):
        return ()

    def update_fn(updates, state, *, params=None, inplace: bool = True):
        if inplace:
            return optree.tree_map(lambda g: g.mul_(neg), updates), state
        return optree.tree_map(lambda g: g * neg, updates), state
    return GradientTransformation(init_fn, update_fn)
