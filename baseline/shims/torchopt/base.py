"""``GradientTransformation`` protocol: a pair ``(init(params) -> state, update(updates, state, *, params, inplace))``."""
from __future__ import annotations

from typing import Any, Callable, NamedTuple


class GradientTransformation(NamedTuple):
    init: Callable[..., Any]
    update: Callable[..., Any]


def chain(*transformations: GradientTransformation) -> GradientTransformation:
    def init_fn(params):
        return tuple(t.init(params) for t in transformations)

    def update_fn(updates, state, *, params=None, inplace: bool = True):
        new_state = []
        for t, s in zip(transformations, state):
            updates, s = t.update(updates, s, params=params, inplace=inplace)
            new_state.append(s)
        return updates, tuple(new_state)

    return GradientTransformation(init_fn, update_fn)
