"""How a privacy budget is spread over parameter groups and paired streams.

Per-group clipping with bounds ``C_i`` gives the MSE-optimal standard
deviations ``σ_i = nm·sqrt(C_i · Σ_j C_j)``: the Mahalanobis sensitivity
``Σ_i C_i²/σ_i²`` then equals ``1/nm²`` exactly, so the accountant still sees
``gaussian(nm)``.  For a paired first/second-moment release with sensitivities
``Δ¹, Δ²`` the same rule over the two streams yields ``σ = nm·sqrt(Δ·S)`` with
``S = Σ(Δ¹+Δ²)``.

Parity: packages/opaque-engine/src/opaque/api/engine/noise_allocation.py:33-95, :136-232.
"""
from __future__ import annotations

import math

from .types import PerGroup

FIRST_MOMENT_FOLD_TAG = 1
SECOND_MOMENT_FOLD_TAG = 2


def per_group_noise_stddev(max_norm: PerGroup, noise_multiplier: float) -> PerGroup:
    vals = dict(max_norm.values)
    for name, c in vals.items():
        if c < 0:
            raise ValueError(f"group {name!r} has a negative bound {c}")
    total = sum(vals.values())
    return PerGroup(max_norm.groups, {k: noise_multiplier * math.sqrt(c * total) for k, c in vals.items()})


def paired_noise_stddev(first, second, noise_multiplier: float):
    """σ for the Σg stream and the Σg² stream released together.

    ``first`` / ``second`` are the two sensitivities (floats or matching
    ``PerGroup``).  Returns ``(σ_first, σ_second)`` of the same kind.
    """
    if isinstance(first, PerGroup) != isinstance(second, PerGroup):
        raise TypeError("paired streams must both be scalar or both PerGroup")
    if isinstance(first, PerGroup):
        if set(first.values) != set(second.values):
            raise ValueError("paired PerGroup streams need the same group names")
        total = sum(first.values.values()) + sum(second.values.values())
        s1 = PerGroup(first.groups, {k: noise_multiplier * math.sqrt(v * total) for k, v in first.values.items()})
        s2 = PerGroup(second.groups, {k: noise_multiplier * math.sqrt(v * total) for k, v in second.values.items()})
        return s1, s2
    total = float(first) + float(second)
    return (noise_multiplier * math.sqrt(float(first) * total),
            noise_multiplier * math.sqrt(float(second) * total))


__all__ = ["FIRST_MOMENT_FOLD_TAG", "SECOND_MOMENT_FOLD_TAG", "paired_noise_stddev", "per_group_noise_stddev"]
