"""Type-level DP pipeline: ``ClippedPytree`` → ``NoisedPytree`` and ``PerGroup``.

A clipped tree carries the public bound ``max_norm`` on one record's
contribution; a noised tree additionally carries the realised noise standard
deviation.  Only operations that keep that interpretation valid (multiplying
or dividing by a public scalar, negation) are allowed on the wrappers;
everything else must go through ``.pytree`` and an explicit re-wrap.

Parity: packages/opaque-engine/src/opaque/api/engine/types.py:70-153 (PerGroup),
:161-188 (state ABCs), :247-401 (ClippedPytree / NoisedPytree), :409-445
(paired second-moment outputs).
"""
from __future__ import annotations

import math
from abc import ABC
from collections.abc import Mapping
from dataclasses import dataclass, replace
from types import MappingProxyType
from typing import Any, Literal, NamedTuple, Union

import torch

from .pytree import ParamPath, param_path, tree_map

TensorPytree = Any


@dataclass(frozen=True)
class PerGroup:
    """Per-group scalars plus the leaf-path → group-name assignment."""

    groups: Mapping[Any, str]
    values: Mapping[str, float]

    def __post_init__(self) -> None:
        norm = {param_path(k): g for k, g in self.groups.items()}
        object.__setattr__(self, "groups", MappingProxyType(norm))
        object.__setattr__(self, "values", MappingProxyType(dict(self.values)))

    @property
    def effective(self) -> float:
        """``sqrt(Σ v²)`` — the scalar the accountant sees."""
        return math.sqrt(sum(float(v) ** 2 for v in self.values.values()))

    def _map(self, fn) -> "PerGroup":
        return PerGroup(self.groups, {k: fn(k, v) for k, v in self.values.items()})

    def __mul__(self, other: Any) -> "PerGroup":
        if isinstance(other, PerGroup):
            if dict(other.groups) != dict(self.groups) or set(other.values) != set(self.values):
                raise ValueError("PerGroup * PerGroup needs identical group assignments and names")
            return self._map(lambda k, v: v * other.values[k])
        return self._map(lambda k, v: v * other)

    def __rmul__(self, scalar: float) -> "PerGroup":
        return self._map(lambda k, v: scalar * v)

    def __truediv__(self, scalar: float) -> "PerGroup":
        return self._map(lambda k, v: v / scalar)

    def for_path(self, path: Any) -> float:
        return self.values[self.groups[param_path(path)]]

    def __hash__(self) -> int:
        return hash((tuple(sorted(self.groups.items(), key=repr)), tuple(sorted(self.values.items()))))

    def __eq__(self, other: Any) -> bool:
        return (isinstance(other, PerGroup) and dict(self.groups) == dict(other.groups)
                and dict(self.values) == dict(other.values))


MaxNorm = Union[float, PerGroup]
NoiseStddev = Union[float, PerGroup, None]


class ClipState(ABC):
    """Marker base for the state threaded through a clipping transform."""


class NoiseState(ABC):
    """Marker base for the state threaded through a noise mechanism."""


def _public_scalar(value: Any, op: str) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        if isinstance(value, torch.Tensor) and value.ndim == 0 and not value.requires_grad:
            return float(value)
        raise TypeError(f"{op}: only a public Python scalar keeps the max_norm meaning")
    if not math.isfinite(float(value)):
        raise ValueError(f"{op}: scalar must be finite")
    return float(value)


def _scale_bound(bound: Any, s: float) -> Any:
    if bound is None:
        return None
    if isinstance(bound, PerGroup):
        return bound * abs(s)
    return float(bound) * abs(s)


def _scale_leaves(tree: Any, s: float) -> Any:
    return tree_map(lambda x: x * s if isinstance(x, torch.Tensor) else x, tree)


def _no(op: str):
    def raiser(self, *a: Any, **k: Any):
        raise TypeError(
            f"ClippedPytree {op} does not keep the max_norm guarantee; work on `.pytree` "
            "and re-wrap with an explicit max_norm")
    return raiser


@dataclass(frozen=True)
class ClippedPytree:
    """A tree whose per-record contribution has L2 norm at most ``max_norm``."""

    pytree: Any
    max_norm: MaxNorm

    @property
    def sensitivity(self) -> float:
        m = self.max_norm
        return float(m.effective) if isinstance(m, PerGroup) else float(m)

    def noise_stddev_for(self, *, noise_multiplier: float,
                         allocation: Literal["isotropic", "optimal"] = "optimal"):
        """σ that ``gaussian(noise_multiplier)`` applies to this tree.

        Scalar bound: ``nm·C``.  Per-group bound: ``optimal`` gives
        ``σ_i = nm·sqrt(C_i·ΣC_j)``; ``isotropic`` gives ``nm·sqrt(ΣC_i²)``.
        """
        if noise_multiplier < 0:
            raise ValueError(f"noise_multiplier must be non-negative, got {noise_multiplier}")
        if allocation not in ("isotropic", "optimal"):
            raise ValueError(f"allocation must be 'isotropic' or 'optimal', got {allocation!r}")
        if isinstance(self.max_norm, PerGroup):
            if allocation == "isotropic":
                return noise_multiplier * self.max_norm.effective
            from .noise_allocation import per_group_noise_stddev
            return per_group_noise_stddev(self.max_norm, noise_multiplier)
        return noise_multiplier * float(self.max_norm)

    def _scaled(self, s: float) -> "ClippedPytree":
        return replace(self, pytree=_scale_leaves(self.pytree, s), max_norm=_scale_bound(self.max_norm, s))

    def __mul__(self, s: Any):
        return self._scaled(_public_scalar(s, "ClippedPytree *"))

    __rmul__ = __mul__

    def __truediv__(self, s: Any):
        f = _public_scalar(s, "ClippedPytree /")
        if f == 0.0:
            raise ZeroDivisionError("ClippedPytree division by zero")
        return self._scaled(1.0 / f)

    def __neg__(self):
        return self._scaled(-1.0)

    __add__ = __radd__ = _no("addition")
    __sub__ = __rsub__ = _no("subtraction")
    __pow__ = _no("power")
    __rtruediv__ = _no("reverse division")

    def _apply(self, name: str, *a: Any, **k: Any):
        return replace(self, pytree=tree_map(
            lambda x: getattr(x, name)(*a, **k) if isinstance(x, torch.Tensor) else x, self.pytree))

    def clone(self):
        return self._apply("clone")

    def detach(self):
        return self._apply("detach")

    def to(self, *a: Any, **k: Any):
        return self._apply("to", *a, **k)


@dataclass(frozen=True)
class NoisedPytree(ClippedPytree):
    """A privatised tree; ``max_norm`` is still the pre-noise record bound."""

    noise_stddev: NoiseStddev = None

    def _scaled(self, s: float) -> "NoisedPytree":
        return replace(self, pytree=_scale_leaves(self.pytree, s),
                       max_norm=_scale_bound(self.max_norm, s),
                       noise_stddev=_scale_bound(self.noise_stddev, s))


class SecondMomentClippingOutput(NamedTuple):
    """Clipped Σg and clipped Σg² (each with its own bound), before noise."""

    grads: ClippedPytree
    squared_grads: ClippedPytree


class SecondMomentNoiseOutput(NamedTuple):
    """Noised Σg and noised Σg² for optimizers with a private second moment."""

    noisy_grads: NoisedPytree
    noisy_squared_grads: NoisedPytree


def clipped(pytree: Any, max_norm: MaxNorm) -> ClippedPytree:
    """Manually assert that ``pytree`` has per-record L2 norm ≤ ``max_norm``."""
    return ClippedPytree(pytree, max_norm)


def noised(pytree: Any, max_norm: MaxNorm, noise_stddev: NoiseStddev) -> NoisedPytree:
    """Manually assert that ``pytree`` already carries noise of the stated σ."""
    return NoisedPytree(pytree, max_norm, noise_stddev)


__all__ = [
    "ClipState", "ClippedPytree", "MaxNorm", "NoiseState", "NoiseStddev", "NoisedPytree",
    "ParamPath", "PerGroup", "SecondMomentClippingOutput", "SecondMomentNoiseOutput",
    "TensorPytree", "clipped", "noised",
]
