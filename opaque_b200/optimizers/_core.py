"""Gradient-transformation chain owned by the framework (no torchopt dependency).

A ``GradientTransformation`` is ``(init, update)`` with
``update(updates, state, *, params=None, **extra) -> (new_updates, new_state)``.
``make_optimizer_chain`` turns a *moment scaler* into a full optimizer and is
the only place DP metadata is unwrapped: it accepts ``NoisedPytree`` (routing
``noise_stddev`` to scalers that want it) and ``SecondMomentNoiseOutput``
(routing the privatised Σg² stream), and it REJECTS a bare ``ClippedPytree`` —
gradients that never met a noise mechanism must not reach an optimizer.

Parity: packages/opaque-optimizers/src/opaque/api/optimizers/_chain.py:37-248,
_bias_correction.py:52-160.
"""
from __future__ import annotations

import inspect
from collections.abc import Callable
from typing import Any, NamedTuple, Union

import torch

from ..pytree import tree_flatten_with_paths, tree_leaves, tree_map, tree_unflatten
from ..types import ClippedPytree, NoisedPytree, PerGroup, SecondMomentNoiseOutput

LR = Union[float, Callable[[int], float]]


class GradientTransformation(NamedTuple):
    init: Callable[[Any], Any]
    update: Callable[..., tuple[Any, Any]]


def lr_at(lr: LR, step: int) -> float:
    return float(lr(step)) if callable(lr) else float(lr)


def zeros_like_tree(params: Any, dtype: torch.dtype | None = None) -> Any:
    return tree_map(lambda p: torch.zeros_like(p, dtype=dtype or p.dtype) if isinstance(p, torch.Tensor) else p, params)


def map_leaves_with_path(fn: Callable, tree: Any, *rest: Any) -> Any:
    """``fn(path, leaf, *others)`` over tensor leaves."""
    paths, leaves, td = tree_flatten_with_paths(tree)
    others = [tree_leaves(r) for r in rest]
    return tree_unflatten(td, [fn(p, x, *(o[i] for o in others)) for i, (p, x) in enumerate(zip(paths, leaves))])


def apply_updates(params: Any, updates: Any, *, inplace: bool = False) -> Any:
    """``params + updates`` leaf-wise (the update is cast to the parameter dtype)."""
    def add(p, u):
        if not isinstance(p, torch.Tensor) or u is None:
            return p
        if inplace:
            p.add_(u.to(p.dtype))
            return p
        return p + u.to(p.dtype)
    return tree_map(add, params, updates)


# ---- noise bias correction ---------------------------------------------------------------

def resolve_noise_variance(noise_stddev: Any):
    """σ² as a float, a ``{group: σ²}`` PerGroup, or None when no σ was published."""
    if noise_stddev is None:
        return None
    if isinstance(noise_stddev, PerGroup):
        return noise_stddev * noise_stddev
    return float(noise_stddev) ** 2


def init_phi(noise_like: Any = None):
    return 0.0


def update_phi_ema(phi: Any, variance: Any, decay: float):
    """``φ ← decay·φ + (1−decay)·σ²`` for a scalar or per-group σ²."""
    if variance is None:
        return phi
    if isinstance(variance, PerGroup):
        old = phi.values if isinstance(phi, PerGroup) else {g: float(phi or 0.0) for g in variance.values}
        return PerGroup(variance.groups, {g: decay * old.get(g, 0.0) + (1 - decay) * v for g, v in variance.values.items()})
    base = phi.effective if isinstance(phi, PerGroup) else float(phi or 0.0)
    return decay * base + (1 - decay) * variance


def accumulate_phi(phi: Any, variance: Any):
    """``φ ← φ + σ²`` (Adagrad-style running sums)."""
    if variance is None:
        return phi
    if isinstance(variance, PerGroup):
        old = phi.values if isinstance(phi, PerGroup) else {g: float(phi or 0.0) for g in variance.values}
        return PerGroup(variance.groups, {g: old.get(g, 0.0) + v for g, v in variance.values.items()})
    return float(phi or 0.0) + variance


def phi_for(phi: Any, path: Any) -> float:
    return float(phi.for_path(path)) if isinstance(phi, PerGroup) else float(phi or 0.0)


def debias_second_moment(v_hat: torch.Tensor, phi_hat: float) -> torch.Tensor:
    """``v̂ − φ̂`` where that is positive, else ``v̂`` (noise floor removed from the denominator)."""
    if phi_hat == 0.0:
        return v_hat
    corrected = v_hat - phi_hat
    return torch.where(corrected > 0, corrected, v_hat)


# ---- chain ---------------------------------------------------------------------------------

def _global_rms(tree: Any) -> float:
    total, count = 0.0, 0
    for x in tree_leaves(tree):
        if isinstance(x, torch.Tensor):
            total += float(x.detach().double().square().sum())
            count += x.numel()
    return (total / max(count, 1)) ** 0.5


def clip_by_global_rms(updates: Any, threshold: float) -> Any:
    """StableAdamW: divide by ``max(1, rms/threshold)`` with the RMS taken model-wide in fp64."""
    denom = max(1.0, _global_rms(updates) / threshold)
    if denom == 1.0:
        return updates
    return tree_map(lambda u: u / denom if isinstance(u, torch.Tensor) else u, updates)


def _accepts(fn: Callable, name: str) -> bool:
    ps = inspect.signature(fn).parameters
    return name in ps or any(p.kind is inspect.Parameter.VAR_KEYWORD for p in ps.values())


def unwrap_updates(updates: Any, *, want_stddev: bool, want_second: bool) -> tuple[Any, dict[str, Any]]:
    """Strip DP wrappers, returning the raw tree and the metadata kwargs for the moment scaler."""
    if isinstance(updates, SecondMomentNoiseOutput):
        first, second = updates.noisy_grads, updates.noisy_squared_grads
        for name, v in (("noisy_grads", first), ("noisy_squared_grads", second)):
            if isinstance(v, ClippedPytree) and not isinstance(v, NoisedPytree):
                raise TypeError(f"SecondMomentNoiseOutput.{name} is a ClippedPytree that has not passed through a noise mechanism.")
        if not want_second:
            raise TypeError("this optimizer has no private-second-moment branch; pass the first stream only")
        kw: dict[str, Any] = {"noisy_squared_grads": second.pytree if isinstance(second, NoisedPytree) else second}
        if want_stddev and isinstance(first, NoisedPytree):
            kw["noise_stddev"] = first.noise_stddev
        return (first.pytree if isinstance(first, NoisedPytree) else first), kw
    if isinstance(updates, NoisedPytree):
        return updates.pytree, ({"noise_stddev": updates.noise_stddev} if want_stddev else {})
    if isinstance(updates, ClippedPytree):
        raise TypeError(
            "optimizer.update() received ClippedPytree updates that have not passed through a noise mechanism. "
            "Pass NoisedPytree outputs from a DP mechanism, or unwrap `.pytree` explicitly for non-private use.")
    return updates, {}


class ChainState(NamedTuple):
    moment: Any
    step: int


def make_optimizer_chain(moment_scaler: GradientTransformation, lr: LR, weight_decay: float, *,
                         decoupled_weight_decay: bool = True, update_rms_clip: float | None = None,
                         maximize: bool = False) -> GradientTransformation:
    """decoupled: scaler → [rms clip] → +wd·p → ×(−lr);  L2: +wd·p → scaler → [rms clip] → ×(−lr)."""
    if weight_decay < 0:
        raise ValueError("weight_decay must be >= 0")
    if update_rms_clip is not None and update_rms_clip <= 0:
        raise ValueError("update_rms_clip must be > 0")
    want_std = _accepts(moment_scaler.update, "noise_stddev")
    want_sq = _accepts(moment_scaler.update, "noisy_squared_grads")

    def init(params: Any) -> ChainState:
        return ChainState(moment_scaler.init(params), 0)

    def update(updates: Any, state: ChainState, *, params: Any = None):
        raw, kw = unwrap_updates(updates, want_stddev=want_std, want_second=want_sq)
        if maximize:
            raw = tree_map(lambda g: -g if isinstance(g, torch.Tensor) else g, raw)
        if weight_decay and params is None:
            raise ValueError("weight decay needs `params=`")
        if weight_decay and not decoupled_weight_decay:
            raw = tree_map(lambda g, p: g + weight_decay * p.to(g.dtype), raw, params)
        scaled, moment = moment_scaler.update(raw, state.moment, params=params, **kw)
        if update_rms_clip is not None:
            scaled = clip_by_global_rms(scaled, update_rms_clip)
        if weight_decay and decoupled_weight_decay:
            scaled = tree_map(lambda u, p: u + weight_decay * p.to(u.dtype), scaled, params)
        rate = lr_at(lr, state.step)
        return tree_map(lambda u: -rate * u if isinstance(u, torch.Tensor) else u, scaled), ChainState(moment, state.step + 1)

    return GradientTransformation(init, update)
