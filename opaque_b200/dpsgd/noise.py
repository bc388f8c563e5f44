"""Gaussian noise for DP-SGD.

``gaussian_noise(noise_multiplier=…, key=…)`` returns ``(noise_fn, state)``;
``noise_fn(ClippedPytree, state)`` adds ``N(0, (nm·max_norm)²)`` to every
coordinate and returns a ``NoisedPytree`` that records the realised σ.

Two generators, one contract.  On a B200 the noise is produced on the device by
a counter-based Philox-4x32-10 kernel: the Philox key is the 64-bit seed of the
per-step key ``fold_in(key, step)``, the counter is the coordinate's position
in the flattened tree, so the noise added to a coordinate does not depend on
how coordinates are split over leaves, shards or ranks, and nothing crosses
PCIe.  On CPU (and as the statistical cross-check) uniforms come from a CPU
``torch.Generator`` seeded from the step key and are mapped through
``μ + σ√2·erfinv(2u−1)`` with ``u`` clamped to ``[eps, 1−eps]``.

``bound`` selects the bounded Gaussian mechanism of Chen & Hale: the normal is
renormalised over ``[lo, hi]`` by mapping ``u`` into ``[Φ(lo), Φ(hi)]``.

Parity: packages/opaque-dpsgd/src/opaque/api/dpsgd/noise/_gaussian.py:147-410,
_distributed.py:19-50.
"""
from __future__ import annotations

import dataclasses
import math
from typing import Any

import torch

from ..noise_allocation import (FIRST_MOMENT_FOLD_TAG, SECOND_MOMENT_FOLD_TAG, paired_noise_stddev,
                                per_group_noise_stddev)
from ..pytree import tree_flatten_with_paths, tree_unflatten
from ..random import RngKey, fold_in, generator_from_key
from ..types import (ClippedPytree, NoisedPytree, NoiseState, PerGroup, SecondMomentClippingOutput,
                     SecondMomentNoiseOutput)


@dataclasses.dataclass(frozen=True)
class GaussianNoiseState(NoiseState):
    _step_counter: int
    _rng_key: RngKey


def _check_std(std: Any) -> None:
    vals = list(std.values.values()) if isinstance(std, PerGroup) else [std]
    for v in vals:
        if not math.isfinite(v) or v < 0:
            raise ValueError(f"noise standard deviation must be finite and non-negative, got {v}")


def _resolve_bound(bound: Any):
    if bound is None:
        return None
    if isinstance(bound, (tuple, list)):
        if len(bound) != 2:
            raise ValueError("bound must be a scalar or a (low, high) pair")
        lo, hi = float(bound[0]), float(bound[1])
    else:
        b = float(bound)
        if not b > 0:
            raise ValueError(f"a scalar bound must be > 0, got {bound}")
        lo, hi = -b, b
    if not (lo <= 0.0 <= hi) or lo == hi:
        raise ValueError(f"bound must satisfy low <= 0 <= high with low < high, got ({lo}, {hi})")
    return lo, hi


def _phi(x: float) -> float:
    return 0.5 * (1.0 + math.erf(x / math.sqrt(2.0)))


def sample_gaussian_cpu(x: torch.Tensor, std: float, gen: torch.Generator, bound, compute_dtype: torch.dtype):
    """``x + N(0, std²)`` through the inverse CDF of CPU uniforms (``std == 0`` → ``x``)."""
    if std == 0.0:
        return x
    u = torch.rand(x.shape, generator=gen, dtype=compute_dtype).to(x.device)
    eps = torch.finfo(compute_dtype).eps
    center = x.to(compute_dtype)
    if bound is not None:
        lo, hi = bound
        a = torch.special.ndtr((lo - center) / std)
        b = torch.special.ndtr((hi - center) / std)
        u = a + u * (b - a)
    u = u.clamp(eps, 1.0 - eps)
    out = center + std * math.sqrt(2.0) * torch.erfinv(2.0 * u - 1.0)
    if bound is not None:
        out = out.clamp(bound[0], bound[1])
    return out.to(x.dtype)


def _use_device_philox(x: torch.Tensor, bound) -> bool:
    if not x.is_cuda or bound is not None or x.dtype not in (torch.float32, torch.bfloat16):
        return False
    from ..device import fused_kernels_available
    return fused_kernels_available()


def add_noise_tree(tree: Any, std: Any, step_key: RngKey, bound=None, compute_dtype=torch.float32) -> Any:
    """Add independent Gaussian noise to every tensor leaf (per-group σ by leaf path)."""
    _check_std(std)
    paths, leaves, td = tree_flatten_with_paths(tree)
    gen = None
    offset = 0
    out = []
    for p, x in zip(paths, leaves):
        if not isinstance(x, torch.Tensor):
            if isinstance(std, PerGroup):
                raise TypeError(f"gaussian_noise with PerGroup stddev expects tensor leaves; got {type(x).__name__} at {p!r}")
            out.append(x)
            continue
        s = float(std.for_path(p)) if isinstance(std, PerGroup) else float(std)
        if _use_device_philox(x, bound):
            from .. import ops
            y = x.clone() if s != 0.0 else x
            if s != 0.0:
                ops.philox_normal_add_(y, seed=step_key.seed, offset=offset, std=s)
            out.append(y)
        else:
            if gen is None:
                gen = generator_from_key(step_key)
            out.append(sample_gaussian_cpu(x, s, gen, bound, compute_dtype))
        offset += x.numel()
    return tree_unflatten(td, out)


def gaussian_noise(*, noise_multiplier: float, key: RngKey, bound: Any = None,
                   compute_dtype: torch.dtype = torch.float32):
    """Build ``(noise_fn, GaussianNoiseState)``; the same ``key`` on every rank gives identical noise."""
    nm = float(noise_multiplier)
    if not math.isfinite(nm) or nm < 0:
        raise ValueError(f"noise_multiplier must be finite and non-negative, got {noise_multiplier}")
    if not isinstance(key, RngKey):
        raise TypeError(f"key must be RngKey, got {type(key)}")
    rb = _resolve_bound(bound)

    def stddev_of(c: ClippedPytree):
        if isinstance(c.max_norm, PerGroup):
            return per_group_noise_stddev(c.max_norm, nm)
        std = 0.0 if nm == 0.0 else nm * float(c.max_norm)   # nm = 0 with max_norm = inf must give 0, not NaN
        _check_std(std)
        return std

    def noise_fn(grads: Any, st: GaussianNoiseState):
        with torch.profiler.record_function("opaque::gaussian_noise"):
            nxt = GaussianNoiseState(st._step_counter + 1, st._rng_key)
            if isinstance(grads, SecondMomentClippingOutput):
                g1, g2 = grads.grads, grads.squared_grads
                s1, s2 = paired_noise_stddev(g1.max_norm, g2.max_norm, nm)
                k1 = fold_in(fold_in(st._rng_key, FIRST_MOMENT_FOLD_TAG), st._step_counter)
                k2 = fold_in(fold_in(st._rng_key, SECOND_MOMENT_FOLD_TAG), st._step_counter)
                return SecondMomentNoiseOutput(
                    NoisedPytree(add_noise_tree(g1.pytree, s1, k1, rb, compute_dtype), g1.max_norm, s1),
                    NoisedPytree(add_noise_tree(g2.pytree, s2, k2, rb, compute_dtype), g2.max_norm, s2)), nxt
            if isinstance(grads, NoisedPytree):
                raise TypeError("gaussian_noise expects ClippedPytree inputs, not values that already carry noise")
            if not isinstance(grads, ClippedPytree):
                raise TypeError("gaussian_noise expects ClippedPytree inputs; wrap manual values with types.clipped(...)")
            std = stddev_of(grads)
            step_key = fold_in(st._rng_key, st._step_counter)
            return NoisedPytree(add_noise_tree(grads.pytree, std, step_key, rb, compute_dtype),
                                grads.max_norm, std), nxt

    return noise_fn, GaussianNoiseState(0, key)


def sync_gaussian_noise_state(state: GaussianNoiseState) -> GaussianNoiseState:
    """All ranks must hold the same step counter and seed (checked through one packed reduce)."""
    from ..distributed import assert_scalar_equal, assert_string_equal, is_distributed
    if is_distributed():
        assert_scalar_equal(state._step_counter, name="GaussianNoiseState._step_counter")
        assert_string_equal(f"{state._rng_key.seed}:{state._rng_key.impl}", name="GaussianNoiseState._rng_key")
    return state


from ..distributed import register_sync_type as _rst  # noqa: E402

_rst(GaussianNoiseState, sync_gaussian_noise_state)

__all__ = ["GaussianNoiseState", "add_noise_tree", "gaussian_noise", "sample_gaussian_cpu",
           "sync_gaussian_noise_state"]

from ..utils.namespaces import submodule as _sub  # noqa: E402


def _register_type_namespace() -> None:
    from .. import _type_names as T
    _sub(__name__, "types", "Types of the Gaussian noise mechanism.",
         {"GaussianNoiseFn": T.GaussianNoiseFn, "GaussianNoiseInput": T.GaussianNoiseInput, "GaussianNoiseOutput": T.GaussianNoiseOutput,
          "GaussianNoiseState": GaussianNoiseState}, bind=False)


_register_type_namespace()
