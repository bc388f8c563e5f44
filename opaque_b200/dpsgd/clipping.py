"""DP-SGD clipping front-ends: fixed, AUTO-S, per-group and adaptive (quantile-tracking).

Adaptive clipping (Andrew et al.): after each step the threshold moves
geometrically toward the target quantile of per-example gradient norms,
``C ← clamp(C·exp(η·(ρ̃ − γ)), C_min, C_max)`` with ``ρ`` the fraction of
examples whose norm exceeded ``C`` and ``ρ̃ = ρ + fraction_noise_std·N(0,1)``;
the normal draw comes from ``generator_from_key(fold_in(key, step))``.  Under
data parallelism the clipped / total counts are summed over ranks before the
update and every rank uses the same key, so the new threshold is identical
everywhere.  The accountant pays for the noisy fraction through ``adaclip``.

Parity: packages/opaque-dpsgd/src/opaque/api/dpsgd/clipping/_adaptive.py:88-642,
_distributed.py:53-133; engine re-exports.
"""
from __future__ import annotations

import dataclasses
import math
from collections.abc import Callable
from typing import Any

import torch

from ..engine.clipping import (AutoClipState, ClippedGradAux, ClippingStats, FixedClipState, auto_clipped_fun,
                               auto_clipped_grad, clip_pytree, clipped_fun, clipped_grad, per_group)
from ..random import RngKey, fold_in, generator_from_key
from ..types import ClipState, PerGroup


@dataclasses.dataclass(frozen=True)
class AdaptiveClipState(ClipState):
    clipping_norm: Any                  # float | PerGroup — threshold for the NEXT step
    step: int
    target_quantile: float
    learning_rate: float
    clipping_norm_min: float
    clipping_norm_max: float
    fraction_noise_std: float
    _rng_key: RngKey
    _num_clipped: Any = 0.0             # local counts from the last step (summed across ranks by sync)
    _batch_size: int = 0
    _prev_clipping_norm: Any = None     # threshold the last step was clipped at


def next_clipping_norm(c: float, rate: float, noise: float, st: AdaptiveClipState) -> float:
    """One geometric quantile-tracking update of a scalar threshold."""
    noisy = rate + st.fraction_noise_std * noise
    new = c * math.exp(st.learning_rate * (noisy - st.target_quantile))
    return min(max(new, st.clipping_norm_min), st.clipping_norm_max)


def _draws(key: RngKey, step: int, names: list[str]) -> dict[str, float]:
    if len(names) == 1 and names[0] == "":
        g = generator_from_key(fold_in(key, step))
        return {"": float(torch.randn(1, generator=g))}
    return {n: float(torch.randn(1, generator=generator_from_key(fold_in(fold_in(key, step), n)))) for n in names}


def _updated(st: AdaptiveClipState, used: Any, num_clipped: Any, batch: int, step_for_key: int) -> Any:
    if batch <= 0:
        return used
    if isinstance(used, PerGroup):
        z = _draws(st._rng_key, step_for_key, sorted(used.values))
        vals = {g: next_clipping_norm(v, float(num_clipped.get(g, 0.0)) / batch, z[g], st) for g, v in used.values.items()}
        return PerGroup(used.groups, vals)
    z = _draws(st._rng_key, step_for_key, [""])[""]
    return next_clipping_norm(float(used), float(num_clipped) / batch, z, st)


def adaptive_clipped_grad(loss_fn: Callable, argnums=0, has_aux: bool = False, *,
                          initial_clipping_norm: float | PerGroup = 0.1, target_quantile: float = 0.5,
                          learning_rate: float = 0.2, clipping_norm_min: float = 0.01,
                          clipping_norm_max: float = 100.0, fraction_noise_std: float = 0.05, key: RngKey,
                          return_aux: bool = False, return_stats: bool = False,
                          pre_clipping_transform: Callable = lambda x: x, **clipped_grad_kwargs: Any):
    """Quantile-tracking adaptive clipping; the state carries the live threshold."""
    if not 0.0 < target_quantile < 1.0:
        raise ValueError("target_quantile must be in (0, 1)")
    if not 0 < clipping_norm_min <= clipping_norm_max:
        raise ValueError("need 0 < clipping_norm_min <= clipping_norm_max")
    if fraction_noise_std < 0:
        raise ValueError("fraction_noise_std must be >= 0")
    if not isinstance(key, RngKey):
        raise TypeError(f"key must be RngKey, got {type(key)}")
    state0 = AdaptiveClipState(initial_clipping_norm, 0, target_quantile, learning_rate, clipping_norm_min,
                               clipping_norm_max, fraction_noise_std, key)

    def grad_fn(*args: Any, state: AdaptiveClipState = state0):
        with torch.profiler.record_function("opaque::adaptive_clipped_grad"):
            c = state.clipping_norm
            inner, _ = clipped_grad(loss_fn, argnums, has_aux, clipping_norm=c, return_aux=return_aux,
                                    return_stats=not return_aux, pre_clipping_transform=pre_clipping_transform,
                                    _range_name="opaque::clipped_grad", **clipped_grad_kwargs)
            (tree, extra), _ = inner(*args, state=FixedClipState())
            if return_aux:
                n = extra.batch_size
                if isinstance(c, PerGroup):
                    num = {g: float((extra.group_norms[g] > c.values[g]).sum()) for g in c.values} if n else {g: 0.0 for g in c.values}
                else:
                    num = float((extra.grad_norms > float(c)).sum()) if n else 0.0
            else:
                n, num = extra.batch_size, extra.num_clipped
            nxt = _updated(state, c, num, n, state.step)
            new_state = dataclasses.replace(state, clipping_norm=nxt, step=state.step + 1, _num_clipped=num,
                                            _batch_size=n, _prev_clipping_norm=c)
            if return_aux or return_stats:
                return (tree, extra), new_state
            return tree, new_state

    return grad_fn, state0


def sync_adaptive_clip_state(state: AdaptiveClipState) -> AdaptiveClipState:
    """Redo the last threshold update from cluster-wide counts (same ``step − 1`` key on every rank)."""
    from ..distributed import is_distributed, reduce_scalar
    if not is_distributed() or state.step == 0:
        return state
    used = state._prev_clipping_norm
    n = int(reduce_scalar(int(state._batch_size), "sum"))
    if isinstance(used, PerGroup):
        num = {g: float(reduce_scalar(float(state._num_clipped.get(g, 0.0) if isinstance(state._num_clipped, dict) else 0.0), "sum"))
               for g in sorted(used.values)}
    else:
        num = float(reduce_scalar(float(state._num_clipped), "sum"))
    nxt = _updated(state, used, num, n, state.step - 1)
    return dataclasses.replace(state, clipping_norm=nxt, _num_clipped=num, _batch_size=n)


from ..distributed import register_sync_type as _rst  # noqa: E402

_rst(AdaptiveClipState, sync_adaptive_clip_state)
_rst(FixedClipState, lambda s: s)
_rst(AutoClipState, lambda s: s)


def _sync_aux(aux: ClippedGradAux) -> ClippedGradAux:
    """Gather per-example diagnostics from all ranks with tensor collectives (no pickling)."""
    from ..distributed import gather_tensors, is_distributed, reduce_scalar
    if not is_distributed():
        return aux
    def g(x):
        return gather_tensors(x) if isinstance(x, torch.Tensor) else x
    n = int(reduce_scalar(int(aux.batch_size), "sum"))
    rate = aux.clipping_rate
    if isinstance(rate, dict):
        rate = {k: (float(reduce_scalar(float(v) * aux.batch_size, "sum")) / n if n else None) for k, v in sorted(rate.items())}
    else:
        tot = float(reduce_scalar(float(rate or 0.0) * aux.batch_size, "sum"))
        rate = tot / n if n else None
    gn = None if aux.group_norms is None else {k: g(v) for k, v in sorted(aux.group_norms.items())}
    return dataclasses.replace(aux, loss_values=g(aux.loss_values), grad_norms=g(aux.grad_norms),
                               clipped_grad_norms=g(aux.clipped_grad_norms), clipping_rate=rate, batch_size=n,
                               group_norms=gn)


def _sync_stats(s: ClippingStats) -> ClippingStats:
    from ..distributed import is_distributed, reduce_scalar
    if not is_distributed():
        return s
    n = int(reduce_scalar(int(s.batch_size), "sum"))
    if isinstance(s.num_clipped, dict):
        num = {k: float(reduce_scalar(float(v), "sum")) for k, v in sorted(s.num_clipped.items())}
        rate = {k: (v / n if n else None) for k, v in num.items()}
    else:
        num = float(reduce_scalar(float(s.num_clipped), "sum"))
        rate = num / n if n else None
    fin = bool(reduce_scalar(int(s.all_finite), "min"))
    return ClippingStats(num, rate, n, fin)


_rst(ClippedGradAux, _sync_aux)
_rst(ClippingStats, _sync_stats)

__all__ = ["AdaptiveClipState", "AutoClipState", "FixedClipState", "adaptive_clipped_grad", "auto_clipped_fun",
           "auto_clipped_grad", "clip_pytree", "clipped_fun", "clipped_grad", "next_clipping_norm", "per_group",
           "sync_adaptive_clip_state"]

from ..engine import clipping as _eng  # noqa: E402
from ..utils.namespaces import submodule as _sub  # noqa: E402


def _register_type_namespaces() -> None:
    from .. import _type_names as T
    fun = {"auto_clipped_fun": auto_clipped_fun, "auto_scale_pytree": _eng.auto_scale_pytree, "clip_pytree": clip_pytree, "clipped_fun": clipped_fun}
    common = {"AutoClipState": AutoClipState, "FixedClipState": FixedClipState, "AutoClippedFunAux": T.AutoClippedFunAux,
              "AutoClippedGradAux": T.AutoClippedGradAux, "ClippedGradFn": T.ClippedGradFn, "ClippedGradResult": T.ClippedGradResult}
    _sub(__name__, "fun", "Clipping of arbitrary per-example functions and of pytrees.", fun, bind=False)
    _sub(__name__, "types", "State and result types of the clipping transforms.",
         {**common, "AdaptiveClipState": AdaptiveClipState, "AdaptiveClippedGradAux": T.AdaptiveClippedGradAux, "ClippingStats": _eng.ClippingStats,
          "ClipPytreeAux": _eng.ClipPytreeAux, "ClippedFunAux": _eng.ClippedFunAux, "ClippedGradAux": _eng.ClippedGradAux}, bind=False)
    # the DP-FTRL façade re-exports this module as ``dpftrl.clipping``: same namespaces under that path
    for name in ("fun", "types"):
        import sys
        sys.modules["opaque_b200.dpftrl.clipping." + name] = sys.modules[__name__ + "." + name]


_register_type_namespaces()
