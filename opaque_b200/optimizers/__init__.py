"""DP-aware optimizers as pure ``(init, update)`` pairs.

Every factory returns a ``GradientTransformation`` built by
``make_optimizer_chain``; ``optimizer.update(noised, state, params=params)``
returns ``(updates, new_state)`` and ``apply_updates`` adds them.  With
``noise_bias_correction=True`` the second-moment optimizers keep ``φ``, a
running copy of the injected noise variance with the SAME averaging rule as
their second moment, and use ``v̂ − φ̂`` (where positive) in the denominator:
DP noise inflates ``E[g²]`` by exactly ``σ²``, and removing it restores the
signal-driven step size (AdamW-BC).  If a privatised ``Σg²`` stream is supplied
(``SecondMomentNoiseOutput``) Adam uses it directly instead.

Parity: packages/opaque-optimizers/src/opaque/api/optimizers/_adam.py:91-384 and the
sibling modules _sgd / _lion / _adagrad / _rmsprop / _radam / _adadelta / _adafactor /
_ademamix / _schedule_free; distributed.py:85-211.
"""
from __future__ import annotations

import dataclasses
import math
from typing import Any, NamedTuple

import torch

from ..pytree import tree_leaves, tree_map
from ..types import NoisedPytree
from . import _core as types  # noqa: F401  (``optimizers.types`` namespace of the reference)
from ._core import (LR, ChainState, GradientTransformation, accumulate_phi, apply_updates, clip_by_global_rms,
                    debias_second_moment, lr_at, make_optimizer_chain, map_leaves_with_path, phi_for,
                    resolve_noise_variance, unwrap_updates, update_phi_ema, zeros_like_tree)


def _f32(params):
    return zeros_like_tree(params, torch.float32)


def _up(g: torch.Tensor) -> torch.Tensor:
    return g.float() if g.dtype in (torch.bfloat16, torch.float16) else g


# ------------------------------------------------------------------------------------------ SGD

class SGDState(NamedTuple):
    momentum: Any
    step: int


def sgd(lr: LR = 1e-3, momentum: float = 0.0, dampening: float = 0.0, weight_decay: float = 0.0,
        nesterov: bool = False, *, moment_requires_grad: bool = False, maximize: bool = False):
    """SGD with optional (Nesterov) momentum and L2 weight decay, PyTorch semantics."""
    if nesterov and (momentum <= 0 or dampening != 0):
        raise ValueError("Nesterov momentum requires momentum > 0 and zero dampening")

    def init(params):
        return SGDState(_f32(params) if momentum else None, 0)

    def update(grads, state: SGDState, *, params=None):
        if state.momentum is None:
            return tree_map(_up, grads), SGDState(None, state.step + 1)
        first = state.step == 0
        buf = tree_map(lambda b, g: _up(g).clone() if first else momentum * b + (1 - dampening) * _up(g), state.momentum, grads)
        out = tree_map(lambda g, b: _up(g) + momentum * b, grads, buf) if nesterov else buf
        return out, SGDState(buf, state.step + 1)

    return make_optimizer_chain(GradientTransformation(init, update), lr, weight_decay,
                                decoupled_weight_decay=False, maximize=maximize)


# ------------------------------------------------------------------------------------------ Adam

@dataclasses.dataclass(frozen=True)
class AdamState:
    mu: Any
    nu: Any
    phi: Any
    step: int


def scale_by_adam(b1: float, b2: float, eps: float, noise_bias_correction: bool = False, bc_floor: float | None = None):
    """Adam direction ``m̂/(√v_eff + eps)`` with three second-moment branches.

    private   – ``v`` tracks a separately privatised ``Σg²`` stream; ``v_eff = v̂`` where positive,
                else ``m̂²``, floored at ``eps²``.
    corrected – ``φ ← b2·φ + (1−b2)·σ²``; ``v_eff = v̂ − φ̂`` where positive, else ``v̂``.
    vanilla   – ``v_eff = v̂``.
    """
    floor = eps * eps if bc_floor is None else bc_floor

    def init(params):
        return AdamState(_f32(params), _f32(params), 0.0, 0)

    def update(grads, state: AdamState, *, params=None, noise_stddev=None, noisy_squared_grads=None):
        t = state.step + 1
        c1, c2 = 1 - b1 ** t, 1 - b2 ** t
        mu = tree_map(lambda m, g: b1 * m + (1 - b1) * _up(g), state.mu, grads)
        if noisy_squared_grads is not None:
            nu = tree_map(lambda v, s: b2 * v + (1 - b2) * _up(s), state.nu, noisy_squared_grads)

            def direction(path, m, v):
                m_hat, v_hat = m / c1, v / c2
                v_eff = torch.where(v_hat > 0, v_hat, m_hat * m_hat).clamp(min=floor)
                return m_hat / (v_eff.sqrt() + eps)
            return map_leaves_with_path(direction, mu, nu), AdamState(mu, nu, state.phi, t)
        nu = tree_map(lambda v, g: b2 * v + (1 - b2) * _up(g) ** 2, state.nu, grads)
        phi = update_phi_ema(state.phi, resolve_noise_variance(noise_stddev), b2) if noise_bias_correction else state.phi

        def direction(path, m, v):
            v_hat = v / c2
            if noise_bias_correction:
                v_hat = debias_second_moment(v_hat, phi_for(phi, path) / c2)
            return (m / c1) / (v_hat.sqrt() + eps)
        return map_leaves_with_path(direction, mu, nu), AdamState(mu, nu, phi, t)

    return GradientTransformation(init, update)


def adam(lr: LR = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0, *,
         update_rms_clip: float | None = None, noise_bias_correction: bool = False):
    """Adam with L2 weight decay folded into the gradient."""
    return make_optimizer_chain(scale_by_adam(betas[0], betas[1], eps, noise_bias_correction), lr, weight_decay,
                                decoupled_weight_decay=False, update_rms_clip=update_rms_clip)


def adamw(lr: LR = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01, *,
          decoupled_weight_decay: bool = True, update_rms_clip: float | None = None,
          noise_bias_correction: bool = False):
    """AdamW; ``noise_bias_correction=True`` is AdamW-BC."""
    return make_optimizer_chain(scale_by_adam(betas[0], betas[1], eps, noise_bias_correction), lr, weight_decay,
                                decoupled_weight_decay=decoupled_weight_decay, update_rms_clip=update_rms_clip)


# ------------------------------------------------------------------------------------------ Lion

@dataclasses.dataclass(frozen=True)
class LionState:
    mu: Any
    step: int


def lion(lr: LR = 1e-4, betas=(0.9, 0.99), weight_decay: float = 0.0, *, decoupled_weight_decay: bool = True):
    """Lion: ``sign(b1·m + (1−b1)·g)``; ``m ← b2·m + (1−b2)·g``."""
    b1, b2 = betas

    def init(params):
        return LionState(_f32(params), 0)

    def update(grads, state, *, params=None):
        out = tree_map(lambda m, g: torch.sign(b1 * m + (1 - b1) * _up(g)), state.mu, grads)
        mu = tree_map(lambda m, g: b2 * m + (1 - b2) * _up(g), state.mu, grads)
        return out, LionState(mu, state.step + 1)

    return make_optimizer_chain(GradientTransformation(init, update), lr, weight_decay,
                                decoupled_weight_decay=decoupled_weight_decay)


# ------------------------------------------------------------------------------------------ Adagrad

@dataclasses.dataclass(frozen=True)
class AdagradState:
    sum_sq: Any
    phi: Any
    step: int


def adagrad(lr: LR = 1e-2, eps: float = 1e-10, weight_decay: float = 0.0, initial_accumulator_value: float = 0.0, *,
            decoupled_weight_decay: bool = True, noise_bias_correction: bool = False):
    """Adagrad; the bias correction subtracts the accumulated ``Σσ²`` from ``Σg²``."""
    def init(params):
        return AdagradState(tree_map(lambda p: torch.full_like(p, initial_accumulator_value, dtype=torch.float32), params), 0.0, 0)

    def update(grads, state, *, params=None, noise_stddev=None):
        acc = tree_map(lambda a, g: a + _up(g) ** 2, state.sum_sq, grads)
        phi = accumulate_phi(state.phi, resolve_noise_variance(noise_stddev)) if noise_bias_correction else state.phi

        def direction(path, g, a):
            a_eff = debias_second_moment(a, phi_for(phi, path)) if noise_bias_correction else a
            return _up(g) / (a_eff.sqrt() + eps)
        return map_leaves_with_path(direction, grads, acc), AdagradState(acc, phi, state.step + 1)

    return make_optimizer_chain(GradientTransformation(init, update), lr, weight_decay,
                                decoupled_weight_decay=decoupled_weight_decay)


# ------------------------------------------------------------------------------------------ RMSprop

@dataclasses.dataclass(frozen=True)
class RMSpropState:
    nu: Any
    phi: Any
    step: int


def rmsprop(lr: LR = 1e-2, alpha: float = 0.99, eps: float = 1e-8, weight_decay: float = 0.0, *,
            decoupled_weight_decay: bool = True, update_rms_clip: float | None = None,
            noise_bias_correction: bool = False):
    """RMSprop with optional momentum and centring."""
    def init(params):
        return RMSpropState(_f32(params), 0.0, 0)

    def update(grads, state, *, params=None, noise_stddev=None):
        nu = tree_map(lambda v, g: alpha * v + (1 - alpha) * _up(g) ** 2, state.nu, grads)
        phi = update_phi_ema(state.phi, resolve_noise_variance(noise_stddev), alpha) if noise_bias_correction else state.phi

        def direction(path, g, v):
            v_eff = debias_second_moment(v, phi_for(phi, path)) if noise_bias_correction else v
            return _up(g) / (v_eff.sqrt() + eps)
        return map_leaves_with_path(direction, grads, nu), RMSpropState(nu, phi, state.step + 1)

    return make_optimizer_chain(GradientTransformation(init, update), lr, weight_decay,
                                decoupled_weight_decay=decoupled_weight_decay, update_rms_clip=update_rms_clip)


# ------------------------------------------------------------------------------------------ RAdam

@dataclasses.dataclass(frozen=True)
class RAdamState:
    mu: Any
    nu: Any
    phi: Any
    step: int


def _rectification(b2: float, t: int) -> float | None:
    rho_inf = 2.0 / (1.0 - b2) - 1.0
    rho_t = rho_inf - 2.0 * t * b2 ** t / (1.0 - b2 ** t)
    if rho_t <= 5.0:
        return None
    return math.sqrt((rho_t - 4) * (rho_t - 2) * rho_inf / ((rho_inf - 4) * (rho_inf - 2) * rho_t))


def radam(lr: LR = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0, *,
          decoupled_weight_decay: bool = False, update_rms_clip: float | None = None,
          noise_bias_correction: bool = False):
    """Rectified Adam: plain momentum until the variance estimate is trustworthy."""
    b1, b2 = betas

    def init(params):
        return RAdamState(_f32(params), _f32(params), 0.0, 0)

    def update(grads, state, *, params=None, noise_stddev=None):
        t = state.step + 1
        mu = tree_map(lambda m, g: b1 * m + (1 - b1) * _up(g), state.mu, grads)
        nu = tree_map(lambda v, g: b2 * v + (1 - b2) * _up(g) ** 2, state.nu, grads)
        phi = update_phi_ema(state.phi, resolve_noise_variance(noise_stddev), b2) if noise_bias_correction else state.phi
        rect = _rectification(b2, t)
        c1, c2 = 1 - b1 ** t, 1 - b2 ** t

        def direction(path, m, v):
            m_hat = m / c1
            if rect is None:
                return m_hat
            v_hat = v / c2
            if noise_bias_correction:
                v_hat = debias_second_moment(v_hat, phi_for(phi, path) / c2)
            return rect * m_hat / (v_hat.sqrt() + eps)
        return map_leaves_with_path(direction, mu, nu), RAdamState(mu, nu, phi, t)

    return make_optimizer_chain(GradientTransformation(init, update), lr, weight_decay,
                                decoupled_weight_decay=decoupled_weight_decay, update_rms_clip=update_rms_clip)


# ------------------------------------------------------------------------------------------ Adadelta

@dataclasses.dataclass(frozen=True)
class AdadeltaState:
    sq_avg: Any
    acc_delta: Any
    phi: Any
    step: int


def adadelta(lr: LR = 1.0, rho: float = 0.9, eps: float = 1e-6, weight_decay: float = 0.0, *,
             decoupled_weight_decay: bool = True, update_rms_clip: float | None = None,
             noise_bias_correction: bool = False):
    """Adadelta (running averages of squared gradients and squared updates)."""
    def init(params):
        return AdadeltaState(_f32(params), _f32(params), 0.0, 0)

    def update(grads, state, *, params=None, noise_stddev=None):
        sq = tree_map(lambda s, g: rho * s + (1 - rho) * _up(g) ** 2, state.sq_avg, grads)
        phi = update_phi_ema(state.phi, resolve_noise_variance(noise_stddev), rho) if noise_bias_correction else state.phi

        def direction(path, g, s, d):
            s_eff = debias_second_moment(s, phi_for(phi, path)) if noise_bias_correction else s
            return _up(g) * (d + eps).sqrt() / (s_eff + eps).sqrt()
        delta = map_leaves_with_path(direction, grads, sq, state.acc_delta)
        acc = tree_map(lambda d, u: rho * d + (1 - rho) * u ** 2, state.acc_delta, delta)
        return delta, AdadeltaState(sq, acc, phi, state.step + 1)

    return make_optimizer_chain(GradientTransformation(init, update), lr, weight_decay,
                                decoupled_weight_decay=decoupled_weight_decay, update_rms_clip=update_rms_clip)


# ------------------------------------------------------------------------------------------ Adafactor

@dataclasses.dataclass(frozen=True)
class AdafactorState:
    v_row: Any
    v_col: Any
    v_full: Any
    mu: Any
    phi: Any
    step: int


def adafactor(lr: LR = 1e-3, beta1: float = 0.0, decay_rate: float = -0.8, eps_grad: float = 1e-30,
              eps_root: float = 1e-3, weight_decay: float = 0.0, update_rms_clip: float = 1.0, *,
              decoupled_weight_decay: bool = True, noise_bias_correction: bool = False):
    """Adafactor: matrices keep row / column second-moment factors (``β₂_t = 1 − t^decay_rate``), floors are relative to each
    tensor's own scale (``eps_root``), and the whole update is clipped to a global RMS of ``update_rms_clip``.

    Parity: packages/opaque-optimizers/src/opaque/api/optimizers/_adafactor.py:150-290."""
    def factored(p):
        return isinstance(p, torch.Tensor) and p.ndim >= 2

    def init(params):
        row = tree_map(lambda p: torch.zeros(p.shape[:-1], dtype=torch.float32, device=p.device) if factored(p) else torch.zeros((), device=p.device), params)
        col = tree_map(lambda p: torch.zeros(p.shape[:-2] + p.shape[-1:], dtype=torch.float32, device=p.device) if factored(p) else torch.zeros((), device=p.device), params)
        full = tree_map(lambda p: torch.zeros((), device=p.device) if factored(p) else torch.zeros_like(p, dtype=torch.float32), params)
        mu = _f32(params) if beta1 > 0 else None
        return AdafactorState(row, col, full, mu, 0.0, 0)

    def update(grads, state, *, params=None, noise_stddev=None):
        t = state.step + 1
        beta2 = 1.0 - t ** decay_rate
        var = resolve_noise_variance(noise_stddev)
        phi = update_phi_ema(state.phi, var, beta2) if noise_bias_correction else state.phi
        new_row, new_col, new_full, outs = [], [], [], []
        from ..pytree import tree_flatten_with_paths, tree_unflatten
        paths, gl, td = tree_flatten_with_paths(grads)
        rows, cols, fulls = tree_leaves(state.v_row), tree_leaves(state.v_col), tree_leaves(state.v_full)

        def floor_scaled(v):         # sqrt(v) with a floor RELATIVE to the tensor's own scale: eps_root · sqrt(mean v)
            return v.sqrt().clamp(min=eps_root * v.mean().clamp(min=1e-30).sqrt())
        for path, g, r, c, f in zip(paths, gl, rows, cols, fulls):
            g = _up(g)
            sq = g * g + eps_grad
            ph = phi_for(phi, path) if noise_bias_correction else 0.0
            if factored(g):
                r = beta2 * r + (1 - beta2) * sq.mean(dim=-1)
                c = beta2 * c + (1 - beta2) * sq.mean(dim=-2)
                # the noise floor is removed from each factor (both estimate E[g²] along their axis), then
                # v̂ ≈ row ⊗ col / mean(row), the mean floored relative to the factor's scale
                r_eff, c_eff = debias_second_moment(r, ph), debias_second_moment(c, ph)
                r_mean = r_eff.mean(dim=-1, keepdim=True).clamp(min=eps_root * r_eff.mean().clamp(min=1e-30))
                v_hat = (r_eff / r_mean).unsqueeze(-1) * c_eff.unsqueeze(-2)
            else:
                f = beta2 * f + (1 - beta2) * sq
                v_hat = debias_second_moment(f, ph)
            outs.append(g / floor_scaled(v_hat))
            new_row.append(r); new_col.append(c); new_full.append(f)
        # ONE clip factor for the whole update: its parameter-count-weighted RMS is brought down to update_rms_clip
        total = sum(float(u.double().square().sum()) for u in outs)
        count = sum(u.numel() for u in outs)
        scale = max(1.0, math.sqrt(total / count) / update_rms_clip) if count else 1.0
        out = tree_unflatten(td, [u / scale for u in outs])
        mu = state.mu
        if beta1 > 0:
            mu = tree_map(lambda m, u: beta1 * m + (1 - beta1) * u, state.mu, out)
            out = mu
        return out, AdafactorState(tree_unflatten(td, new_row), tree_unflatten(td, new_col), tree_unflatten(td, new_full), mu, phi, t)

    return make_optimizer_chain(GradientTransformation(init, update), lr, weight_decay,
                                decoupled_weight_decay=decoupled_weight_decay)


# ------------------------------------------------------------------------------------------ AdEMAMix

@dataclasses.dataclass(frozen=True)
class AdEMAMixState:
    mu_fast: Any
    mu_slow: Any
    nu: Any
    phi: Any
    step: int


def ademamix(lr: LR = 1e-3, betas=(0.9, 0.999, 0.9999), alpha: float = 5.0, eps: float = 1e-8,
             weight_decay: float = 0.0, *, decoupled_weight_decay: bool = True,
             update_rms_clip: float | None = None, noise_bias_correction: bool = False):
    """AdEMAMix: ``(m̂_fast + α·m_slow)/(√v̂ + eps)`` with a second, very slow momentum."""
    b1, b2, b3 = betas

    def init(params):
        return AdEMAMixState(_f32(params), _f32(params), _f32(params), 0.0, 0)

    def update(grads, state, *, params=None, noise_stddev=None):
        t = state.step + 1
        c1, c2 = 1 - b1 ** t, 1 - b2 ** t
        fast = tree_map(lambda m, g: b1 * m + (1 - b1) * _up(g), state.mu_fast, grads)
        slow = tree_map(lambda m, g: b3 * m + (1 - b3) * _up(g), state.mu_slow, grads)
        nu = tree_map(lambda v, g: b2 * v + (1 - b2) * _up(g) ** 2, state.nu, grads)
        phi = update_phi_ema(state.phi, resolve_noise_variance(noise_stddev), b2) if noise_bias_correction else state.phi

        def direction(path, mf, ms, v):
            v_hat = v / c2
            if noise_bias_correction:
                v_hat = debias_second_moment(v_hat, phi_for(phi, path) / c2)
            return (mf / c1 + alpha * ms) / (v_hat.sqrt() + eps)
        return map_leaves_with_path(direction, fast, slow, nu), AdEMAMixState(fast, slow, nu, phi, t)

    return make_optimizer_chain(GradientTransformation(init, update), lr, weight_decay,
                                decoupled_weight_decay=decoupled_weight_decay, update_rms_clip=update_rms_clip)


# ------------------------------------------------------------------------------------------ schedule-free

@dataclasses.dataclass(frozen=True)
class ScheduleFreeState:
    base: Any
    z: Any
    weight_sum: float
    step: int


def schedule_free(base: GradientTransformation, lr: LR = 1e-3, beta: float = 0.9, warmup_steps: int = 0):
    """Schedule-free wrapper (Defazio et al.): the params passed in are the interpolation ``y``.

    ``z ← z + Δ_base``; ``x ← (1−c)·x + c·z`` with ``c = w_t/Σw``, ``w_t = lr_t²``;
    ``y = (1−β)·z + β·x``.  The returned update moves ``y`` to its new value.
    """
    def init(params):
        return ScheduleFreeState(base.init(params), tree_map(lambda p: p.detach().clone().float(), params), 0.0, 0)

    def update(updates, state, *, params=None):
        if params is None:
            raise ValueError("schedule_free needs `params=`")
        raw, _ = unwrap_updates(updates, want_stddev=False, want_second=False)
        wrapped = updates if isinstance(updates, NoisedPytree) else raw
        delta, base_state = base.update(wrapped, state.base, params=params)
        t = state.step + 1
        sched = min(1.0, t / warmup_steps) if warmup_steps > 0 else 1.0
        w = (lr_at(lr, state.step) * sched) ** 2
        total = state.weight_sum + w
        c = w / total if total > 0 else 1.0
        z_new = tree_map(lambda z, d: z + sched * d.float(), state.z, delta)
        # x is recovered from y = (1−β) z + β x
        def step_y(y, z_old, z_n):
            x_old = (y.float() - (1 - beta) * z_old) / beta if beta > 0 else z_old
            x_new = (1 - c) * x_old + c * z_n
            return ((1 - beta) * z_n + beta * x_new) - y.float()
        out = tree_map(step_y, params, state.z, z_new)
        return out, ScheduleFreeState(base_state, z_new, total, t)

    return GradientTransformation(init, update)


def schedule_free_sgd(lr: LR = 1.0, beta: float = 0.9, warmup_steps: int = 0, weight_decay: float = 0.0):
    """Schedule-free SGD."""
    return schedule_free(sgd(lr=lr, weight_decay=weight_decay), lr=lr, beta=beta, warmup_steps=warmup_steps)


def schedule_free_adamw(lr: LR = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0,
                        warmup_steps: int = 0, noise_bias_correction: bool = False):
    """Schedule-free AdamW (interpolated iterate sequences, no learning-rate schedule)."""
    inner = make_optimizer_chain(_scale_by_rms(betas[1], eps, noise_bias_correction), lr, weight_decay)
    return schedule_free(inner, lr=lr, beta=betas[0], warmup_steps=warmup_steps)


def _scale_by_rms(b2: float, eps: float, bc: bool):
    def init(params):
        return RMSpropState(_f32(params), 0.0, 0)

    def update(grads, state, *, params=None, noise_stddev=None):
        t = state.step + 1
        nu = tree_map(lambda v, g: b2 * v + (1 - b2) * _up(g) ** 2, state.nu, grads)
        phi = update_phi_ema(state.phi, resolve_noise_variance(noise_stddev), b2) if bc else state.phi
        c2 = 1 - b2 ** t

        def direction(path, g, v):
            v_hat = v / c2
            if bc:
                v_hat = debias_second_moment(v_hat, phi_for(phi, path) / c2)
            return _up(g) / (v_hat.sqrt() + eps)
        return map_leaves_with_path(direction, grads, nu), RMSpropState(nu, phi, t)
    return GradientTransformation(init, update)


# ------------------------------------------------------------------------------------------ audit

def _tensor_fingerprint(x: torch.Tensor) -> list[float]:
    d = x.detach().double()
    if d.numel() == 0:
        return [0.0, 0.0, 0.0, 0.0, 0.0]
    return [float(d.sum()), float((d * d).sum()), float(d.min()), float(d.max()), float(d.numel())]


def sync_optimizer_state(state: Any, *, atol: float = 0.0, rtol: float = 0.0) -> Any:
    """Assert that replicated optimizer state is identical on every rank (debug audit).

    Each tensor contributes (sum, sumsq, min, max, numel); all fingerprints of the
    state travel in ONE packed min-reduce.
    """
    from ..distributed import _reduce_many, is_distributed
    if not is_distributed():
        return state
    vals: list[float] = []
    stack = [state]
    while stack:
        node = stack.pop()
        if isinstance(node, torch.Tensor):
            vals += _tensor_fingerprint(node)
        elif isinstance(node, (int, float)) and not isinstance(node, bool):
            vals.append(float(node))
        elif dataclasses.is_dataclass(node) and not isinstance(node, type):
            stack += [getattr(node, f.name) for f in dataclasses.fields(node)][::-1]
        elif isinstance(node, (tuple, list)):
            stack += list(node)[::-1]
        elif isinstance(node, dict):
            stack += [node[k] for k in sorted(node)][::-1]
    lows = _reduce_many(vals + [-v for v in vals], "min", None)
    k = len(vals)
    for i in range(k):
        lo, hi = lows[i], -lows[k + i]
        if abs(hi - lo) > atol + rtol * max(abs(hi), abs(lo)):
            raise RuntimeError(f"optimizer state differs across ranks at fingerprint slot {i}: min={lo} max={hi}")
    return state


from ..distributed import register_sync_type as _rst  # noqa: E402

for _t in (ChainState, SGDState, AdamState, LionState, AdagradState, RMSpropState, RAdamState, AdadeltaState,
           AdafactorState, AdEMAMixState, ScheduleFreeState):
    _rst(_t, sync_optimizer_state)

__all__ = ["AdamState", "GradientTransformation", "adadelta", "adafactor", "adagrad", "adam", "adamw", "ademamix",
           "apply_updates", "lion", "make_optimizer_chain", "radam", "rmsprop", "scale_by_adam", "schedule_free",
           "schedule_free_adamw", "schedule_free_sgd", "sgd", "sync_optimizer_state", "types"]

from ..utils.namespaces import submodule as _sub  # noqa: E402

_sub(__name__, "types", "Optimizer state classes.", {n: globals()[n] for n in (
    "AdEMAMixState AdadeltaState AdafactorState AdagradState AdamState LionState RAdamState RMSpropState ScheduleFreeState").split()}, bind=False)
