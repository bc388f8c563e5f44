"""Step → value schedules as frozen, serialisable dataclass recipes.

A schedule is any ``Callable[[int], float]``.  Each recipe here is a frozen
dataclass so that it hashes, compares and round-trips through
``opaque_b200.serialization`` (and through the DP-FTRL strategy codec, which
tags recipes with their class name).

Parity: packages/opaque-engine/src/opaque/api/engine/scheduling/*.py.
"""
from __future__ import annotations

import math
from collections.abc import Callable
from dataclasses import dataclass
from typing import Union

Schedule = Callable[[int], float]
Shape = Union[str, Callable[[float], float]]

# progress in [0, 1] -> factor rising 0 -> 1
NAMED_RAMPS: dict[str, Callable[[float], float]] = {
    "linear": lambda p: p,
    "cosine": lambda p: 0.5 - 0.5 * math.cos(math.pi * p),
    "1-sqrt": lambda p: 1.0 - math.sqrt(1.0 - p),
}
# progress in [0, 1] -> factor falling 1 -> 0
NAMED_DECAYS: dict[str, Callable[[float], float]] = {
    "linear": lambda p: 1.0 - p,
    "cosine": lambda p: 0.5 + 0.5 * math.cos(math.pi * p),
    "1-sqrt": lambda p: 1.0 - math.sqrt(p),
}


def _resolve(shape: Shape, table: dict, field: str) -> Callable[[float], float]:
    if callable(shape):
        return shape
    try:
        return table[shape]
    except KeyError:
        raise ValueError(f"Unknown {field}={shape!r}; expected one of {sorted(table)} or a callable") from None


def resolve_ramp(ramp: Shape, *, field: str = "ramp"):
    """A named warm-up ramp (or a callable) as a function of the progress in [0, 1]."""
    return _resolve(ramp, NAMED_RAMPS, field)


def resolve_decay(decay: Shape, *, field: str = "decay_shape"):
    """A named decay shape (or a callable) as a function of the progress in [0, 1]."""
    return _resolve(decay, NAMED_DECAYS, field)


def _count(step: int, begin: int, span: int) -> int:
    return max(0, min(span, step - begin))


@dataclass(frozen=True, slots=True)
class ConstantSchedule:
    value: float

    def __call__(self, step: int) -> float:
        return self.value


@dataclass(frozen=True, slots=True)
class PolynomialSchedule:
    """``end + (init-end)·(1 - count/T)^power`` with ``count`` clamped to ``[0, T]``."""
    init_value: float
    end_value: float
    power: float
    transition_steps: int
    transition_begin: int = 0

    def __call__(self, step: int) -> float:
        span = max(1, self.transition_steps)
        left = 1.0 - _count(step, self.transition_begin, span) / span
        return self.end_value + (self.init_value - self.end_value) * left ** self.power


@dataclass(frozen=True, slots=True)
class LinearSchedule:
    init_value: float
    end_value: float
    transition_steps: int
    transition_begin: int = 0

    def __call__(self, step: int) -> float:
        span = max(1, self.transition_steps)
        left = 1.0 - _count(step, self.transition_begin, span) / span
        return self.end_value + (self.init_value - self.end_value) * left


@dataclass(frozen=True, slots=True)
class CosineSchedule:
    """Half-cosine by default; past the end the cosine keeps going, clipped at zero."""
    init_value: float
    end_value: float
    transition_steps: int
    transition_begin: int = 0
    num_cycles: float = 0.5

    def __call__(self, step: int) -> float:
        span = max(1, self.transition_steps)
        progress = max(0, step - self.transition_begin) / span
        wave = 0.5 * (1.0 + math.cos(2.0 * math.pi * self.num_cycles * progress))
        return self.end_value + (self.init_value - self.end_value) * max(0.0, wave)


@dataclass(frozen=True, slots=True)
class ExponentialSchedule:
    init_value: float
    decay_rate: float
    transition_begin: int = 0
    transition_steps: int = 1
    staircase: bool = False
    end_value: float | None = None

    def __call__(self, step: int) -> float:
        elapsed = step - self.transition_begin
        if self.transition_steps <= 0 or self.decay_rate == 0 or elapsed <= 0:
            return float(self.init_value)
        exponent = elapsed / self.transition_steps
        if self.staircase:
            exponent = math.floor(exponent)
        value = self.init_value * self.decay_rate ** exponent
        if self.end_value is None:
            return value
        return max(value, self.end_value) if self.decay_rate < 1.0 else min(value, self.end_value)


@dataclass(frozen=True, slots=True)
class InverseSqrtSchedule:
    """``init·sqrt(T/(s+T))``: ``init`` at ``s=0``, ``init/√2`` at ``s=T``."""
    init_value: float
    transition_steps: int
    transition_begin: int = 0

    def __call__(self, step: int) -> float:
        span = max(1, self.transition_steps)
        s = max(0, step - self.transition_begin)
        return self.init_value * math.sqrt(span / (s + span))


@dataclass(frozen=True, slots=True)
class OneMinusSqrtSchedule:
    init_value: float
    end_value: float
    transition_steps: int
    transition_begin: int = 0

    def __call__(self, step: int) -> float:
        span = max(1, self.transition_steps)
        progress = min(1.0, max(0, step - self.transition_begin) / span)
        return self.end_value + (self.init_value - self.end_value) * (1.0 - math.sqrt(progress))


@dataclass(frozen=True, slots=True)
class WarmupStableDecay:
    """Ramp 0→init, hold, then decay init→end (Hägele et al. 2024)."""
    init_value: float
    end_value: float
    num_warmup_steps: int
    num_stable_steps: int
    num_decay_steps: int
    warmup_ramp: Shape = "linear"
    decay_shape: Shape = "1-sqrt"

    def __call__(self, step: int) -> float:
        hold_end = self.num_warmup_steps + self.num_stable_steps
        if step < self.num_warmup_steps:
            return resolve_ramp(self.warmup_ramp, field="warmup_ramp")(step / self.num_warmup_steps) * self.init_value
        if step < hold_end:
            return self.init_value
        if step < hold_end + self.num_decay_steps:
            p = (step - hold_end) / self.num_decay_steps
            return self.end_value + (self.init_value - self.end_value) * resolve_decay(self.decay_shape)(p)
        return self.end_value


@dataclass(frozen=True, slots=True)
class WithRestarts:
    """Replay ``schedule`` ``num_cycles`` times over the transition window."""
    schedule: Schedule
    transition_steps: int
    num_cycles: int
    transition_begin: int = 0

    def __call__(self, step: int) -> float:
        period = self.transition_steps / self.num_cycles
        rel = step - self.transition_begin
        if rel < 0:
            return self.schedule(0)
        if rel >= self.transition_steps:
            return self.schedule(period)
        return self.schedule(rel - (rel // period) * period)


@dataclass(frozen=True, slots=True)
class WithWarmup:
    """Multiply ``schedule`` by a ramp factor during the first ``transition_steps``."""
    schedule: Schedule
    transition_steps: int
    ramp: Shape = "linear"
    init_value: float = 0.0

    def __call__(self, step: int) -> float:
        value = self.schedule(step)
        if step >= self.transition_steps:
            return value
        factor = resolve_ramp(self.ramp)(step / self.transition_steps)
        if self.init_value != 0.0:
            factor = self.init_value + (1.0 - self.init_value) * factor
        return factor * value


def constant_schedule(value: float) -> ConstantSchedule:
    """``step -> value`` for every step."""
    return ConstantSchedule(float(value))


def cosine_schedule(init_value, end_value, transition_steps, transition_begin=0, num_cycles=0.5):
    """Cosine transition from ``init_value`` to ``end_value`` over ``transition_steps`` (``num_cycles`` of the cosine; 0.5 = one half-wave)."""
    return CosineSchedule(float(init_value), float(end_value), int(transition_steps),
                          int(transition_begin), float(num_cycles))


def exponential_schedule(init_value, decay_rate, transition_begin=0, transition_steps=1,
                         staircase=False, end_value=None):
    """``init_value * decay_rate ** ((step - transition_begin) / transition_steps)``, optionally in stair-steps and bounded by ``end_value``."""
    return ExponentialSchedule(float(init_value), float(decay_rate), int(transition_begin),
                               int(transition_steps), bool(staircase),
                               None if end_value is None else float(end_value))


def inverse_sqrt_schedule(init_value, transition_steps, transition_begin=0):
    """Flat at ``init_value`` for ``transition_steps`` steps, then inverse-square-root decay."""
    return InverseSqrtSchedule(float(init_value), int(transition_steps), int(transition_begin))


def linear_schedule(init_value, end_value, transition_steps, transition_begin=0):
    """Linear interpolation from ``init_value`` to ``end_value`` over ``transition_steps``."""
    return LinearSchedule(float(init_value), float(end_value), int(transition_steps), int(transition_begin))


def one_minus_sqrt_schedule(init_value, end_value, transition_steps, transition_begin=0):
    """``1 - sqrt(progress)`` transition from ``init_value`` to ``end_value`` over ``transition_steps``."""
    return OneMinusSqrtSchedule(float(init_value), float(end_value), int(transition_steps), int(transition_begin))


def polynomial_schedule(init_value, end_value, power, transition_steps, transition_begin=0):
    """Polynomial interpolation of the given ``power`` from ``init_value`` to ``end_value``."""
    return PolynomialSchedule(float(init_value), float(end_value), float(power),
                              int(transition_steps), int(transition_begin))


def warmup_stable_decay(init_value, end_value=0.0, *, num_warmup_steps, num_stable_steps,
                        num_decay_steps, warmup_ramp="linear", decay_shape="1-sqrt"):
    """Warm up to ``init_value``, hold it for ``num_stable_steps``, then decay to ``end_value`` (the WSD recipe)."""
    if num_warmup_steps <= 0:
        raise ValueError(f"warmup_stable_decay requires num_warmup_steps > 0; got {num_warmup_steps}.")
    if num_stable_steps < 0:
        raise ValueError(f"warmup_stable_decay requires num_stable_steps >= 0; got {num_stable_steps}.")
    if num_decay_steps <= 0:
        raise ValueError(f"warmup_stable_decay requires num_decay_steps > 0; got {num_decay_steps}.")
    resolve_ramp(warmup_ramp, field="warmup_ramp")
    resolve_decay(decay_shape, field="decay_shape")
    return WarmupStableDecay(float(init_value), float(end_value), int(num_warmup_steps),
                             int(num_stable_steps), int(num_decay_steps), warmup_ramp, decay_shape)


def with_restarts(schedule, transition_steps, num_cycles, transition_begin=0):
    """Restart ``schedule`` every ``transition_steps`` steps, ``num_cycles`` times (warm restarts)."""
    if num_cycles <= 0:
        raise ValueError(f"with_restarts requires num_cycles > 0; got {num_cycles}.")
    if transition_steps <= 0:
        raise ValueError(f"with_restarts requires transition_steps > 0; got {transition_steps}.")
    return WithRestarts(schedule, int(transition_steps), int(num_cycles), int(transition_begin))


def with_warmup(schedule, transition_steps, *, ramp="linear", init_value=0.0):
    """Multiply ``schedule`` by a warm-up ramp over its first ``transition_steps`` steps (from ``init_value`` of its value)."""
    if transition_steps <= 0:
        raise ValueError(f"with_warmup requires transition_steps > 0; got {transition_steps}.")
    if not 0.0 <= init_value <= 1.0:
        raise ValueError(f"with_warmup requires init_value in [0, 1]; got {init_value}.")
    resolve_ramp(ramp)
    inner = schedule if callable(schedule) else ConstantSchedule(float(schedule))
    return WithWarmup(inner, int(transition_steps), ramp, float(init_value))


RECIPES: dict[str, type] = {c.__name__: c for c in (
    ConstantSchedule, CosineSchedule, ExponentialSchedule, InverseSqrtSchedule, LinearSchedule,
    OneMinusSqrtSchedule, PolynomialSchedule, WarmupStableDecay, WithRestarts, WithWarmup)}

RECIPE_TAG = "__opaque_recipe__"


def schedule_to_wire(schedule):
    """Nested JSON-able form ``{"__opaque_recipe__": ClassName, **fields}``."""
    import dataclasses
    if schedule is None or isinstance(schedule, (int, float)):
        return schedule
    cls = type(schedule)
    if cls.__name__ not in RECIPES or RECIPES[cls.__name__] is not cls:
        raise TypeError(f"{cls.__name__} is not a serialisable schedule recipe")
    wire = {RECIPE_TAG: cls.__name__}
    for f in dataclasses.fields(schedule):
        v = getattr(schedule, f.name)
        if callable(v) and type(v).__name__ in RECIPES:
            v = schedule_to_wire(v)
        elif callable(v):
            raise TypeError(f"field {f.name!r} holds a raw callable and cannot be serialised")
        wire[f.name] = v
    return wire


def schedule_from_wire(wire):
    """Rebuild a schedule from its serialised (wire) description."""
    if not isinstance(wire, dict) or RECIPE_TAG not in wire:
        return wire
    cls = RECIPES[wire[RECIPE_TAG]]
    kwargs = {k: schedule_from_wire(v) for k, v in wire.items() if k != RECIPE_TAG}
    return cls(**kwargs)


__all__ = [
    "ConstantSchedule", "CosineSchedule", "ExponentialSchedule", "InverseSqrtSchedule",
    "LinearSchedule", "NAMED_DECAYS", "NAMED_RAMPS", "OneMinusSqrtSchedule", "PolynomialSchedule",
    "RECIPES", "Schedule", "WarmupStableDecay", "WithRestarts", "WithWarmup", "constant_schedule",
    "cosine_schedule", "exponential_schedule", "inverse_sqrt_schedule", "linear_schedule",
    "one_minus_sqrt_schedule", "polynomial_schedule", "resolve_decay", "resolve_ramp",
    "schedule_from_wire", "schedule_to_wire", "warmup_stable_decay", "with_restarts", "with_warmup",
]

from ..utils.namespaces import submodule as _sub  # noqa: E402

_sub(__name__, "types", "Schedule recipe classes.", {n: globals()[n] for n in (
    "ConstantSchedule CosineSchedule ExponentialSchedule InverseSqrtSchedule LinearSchedule OneMinusSqrtSchedule PolynomialSchedule Schedule "
    "WarmupStableDecay WithRestarts WithWarmup").split()}, bind=False)
