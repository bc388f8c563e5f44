"""Process algebra over the C++ PLD accountant.

A :class:`DpProcess` is a frozen, hashable *description* of a mechanism; nothing numerical happens
until a metric is asked for.  ``p * n`` repeats (nested repeats flatten), ``p | q`` composes
(identities vanish, equal neighbouring leaves merge into a repeat, and long left-leaning spines stay
shallow), and ``process.pld()`` lowers the tree to native PLD objects — repeats become ONE
self-composition (``IFFT(FFT^n)``), which is why ``poisson(gaussian(σ), q) * 10_000`` costs two FFTs.

Parity: packages/opaque-accounting/src/opaque/api/accounting/core/_base.py, composition/*.py,
_accountant.py, _budgets.py, calibration.py, discretization.py, _pld_cache.py, _process_codec.py,
mechanisms/*.py.
"""
from __future__ import annotations

import contextvars
import dataclasses
import json
import math
from abc import ABC, abstractmethod
from collections import OrderedDict
from collections.abc import Callable, Mapping
from typing import Any, ClassVar

from ..serialization import register_serializer
from ..utils import build as _build


def _load_native():
    import importlib
    try:
        return importlib.import_module("opaque_b200.accounting._native")
    except ImportError:
        _build.build_accounting()
        importlib.invalidate_caches()
        return importlib.import_module("opaque_b200.accounting._native")


native = _load_native()

# ----------------------------------------------------------------------------------- discretisation


@dataclasses.dataclass(frozen=True)
class DiscretizationConfig:
    discretization: float = 1e-4
    log_mass_truncation_bound: float = -50.0
    max_grid_size: int = 10_000_000
    tail_mass_truncation: float = 1e-15
    max_conv_grid: int = 32_768
    num_mc_samples: int = 100_000
    seed: int = 42
    # True reproduces the reference library's numbers to 1e-6 (a discretised PMF is rescaled to unit mass, which lowers
    # delta by ~1e-8 relative per mechanism); False (default) keeps every reported epsilon a strict upper bound
    proportional_normalization: bool = False

    @property
    def log_x_mass_truncation_bound(self) -> float:
        """The reference's name of ``log_mass_truncation_bound``."""
        return self.log_mass_truncation_bound

    def __post_init__(self) -> None:
        if not self.discretization > 0:
            raise ValueError("discretization must be > 0")
        if not 0 <= self.tail_mass_truncation < 1:
            raise ValueError("tail_mass_truncation must be in [0, 1)")
        if self.max_grid_size < 2:
            raise ValueError("max_grid_size must be >= 2")

    def to_native(self):
        return native.DiscretizationConfig(self.discretization, self.log_mass_truncation_bound, self.max_grid_size,
                                           self.tail_mass_truncation, self.max_conv_grid, self.num_mc_samples, self.seed,
                                           self.proportional_normalization)


_CONFIG: contextvars.ContextVar[DiscretizationConfig] = contextvars.ContextVar("opaque_b200_discretization",
                                                                               default=DiscretizationConfig())


def get_discretization() -> DiscretizationConfig:
    """The ambient ``DiscretizationConfig``."""
    return _CONFIG.get()


class set_discretization:
    """``set_discretization(cfg)`` sets the ambient config; usable as a context manager to restore it."""

    def __init__(self, config: "DiscretizationConfig | float | None" = None, **overrides: Any):
        if isinstance(config, (int, float)) and not isinstance(config, bool):      # set_discretization(1e-3): the grid step first
            overrides = {"discretization": float(config), **overrides}
            config = None
        if "log_x_mass_truncation_bound" in overrides:                             # the reference's name of this field
            overrides["log_mass_truncation_bound"] = overrides.pop("log_x_mass_truncation_bound")
        base = config or get_discretization()
        self._token = _CONFIG.set(dataclasses.replace(base, **overrides) if overrides else base)

    def __enter__(self):
        return _CONFIG.get()

    def __exit__(self, *exc: Any) -> None:
        _CONFIG.reset(self._token)


# ----------------------------------------------------------------------------------- PLD cache

class _PldCache:
    """Small LRU keyed by ``(config, process key, count)``; values are native PLD objects."""

    def __init__(self, capacity: int = 64):
        self.capacity = capacity
        self._data: OrderedDict[Any, Any] = OrderedDict()

    def get(self, key: Any):
        try:
            self._data.move_to_end(key)
            return self._data[key]
        except KeyError:
            return None

    def put(self, key: Any, value: Any) -> None:
        self._data[key] = value
        self._data.move_to_end(key)
        while len(self._data) > self.capacity:
            self._data.popitem(last=False)

    def clear(self) -> None:
        self._data.clear()


PLD_CACHE = _PldCache()


def clear_caches() -> None:
    PLD_CACHE.clear()


# ----------------------------------------------------------------------------------- processes

_PROCESS_REGISTRY: dict[str, type] = {}


class DpProcess(ABC):
    """Base of all mechanism descriptions (subclasses are frozen dataclasses)."""

    def __init_subclass__(cls, **kw: Any) -> None:
        super().__init_subclass__(**kw)
        _PROCESS_REGISTRY[cls.__name__] = cls
        register_serializer(cls, lambda p: {"": process_to_wire(p)}, lambda t, sd: process_from_wire(sd[""]) if "" in sd else t)

    # -- lowering --------------------------------------------------------------------------
    @abstractmethod
    def _build_pld(self, config: DiscretizationConfig):
        """Native PLD of ONE application."""

    def _cache_key(self):
        return self

    def pld(self, config: DiscretizationConfig | None = None):
        return self.repeated_pld(1, config)

    def repeated_pld(self, count: int, config: DiscretizationConfig | None = None):
        """PLD of ``count`` adaptive applications (one self-composition, cached)."""
        cfg = config or get_discretization()
        key = (cfg, self._cache_key(), count)
        hit = PLD_CACHE.get(key)
        if hit is not None:
            return hit
        base_key = (cfg, self._cache_key(), 1)
        base = PLD_CACHE.get(base_key)
        if base is None:
            base = self._build_pld(cfg)
            PLD_CACHE.put(base_key, base)
        out = base if count == 1 else base.self_compose(count)
        PLD_CACHE.put(key, out)
        return out

    # -- metrics ----------------------------------------------------------------------------
    def epsilon_at(self, delta: float, config: DiscretizationConfig | None = None) -> float:
        if not 0 <= delta <= 1:
            raise ValueError(f"delta must be in [0, 1], got {delta}")
        return self.pld(config).epsilon_at(delta)

    def delta_at(self, epsilon: float, config: DiscretizationConfig | None = None) -> float:
        return min(1.0, self.pld(config).delta_at(epsilon))

    def advantage(self, config: DiscretizationConfig | None = None) -> float:
        return min(1.0, self.pld(config).advantage())

    def beta_at(self, alpha: float, config: DiscretizationConfig | None = None) -> float:
        return self.pld(config).beta_at(alpha)

    def risk_at(self, prior: float, config: DiscretizationConfig | None = None) -> float:
        return self.pld(config).risk_at(prior)

    # -- algebra ----------------------------------------------------------------------------
    def _leaf_and_count(self) -> tuple["DpProcess", int]:
        return self, 1

    def __mul__(self, count: int) -> "DpProcess":
        if isinstance(count, bool) or not isinstance(count, int):
            return NotImplemented
        if count < 0:
            raise ValueError("repeat count must be >= 0")
        if count == 0:
            return Identity()
        leaf, n = self._leaf_and_count()
        if isinstance(leaf, Identity):
            return leaf
        return leaf if n * count == 1 else Repeated(leaf, n * count)

    __rmul__ = __mul__

    def __or__(self, other: "DpProcess") -> "DpProcess":
        if not isinstance(other, DpProcess):
            return NotImplemented
        if isinstance(self, Identity):
            return other
        if isinstance(other, Identity):
            return self
        la, na = self._leaf_and_count()
        lb, nb = other._leaf_and_count()
        if not isinstance(self, Composed) and not isinstance(other, Composed) and la == lb:
            return Repeated(la, na + nb)
        if isinstance(self, Composed) and not isinstance(other, Composed):
            lr, nr = self.right._leaf_and_count()
            if not isinstance(self.right, Composed) and lr == lb:       # merge into the right-most leaf
                return Composed(self.left, Repeated(lr, nr + nb))
        return Composed(self, other)


@dataclasses.dataclass(frozen=True)
class Identity(DpProcess):
    """Perfectly private step (no release)."""

    def _build_pld(self, config):
        return native.identity_pld(config.to_native())


@dataclasses.dataclass(frozen=True)
class NonPrivate(DpProcess):
    """A release with no privacy (all mass at infinite loss)."""

    def _build_pld(self, config):
        return native.nonprivate_pld(config.to_native())


@dataclasses.dataclass(frozen=True)
class EpsDelta(DpProcess):
    epsilon: float
    delta: float = 0.0

    def __post_init__(self):
        if self.epsilon < 0 or not 0 <= self.delta <= 1:
            raise ValueError("need epsilon >= 0 and delta in [0, 1]")

    def _build_pld(self, config):
        return native.eps_delta_pld(self.epsilon, self.delta, config.to_native())


@dataclasses.dataclass(frozen=True)
class Repeated(DpProcess):
    inner: DpProcess
    count: int

    def __post_init__(self):
        if self.count < 1:
            raise ValueError("count must be >= 1")

    def _leaf_and_count(self):
        leaf, n = self.inner._leaf_and_count()
        return leaf, n * self.count

    def _build_pld(self, config):
        leaf, n = self._leaf_and_count()
        return leaf.repeated_pld(n, config)

    def repeated_pld(self, count, config=None):
        leaf, n = self._leaf_and_count()
        return leaf.repeated_pld(n * count, config)


@dataclasses.dataclass(frozen=True)
class Composed(DpProcess):
    left: DpProcess
    right: DpProcess

    def _terms(self) -> list[DpProcess]:
        out, stack = [], [self]
        while stack:
            node = stack.pop()
            if isinstance(node, Composed):
                stack.append(node.right)
                stack.append(node.left)
            else:
                out.append(node)
        return out

    def _build_pld(self, config):
        acc = None
        for term in self._terms():
            p = term.pld(config)
            acc = p if acc is None else acc.compose(p)
        return acc

    def __hash__(self):
        return hash(("Composed", tuple(self._terms())))

    def __eq__(self, other):
        return isinstance(other, Composed) and self._terms() == other._terms()

    def __repr__(self):
        return "Composed(" + " | ".join(repr(t) for t in self._terms()) + ")"


@dataclasses.dataclass(frozen=True)
class CachedProcess(DpProcess):
    """Marks a sub-tree whose PLD should be computed once and reused (e.g. an executed prefix)."""
    inner: DpProcess

    def _build_pld(self, config):
        return self.inner.pld(config)


class DpHorizonProcess(DpProcess):
    """A whole-run mechanism whose PLD depends on the horizon: ``pld_at(n_steps)``."""

    @abstractmethod
    def pld_at(self, n_steps: int, config: DiscretizationConfig | None = None):
        ...


@dataclasses.dataclass(frozen=True)
class PerStep(DpProcess):
    """Per-step view of a horizon process: ``PerStep(h) * n`` evaluates ``h.pld_at(n)``."""
    process: DpHorizonProcess

    def _build_pld(self, config):
        return self.process.pld_at(1, config)

    def repeated_pld(self, count, config=None):
        cfg = config or get_discretization()
        key = (cfg, self, count)
        hit = PLD_CACHE.get(key)
        if hit is None:
            hit = self.process.pld_at(count, cfg)
            PLD_CACHE.put(key, hit)
        return hit


def eps_delta(epsilon: float, delta: float = 0.0) -> EpsDelta:
    """A mechanism known only through an ``(epsilon, delta)`` guarantee."""
    return EpsDelta(float(epsilon), float(delta))


def identity() -> Identity:
    """The process that releases nothing (neutral element of composition)."""
    return Identity()


def nonprivate() -> NonPrivate:
    """A release with no privacy guarantee (infinite loss)."""
    return NonPrivate()


def repeat(process: DpProcess, count: int) -> DpProcess:
    """``n``-fold self-composition of a process (also ``process * n``)."""
    return process * count


def compose(*processes: DpProcess) -> DpProcess:
    """Sequential composition of processes (also available as ``a | b``)."""
    out: DpProcess = Identity()
    for p in processes:
        out = out | p
    return out


def cached(process: DpProcess) -> CachedProcess:
    """Wrap a process so that its PLD is computed once per discretisation config and reused."""
    return process if isinstance(process, CachedProcess) else CachedProcess(process)


def per_step(process: DpHorizonProcess) -> PerStep:
    """View a horizon-dependent process as ``n`` per-step releases (``process.pld_at(n)``)."""
    return PerStep(process)


# ----------------------------------------------------------------------------------- codec

_CUSTOM_WIRE: dict[str, tuple[Callable, Callable]] = {}


def register_process_codec(cls: type, to_wire: Callable[[Any], dict], from_wire: Callable[[dict], Any]) -> None:
    """Custom wire form for a leaf class (e.g. processes that hold an MF strategy)."""
    _CUSTOM_WIRE[cls.__name__] = (to_wire, from_wire)


def process_to_wire(p: DpProcess) -> dict[str, Any]:
    """Nested JSON-able dict with a ``"type"`` discriminator; spines are walked with an explicit stack."""
    def leaf(node: DpProcess) -> dict[str, Any]:
        name = type(node).__name__
        if name in _CUSTOM_WIRE:
            return {"type": name, **_CUSTOM_WIRE[name][0](node)}
        out: dict[str, Any] = {"type": name}
        for f in dataclasses.fields(node):
            v = getattr(node, f.name)
            out[f.name] = process_to_wire(v) if isinstance(v, DpProcess) else v
        return out
    if isinstance(p, Composed):
        return {"type": "Composed", "terms": [process_to_wire(t) for t in p._terms()]}
    return leaf(p)


def process_from_wire(w: Mapping[str, Any]) -> DpProcess:
    name = w["type"]
    if name == "Composed":
        if "terms" in w:
            return compose(*(process_from_wire(t) for t in w["terms"]))
        return Composed(process_from_wire(w["left"]), process_from_wire(w["right"]))
    if name in _CUSTOM_WIRE:
        return _CUSTOM_WIRE[name][1]({k: v for k, v in w.items() if k != "type"})
    cls = _PROCESS_REGISTRY.get(name)
    if cls is None:
        raise ValueError(f"unknown process type {name!r}")
    kwargs = {}
    for f in dataclasses.fields(cls):
        if f.name in w:
            v = w[f.name]
            kwargs[f.name] = process_from_wire(v) if isinstance(v, Mapping) and "type" in v else v
    return cls(**kwargs)


# ----------------------------------------------------------------------------------- budgets

class Budget(ABC):
    value: float
    name: ClassVar[str]
    decreasing: ClassVar[bool]      # True: privacy-LOSS metric (safe at or below the target)

    @abstractmethod
    def evaluate(self, process: DpProcess) -> float:
        ...


@dataclasses.dataclass(frozen=True)
class EpsilonBudget(Budget):
    epsilon: float
    delta: float
    name: ClassVar[str] = "epsilon"
    decreasing: ClassVar[bool] = True

    def __post_init__(self):
        if not self.epsilon > 0 or not 0 <= self.delta < 1:
            raise ValueError("need epsilon > 0 and delta in [0, 1)")

    @property
    def value(self):
        return self.epsilon

    def evaluate(self, process):
        return process.epsilon_at(self.delta)


@dataclasses.dataclass(frozen=True)
class DeltaBudget(Budget):
    delta: float
    epsilon: float
    name: ClassVar[str] = "delta"
    decreasing: ClassVar[bool] = True

    def __post_init__(self):
        if not 0 < self.delta < 1 or self.epsilon < 0:
            raise ValueError("need delta in (0, 1) and epsilon >= 0")

    @property
    def value(self):
        return self.delta

    def evaluate(self, process):
        return process.delta_at(self.epsilon)


@dataclasses.dataclass(frozen=True)
class AdvantageBudget(Budget):
    advantage: float
    name: ClassVar[str] = "advantage"
    decreasing: ClassVar[bool] = True

    def __post_init__(self):
        if not 0 < self.advantage < 1:
            raise ValueError("advantage must be in (0, 1)")

    @property
    def value(self):
        return self.advantage

    def evaluate(self, process):
        return process.advantage()


@dataclasses.dataclass(frozen=True)
class BetaBudget(Budget):
    beta: float
    alpha: float
    name: ClassVar[str] = "beta"
    decreasing: ClassVar[bool] = False

    def __post_init__(self):
        if not 0 < self.beta < 1 or not 0 <= self.alpha <= 1:
            raise ValueError("need beta in (0, 1) and alpha in [0, 1]")

    @property
    def value(self):
        return self.beta

    def evaluate(self, process):
        return process.beta_at(self.alpha)


@dataclasses.dataclass(frozen=True)
class RiskBudget(Budget):
    risk: float
    prior: float
    name: ClassVar[str] = "risk"
    decreasing: ClassVar[bool] = False

    def __post_init__(self):
        if not 0 < self.risk < 1 or not 0 < self.prior < 1:
            raise ValueError("need risk and prior in (0, 1)")

    @property
    def value(self):
        return self.risk

    def evaluate(self, process):
        return process.risk_at(self.prior)


_BUDGETS: dict[str, type] = {c.__name__: c for c in (EpsilonBudget, DeltaBudget, AdvantageBudget, BetaBudget, RiskBudget)}


_BUDGET_CODECS: dict[type, tuple[str, Any, Any]] = {}        # type -> (wire name, state_dict_fn, from_state_dict_fn)


def register_budget_serializer(typ: type, state_dict_fn=None, from_state_dict_fn=None, *, type_name: str | None = None):
    """Register a budget class with the wire codec.

    ``register_budget_serializer(Cls)`` (also usable as a decorator) is enough for a dataclass: its fields are the state.
    With ``state_dict_fn(budget) -> JSON-like dict`` and ``from_state_dict_fn(dict) -> budget`` any class can take part;
    ``type_name`` is the name written into checkpoints (default: the class name) and must be unique."""
    name = type_name or typ.__name__
    if name in _BUDGETS and _BUDGETS[name] is not typ:
        raise ValueError(f"budget type name {name!r} is already registered for {_BUDGETS[name].__name__}")
    if (state_dict_fn is None) != (from_state_dict_fn is None):
        raise ValueError("give both state_dict_fn and from_state_dict_fn, or neither")
    _BUDGETS[name] = typ
    if state_dict_fn is not None:
        _BUDGET_CODECS[typ] = (name, state_dict_fn, from_state_dict_fn)
    return typ


def budget_state_dict(b: Budget | None):
    if b is None:
        return None
    codec = _BUDGET_CODECS.get(type(b))
    if codec is not None:
        return {"type": codec[0], "state": codec[1](b)}
    name = next((n for n, c in _BUDGETS.items() if c is type(b)), type(b).__name__)
    return {"type": name, **dataclasses.asdict(b)}


def budget_from_state_dict(sd: Mapping[str, Any] | None):
    if sd is None:
        return None
    cls = _BUDGETS[sd["type"]]
    codec = _BUDGET_CODECS.get(cls)
    if codec is not None:
        return codec[2](sd["state"])
    return cls(**{k: v for k, v in sd.items() if k != "type"})


def epsilon_budget(epsilon: float, delta: float) -> EpsilonBudget:
    """Budget stated as ``epsilon`` at a fixed ``delta``."""
    return EpsilonBudget(float(epsilon), float(delta))


def delta_budget(delta: float, epsilon: float) -> DeltaBudget:
    """Budget stated as ``delta`` at a fixed ``epsilon``."""
    return DeltaBudget(float(delta), float(epsilon))


def advantage_budget(advantage: float) -> AdvantageBudget:
    """Budget stated as a bound on the membership-inference advantage."""
    return AdvantageBudget(float(advantage))


def beta_budget(beta: float, alpha: float) -> BetaBudget:
    """Budget stated as a false-negative rate ``beta`` at false-positive rate ``alpha`` (trade-off curve point)."""
    return BetaBudget(float(beta), float(alpha))


def risk_budget(risk: float, prior: float) -> RiskBudget:
    """Budget stated as a bound on the Bayes risk of a membership attacker with a given prior."""
    return RiskBudget(float(risk), float(prior))


# ----------------------------------------------------------------------------------- accountant

class Accountant:
    """Running composition of executed steps: ``acct |= step_process``.

    ``prefix`` is a process that was executed before this accountant started (a resumed run or an
    earlier training stage); metrics always cover ``prefix | recorded steps``.
    """

    def __init__(self, budget: Budget | None = None, prefix: DpProcess | None = None):
        self.budget = budget
        self.process: DpProcess = prefix if prefix is not None else Identity()

    def __or__(self, step: DpProcess) -> "Accountant":
        if not isinstance(step, DpProcess):
            return NotImplemented
        out = Accountant(self.budget)
        out.process = self.process | step
        return out

    def __ior__(self, step: DpProcess) -> "Accountant":
        if not isinstance(step, DpProcess):
            return NotImplemented
        self.process = self.process | step
        return self

    def epsilon_at(self, delta: float) -> float:
        return self.process.epsilon_at(delta)

    def delta_at(self, epsilon: float) -> float:
        return self.process.delta_at(epsilon)

    def advantage(self) -> float:
        return self.process.advantage()

    def beta_at(self, alpha: float) -> float:
        return self.process.beta_at(alpha)

    def risk_at(self, prior: float) -> float:
        return self.process.risk_at(prior)

    def budget_exceeded(self) -> bool:
        if self.budget is None:
            return False
        v = self.budget.evaluate(self.process)
        return v > self.budget.value if self.budget.decreasing else v < self.budget.value

    def state_dict(self) -> dict[str, Any]:
        return {"process": process_to_wire(self.process), "budget": budget_state_dict(self.budget)}

    @staticmethod
    def from_state_dict(sd: Mapping[str, Any]) -> "Accountant":
        acct = Accountant(budget_from_state_dict(sd.get("budget")))
        acct.process = process_from_wire(sd["process"])
        return acct

    def to_json(self) -> str:
        return json.dumps(self.state_dict(), separators=(",", ":"))


register_serializer(Accountant, lambda a: a.state_dict(),
                    lambda t, sd: Accountant.from_state_dict(sd) if "process" in sd else t)


# ----------------------------------------------------------------------------------- calibration

@dataclasses.dataclass(frozen=True)
class CalibrateResult:
    param: float
    achieved: float
    target: float
    iterations: int
    converged: bool = True


def calibrate(budget: Budget, process: Callable[[float], DpProcess], param_min: float, param_max: float,
              tolerance: float = 1e-6, max_iterations: int = 100, prefix: DpProcess | None = None) -> CalibrateResult:
    """Bisection on one mechanism parameter; the result is always on the privacy-safe side of the target.

    The direction in which the metric moves with the parameter is detected by probing both
    endpoints; exactly one endpoint must be safe.  Interior probes must stay inside the
    endpoint envelope (monotonicity check).  Caches are cleared afterwards.
    """
    if not (math.isfinite(tolerance) and tolerance > 0):
        raise ValueError("tolerance must be finite and positive")
    if max_iterations <= 0:
        raise ValueError("max_iterations must be positive")
    if not param_min < param_max:
        raise ValueError("param_min must be < param_max")
    target = float(budget.value)
    pre = cached(prefix) if prefix is not None else None

    def metric(x: float) -> float:
        p = process(x)
        return budget.evaluate(pre | p if pre is not None else p)

    def safe(v: float) -> bool:
        return v <= target if budget.decreasing else v >= target

    try:
        lo_v, hi_v = metric(param_min), metric(param_max)
        if math.isnan(lo_v) or math.isnan(hi_v):
            raise ValueError("budget evaluation returned NaN at the bounds")
        if safe(lo_v) == safe(hi_v):
            raise ValueError(f"bounds do not bracket the target {target}: metric({param_min})={lo_v}, "
                             f"metric({param_max})={hi_v}")
        if lo_v == hi_v:
            raise ValueError("metric is flat across the bounds")
        safe_x, unsafe_x = (param_min, param_max) if safe(lo_v) else (param_max, param_min)
        safe_v = lo_v if safe(lo_v) else hi_v
        if math.isinf(safe_v):
            raise ValueError("metric is infinite on the privacy-safe endpoint")
        env_lo, env_hi = min(lo_v, hi_v), max(lo_v, hi_v)
        for it in range(1, max_iterations + 1):
            if math.isclose(safe_v, target, rel_tol=tolerance, abs_tol=0.0):
                return CalibrateResult(safe_x, safe_v, target, it - 1)
            mid = 0.5 * (safe_x + unsafe_x)
            if mid == safe_x or mid == unsafe_x:
                break
            v = metric(mid)
            if math.isnan(v) or (not math.isinf(v) and not (env_lo - 1e-12 <= v <= env_hi + 1e-12)):
                raise ValueError(f"metric({mid})={v} escapes the endpoint envelope [{env_lo}, {env_hi}]: not monotone")
            if safe(v):
                safe_x, safe_v = mid, v
            else:
                unsafe_x = mid
        if math.isclose(safe_v, target, rel_tol=tolerance, abs_tol=0.0):
            return CalibrateResult(safe_x, safe_v, target, max_iterations)
        raise RuntimeError(f"calibration did not converge within {max_iterations} iterations "
                           f"(best safe value {safe_v} for target {target})")
    finally:
        clear_caches()


__all__ = [
    "Accountant", "AdvantageBudget", "BetaBudget", "Budget", "CachedProcess", "CalibrateResult", "Composed",
    "DeltaBudget", "DiscretizationConfig", "DpHorizonProcess", "DpProcess", "EpsDelta", "EpsilonBudget", "Identity",
    "NonPrivate", "PerStep", "Repeated", "RiskBudget", "advantage_budget", "beta_budget", "budget_from_state_dict",
    "budget_state_dict", "cached", "calibrate", "clear_caches", "compose", "delta_budget", "eps_delta",
    "epsilon_budget", "get_discretization", "identity", "native", "nonprivate", "per_step", "process_from_wire",
    "process_to_wire", "register_budget_serializer", "register_process_codec", "repeat", "risk_budget",
    "set_discretization",
]
