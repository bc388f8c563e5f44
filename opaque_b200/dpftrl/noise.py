"""DP-FTRL correlated noise: matrix-factorisation strategies and the streaming ``C⁻¹`` noise engine.

The mechanism releases ``A x + A C⁻¹ z`` for a workload ``A`` (prefix sums, optionally with
momentum / a learning-rate schedule) and a lower-triangular strategy ``C``; per step that means adding
row ``t`` of ``C⁻¹ Z`` (``Z`` iid Gaussian) to the clipped gradient sum.  Every strategy here is a frozen
dataclass (hashable, serialisable through ``strategy_to_wire``) exposing

  ``coefficients(n)``      first column of ``C`` when ``C`` is Toeplitz,
  ``gram_matrix(n)``       ``CᵀC`` for sensitivity / accounting,
  ``sensitivity(n, min_sep, max_participations)``,
  ``streaming_matrix(n)``  a :class:`StreamingMatrix` applying ``C⁻¹`` one row at a time,
  ``fused_mechanism(n, step)``  the parameters of the fused shard kernel
                                (``opaque_b200.parallel.ShardedDPOptimizer``): BLT buffers,
                                banded IIR history or an FIR over past draws.

Strategies: identity (DP-SGD), banded MF (optimised Toeplitz bands), BLT (buffered linear
Toeplitz, constant memory), BSR (banded square root, closed form), BISR (banded INVERSE square
root, an FIR on the noise) and λ-CGD (``n_t = d_t (z_t − λ z_{t−1})``).

Parity: packages/opaque-dpftrl/src/opaque/api/dpftrl/noise/{_engine,_streaming_matrix,_toeplitz,
_blt_math,_identity,_band_mf,_blt,_bsr,_bisr,_lambda_cgd,_mf_gaussian_noise,_strategy_codec}.py.
"""
from __future__ import annotations

import dataclasses
import functools
import math
from collections.abc import Callable
from typing import Any, NamedTuple

import numpy as np
import torch

from ..accounting.core import native
from ..pytree import tree_flatten_with_paths, tree_map, tree_unflatten
from ..random import RngKey, fold_in, generator_from_key
from ..scheduling import schedule_from_wire, schedule_to_wire
from ..types import (ClippedPytree, NoisedPytree, NoiseState, PerGroup, SecondMomentClippingOutput,
                     SecondMomentNoiseOutput)

# =============================================================================== streaming matrices


class StreamingMatrix(NamedTuple):
    """A lower-triangular operator applied one row at a time to a stream of (pytree) inputs."""
    init_multiply: Callable[[Any], Any]                 # template -> state
    multiply_next: Callable[[Any, Any], tuple[Any, Any]]  # (x_t, state) -> (row_t · X, state)
    row_norms_squared: Callable[[int], np.ndarray] | None = None

    def __matmul__(self, other):
        """``self @ other`` for another streaming matrix (composition) or a ``[n, ...]`` tensor (row-by-row product)."""
        if isinstance(other, StreamingMatrix):
            return multiply_streaming_matrices(self, other)
        if isinstance(other, torch.Tensor):
            return multiply_array(self, other)
        return NotImplemented

    def __mul__(self, factor: float) -> "StreamingMatrix":
        return scale_rows_and_columns(self, row_scale=np.array([float(factor)]))

    __rmul__ = __mul__

    def materialize(self, n: int) -> np.ndarray:
        """Dense ``n × n`` matrix (tests / small horizons): column j is the response to ``e_j``."""
        out = np.zeros((n, n))
        for j in range(n):
            state = self.init_multiply(torch.zeros(()))
            for t in range(n):
                y, state = self.multiply_next(torch.tensor(1.0 if t == j else 0.0, dtype=torch.float64), state)
                out[t, j] = float(y)
        return out


def identity_streaming() -> StreamingMatrix:
    return StreamingMatrix(lambda tpl: (), lambda x, s: (x, s), lambda n: np.ones(n))


def prefix_sum_streaming() -> StreamingMatrix:
    def init(tpl):
        return tree_map(lambda t: torch.zeros_like(t, dtype=torch.float32) if isinstance(t, torch.Tensor) else t, tpl)

    def nxt(x, s):
        new = tree_map(lambda a, b: a + b, s, x)
        return new, new
    return StreamingMatrix(init, nxt, lambda n: np.arange(1, n + 1, dtype=float))


# ---- algebra on streaming operators (parity: packages/opaque-dpftrl/src/opaque/api/dpftrl/noise/_streaming_matrix.py:157-305)

def diagonal_streaming(diag) -> StreamingMatrix:
    """``diag(d_0, d_1, ...)``; rows past ``len(diag)`` reuse the last entry.  The state is the row index (a Python int)."""
    d = np.asarray(diag, dtype=np.float64).reshape(-1)
    if d.size == 0:
        raise ValueError("diagonal_streaming needs at least one entry")

    def nxt(x, i):
        f = float(d[min(i, d.size - 1)])
        return tree_map(lambda t: t * f if isinstance(t, torch.Tensor) else t, x), i + 1

    def norms(n):
        return np.concatenate([d[:n], np.full(max(0, n - d.size), d[-1])]) ** 2
    return StreamingMatrix(lambda tpl: 0, nxt, norms)


def multiply_streaming_matrices(a: StreamingMatrix, b: StreamingMatrix) -> StreamingMatrix:
    """``A @ B``: every input goes through ``B``'s row, the result through ``A``'s (both stay streaming)."""
    def init(tpl):
        return a.init_multiply(tpl), b.init_multiply(tpl)

    def nxt(x, state):
        sa, sb = state
        inner, sb = b.multiply_next(x, sb)
        outer, sa = a.multiply_next(inner, sa)
        return outer, (sa, sb)

    def norms(n):                              # no closed form for a product: materialise (small horizons / tests)
        m = StreamingMatrix(init, nxt, None).materialize(n)
        return (m ** 2).sum(1)
    return StreamingMatrix(init, nxt, norms)


def multiply_array(a: StreamingMatrix, x: torch.Tensor) -> torch.Tensor:
    """``A @ x`` for ``x [n, ...]``, one row at a time."""
    state = a.init_multiply(x[0])
    rows = []
    for i in range(x.shape[0]):
        y, state = a.multiply_next(x[i], state)
        rows.append(y)
    return torch.stack(rows)


def scale_rows_and_columns(matrix: StreamingMatrix, row_scale=None, col_scale=None) -> StreamingMatrix:
    """``diag(row_scale) @ matrix @ diag(col_scale)``."""
    out = matrix
    if row_scale is not None:
        out = multiply_streaming_matrices(diagonal_streaming(row_scale), out)
    if col_scale is not None:
        out = multiply_streaming_matrices(out, diagonal_streaming(col_scale))
    return out


def momentum_sgd_matrix(momentum: float = 0.0, learning_rates=None) -> StreamingMatrix:
    """Workload of SGD with momentum and per-step learning rates: row t of ``A`` maps the gradient stream to the
    iterate displacement, ``m_t = μ m_{t-1} + g_t``, ``θ_t = θ_{t-1} + η_t m_t`` (``η`` repeats its last entry)."""
    lr = np.ones(1) if learning_rates is None else np.asarray(learning_rates, dtype=np.float64).reshape(-1)
    if lr.min() <= 0:
        raise ValueError("learning rates must be positive")
    mu = float(momentum)

    def init(tpl):
        zero = tree_map(lambda t: torch.zeros_like(t, dtype=torch.float64 if t.dtype == torch.float64 else torch.float32)
                        if isinstance(t, torch.Tensor) else t, tpl)
        return 0, zero, zero

    def nxt(x, state):
        i, mom, acc = state
        eta = float(lr[min(i, lr.size - 1)])
        mom = tree_map(lambda m, g: mu * m + g, mom, x)
        acc = tree_map(lambda a, m: a + eta * m, acc, mom)
        return acc, (i + 1, mom, acc)

    def norms(n):
        return (StreamingMatrix(init, nxt, None).materialize(n) ** 2).sum(1)
    return StreamingMatrix(init, nxt, norms)


def _zeros_state(tpl: Any, k: int) -> Any:
    return tree_map(lambda t: torch.zeros((k,) + tuple(t.shape), dtype=torch.float32, device=t.device)
                    if isinstance(t, torch.Tensor) else t, tpl)


def toeplitz_inverse_streaming(coef: np.ndarray) -> StreamingMatrix:
    """``C⁻¹`` for banded Toeplitz ``C`` (first column ``coef``): ``x_t = (y_t − Σ_{k≥1} c_k x_{t−k}) / c_0``."""
    c = np.asarray(coef, dtype=np.float64)
    k = len(c) - 1

    def init(tpl):
        return _zeros_state(tpl, max(k, 1))

    def nxt(y, state):
        def one(yv, st):
            if k == 0:
                return yv / c[0], st
            w = torch.as_tensor(c[1:], dtype=st.dtype, device=st.device)
            x = (yv.to(st.dtype) - torch.tensordot(w, st, dims=1)) / c[0]
            return x, torch.cat([x[None], st[:-1]], dim=0)
        paths, ys, td = tree_flatten_with_paths(y)
        sts = tree_flatten_with_paths(state)[1]
        outs = [one(a, b) for a, b in zip(ys, sts)]
        return tree_unflatten(td, [o[0] for o in outs]), tree_unflatten(td, [o[1] for o in outs])

    def row_norms(n):
        inv = inverse_coef(c, n)
        return np.cumsum(inv ** 2)
    return StreamingMatrix(init, nxt, row_norms)


def fir_streaming(taps: np.ndarray) -> StreamingMatrix:
    """Banded Toeplitz applied directly: ``x_t = Σ_k taps_k y_{t−k}``."""
    c = np.asarray(taps, dtype=np.float64)
    k = len(c) - 1

    def init(tpl):
        return _zeros_state(tpl, max(k, 1))

    def nxt(y, state):
        def one(yv, st):
            yv = yv.to(st.dtype)
            if k == 0:
                return c[0] * yv, st
            w = torch.as_tensor(c[1:], dtype=st.dtype, device=st.device)
            return c[0] * yv + torch.tensordot(w, st, dims=1), torch.cat([yv[None], st[:-1]], dim=0)
        paths, ys, td = tree_flatten_with_paths(y)
        sts = tree_flatten_with_paths(state)[1]
        outs = [one(a, b) for a, b in zip(ys, sts)]
        return tree_unflatten(td, [o[0] for o in outs]), tree_unflatten(td, [o[1] for o in outs])
    return StreamingMatrix(init, nxt, lambda n: np.cumsum(np.pad(c, (0, max(0, n - len(c))))[:n] ** 2))


def blt_inverse_streaming(scale: np.ndarray, decay: np.ndarray) -> StreamingMatrix:
    """``C⁻¹`` of a BLT with buffers ``S_j``: ``x = y − Σ_j s_j S_j``; ``S_j ← d_j S_j + x``."""
    s = np.asarray(scale, dtype=np.float64)
    d = np.asarray(decay, dtype=np.float64)

    def init(tpl):
        return _zeros_state(tpl, len(s))

    def nxt(y, state):
        def one(yv, st):
            sw = torch.as_tensor(s, dtype=st.dtype, device=st.device)
            dw = torch.as_tensor(d, dtype=st.dtype, device=st.device).reshape((-1,) + (1,) * (st.ndim - 1))
            x = yv.to(st.dtype) - torch.tensordot(sw, st, dims=1)
            return x, dw * st + x[None]
        paths, ys, td = tree_flatten_with_paths(y)
        sts = tree_flatten_with_paths(state)[1]
        outs = [one(a, b) for a, b in zip(ys, sts)]
        return tree_unflatten(td, [o[0] for o in outs]), tree_unflatten(td, [o[1] for o in outs])

    def row_norms(n):
        inv = blt_inverse_coef(s, d, n)
        return np.cumsum(inv ** 2)
    return StreamingMatrix(init, nxt, row_norms)


# =============================================================================== Toeplitz / BLT math

def sqrt_coefs(n: int) -> np.ndarray:
    """Coefficients of ``(1 − x)^{−1/2}``: ``r_0 = 1, r_k = r_{k−1}(2k−1)/(2k)`` — the optimal Toeplitz strategy."""
    r = np.ones(n)
    for k in range(1, n):
        r[k] = r[k - 1] * (2 * k - 1) / (2 * k)
    return r


def inv_sqrt_coefs(n: int) -> np.ndarray:
    """Coefficients of ``(1 − x)^{1/2}``: ``1, −1/2, −1/8, …``."""
    r = np.ones(n)
    for k in range(1, n):
        r[k] = r[k - 1] * (2 * k - 3) / (2 * k)
    return r


def inverse_coef(coef: np.ndarray, n: int) -> np.ndarray:
    """First ``n`` power-series coefficients of ``1 / C(x)``."""
    from scipy.signal import lfilter
    imp = np.zeros(n)
    imp[0] = 1.0
    c = np.asarray(coef, dtype=np.float64)[:n]
    return lfilter([1.0], c, imp)


def blt_coefs(scale: np.ndarray, decay: np.ndarray, n: int) -> np.ndarray:
    """Toeplitz coefficients of a BLT: ``t_0 = 1, t_k = Σ_j s_j d_j^{k−1}``."""
    s, d = np.asarray(scale, float), np.asarray(decay, float)
    out = np.ones(n)
    if n > 1:
        k = np.arange(n - 1)
        out[1:] = (s[None, :] * d[None, :] ** k[:, None]).sum(1)
    return out


def blt_inverse_coef(scale: np.ndarray, decay: np.ndarray, n: int) -> np.ndarray:
    return inverse_coef(blt_coefs(scale, decay, n), n)


def toeplitz_gram(coef: np.ndarray, n: int) -> np.ndarray:
    c = np.zeros(n)
    m = min(n, len(coef))
    c[:m] = np.asarray(coef, float)[:m]
    from scipy.linalg import toeplitz
    C = np.tril(toeplitz(c))
    return C.T @ C


def prefix_workload_error(inv: np.ndarray, *, kind: str = "max") -> float:
    """Squared error of releasing prefix sums through ``C``: rows of ``B = A C⁻¹`` have entries ``cumsum(inv)``."""
    b = np.cumsum(inv)
    row_sq = np.cumsum(b ** 2)
    return float(row_sq[-1] if kind == "max" else row_sq.mean())


def toeplitz_sensitivity_squared(coef: np.ndarray, n: int, min_sep: int = 1, max_participations: int | None = None) -> float:
    c = np.zeros(n)
    m = min(n, len(coef))
    c[:m] = np.asarray(coef, float)[:m]
    if np.all(c >= 0) and np.all(np.diff(c) <= 1e-15):
        return float(native.toeplitz_minsep_sensitivity_squared(np.minimum.accumulate(c).tolist(), n, min_sep, max_participations))
    g = toeplitz_gram(c, n)
    return float(native.general_sensitivity_squared_upper_bound(g.reshape(-1).tolist(), n, min_sep, max_participations))


def _series_mul(a: torch.Tensor, b: torch.Tensor, n: int) -> torch.Tensor:
    """First ``n`` coefficients of the product of two power series (FFT; differentiable)."""
    a, b = a[:n], b[:n]
    m = a.numel() + b.numel() - 1
    size = 1 << max(1, (m - 1).bit_length())
    out = torch.fft.irfft(torch.fft.rfft(a, size) * torch.fft.rfft(b, size), size)[: min(m, n)]
    return out if out.numel() == n else torch.cat([out, out.new_zeros(n - out.numel())])


def _series_inverse(c: torch.Tensor, n: int) -> torch.Tensor:
    """First ``n`` coefficients of ``1 / C(x)`` by Newton doubling ``g ← g·(2 − C·g)`` (differentiable in ``c``)."""
    g = (1.0 / c[0]).reshape(1)
    m = 1
    while m < n:
        m = min(2 * m, n)
        two_minus = -_series_mul(c, g, m)
        two_minus = two_minus + torch.nn.functional.one_hot(torch.zeros((), dtype=torch.long), m).to(c.dtype) * 2.0
        g = _series_mul(g, two_minus, m)
    return g


def momentum_workload_coefs(momentum: float, n: int) -> np.ndarray | None:
    """Toeplitz coefficients ``β^k`` of the momentum-SGD workload (``None`` = prefix sums, β = 1)."""
    if momentum < 0:
        raise ValueError(f"momentum must be >= 0, got {momentum}")
    return None if momentum == 1.0 else float(momentum) ** np.arange(n)


def toeplitz_workload_error(strategy_coef, n: int, *, workload_coef=None, query_weights=None, kind: str = "mean"):
    """Squared error of answering the workload ``W`` (lower-triangular Toeplitz, first column ``workload_coef``; prefix
    sums when ``None``) through ``C``: query ``t`` has error ``w_t² · Σ_{k≤t} b_k²`` with ``b = workload ⊛ C⁻¹``;
    the mean or the max over queries.  Takes and returns torch values when ``strategy_coef`` is a tensor (differentiable)."""
    as_numpy = not isinstance(strategy_coef, torch.Tensor)
    c = torch.as_tensor(np.asarray(strategy_coef, float) if as_numpy else strategy_coef, dtype=torch.float64)
    inv = _series_inverse(c, n)
    b = torch.cumsum(inv, 0) if workload_coef is None else _series_mul(torch.as_tensor(workload_coef, dtype=torch.float64), inv, n)
    err = torch.cumsum(b * b, 0)
    if query_weights is not None:
        w = torch.as_tensor(query_weights, dtype=torch.float64)
        if w.shape != (n,):
            raise ValueError(f"query_weights must have shape ({n},), got {tuple(w.shape)}")
        err = err * w * w
    out = err.mean() if kind == "mean" else err.max()
    return float(out) if as_numpy else out


@functools.lru_cache(maxsize=64)
def optimize_banded(n: int, bands: int, momentum: float = 1.0, lr_key: tuple[float, ...] | None = None,
                    error: str = "mean") -> tuple[float, ...]:
    """L-BFGS over the first ``bands`` Toeplitz coefficients, minimising (single-participation sensitivity)² × error of
    the momentum workload with per-step learning-rate weights ``lr_key``; exact gradients by autograd.  The result has
    unit L2 norm, so one participation has sensitivity 1 and participations at least ``bands`` steps apart add up in
    quadrature (reference: dpftrl/noise/_toeplitz.py ``optimize``, the same objective and start point)."""
    from scipy.optimize import minimize
    bands = max(1, min(bands, n))
    if bands == 1:
        return (1.0,)
    workload = momentum_workload_coefs(momentum, n)
    weights = None if lr_key is None else np.asarray(lr_key, float)

    def loss(x):
        c = torch.tensor(x, dtype=torch.float64, requires_grad=True)
        val = toeplitz_workload_error(c, n, workload_coef=workload, query_weights=weights, kind=error) * (c * c).sum()
        val.backward()
        return float(val.detach()), c.grad.numpy().copy()
    x0 = sqrt_coefs(bands)
    res = minimize(loss, x0, jac=True, method="L-BFGS-B", options={"maxiter": 250, "ftol": 1e-15, "gtol": 1e-10})
    best = res.x if np.all(np.isfinite(res.x)) and res.fun <= loss(x0)[0] else x0
    best = best * np.sign(best[0])
    return tuple((best / np.linalg.norm(best)).tolist())


@functools.lru_cache(maxsize=64)
def optimize_blt(n: int, num_buffers: int, min_sep: int = 1, max_participations: int | None = None,
                 error: str = "max") -> tuple[tuple[float, ...], tuple[float, ...]]:
    """Fit ``(scale, decay)`` of a BLT: start from a least-squares fit to ``(1−x)^{−1/2}`` and refine with L-BFGS."""
    from scipy.optimize import minimize, nnls
    nb = max(1, num_buffers)
    decay0 = 1.0 - np.logspace(-0.3, -min(3.0, 0.6 * nb + 0.6), nb)
    target = sqrt_coefs(n)[1:]
    k = np.arange(n - 1)
    basis = decay0[None, :] ** k[:, None]
    scale0, _ = nnls(basis, target)
    scale0 = np.maximum(scale0, 1e-6)

    def unpack(x):
        return np.exp(x[:nb]), 1.0 / (1.0 + np.exp(-x[nb:]))

    def loss(x):
        s, d = unpack(x)
        sens = native.blt_sensitivity_squared(s.tolist(), d.tolist(), n, min_sep, max_participations)
        inv = blt_inverse_coef(s, d, n)
        err = prefix_workload_error(inv, kind=error)
        if not (np.isfinite(sens) and np.isfinite(err)) or sens <= 0 or err <= 0:
            return 1e30
        return math.log(sens) + math.log(err)
    x0 = np.concatenate([np.log(scale0), np.log(decay0 / (1 - decay0))])
    res = minimize(loss, x0, method="L-BFGS-B", options={"maxiter": 300})
    best = res.x if res.fun <= loss(x0) else x0
    s, d = unpack(best)
    return tuple(s.tolist()), tuple(d.tolist())


# =============================================================================== strategies

def _lr_weights(lr_schedule, n: int) -> np.ndarray | None:
    if lr_schedule is None:
        return None
    return np.array([float(lr_schedule(t)) for t in range(n)])


def _accept_n_steps(fn):
    """The reference calls the strategy methods with keywords — ``coefficients(n_steps=…, min_sep=…, max_participations=…)``.
    Accept ``n_steps=`` for the first positional argument, and drop participation keywords a method does not take."""
    import functools
    import inspect
    takes = set(inspect.signature(fn).parameters)

    @functools.wraps(fn)
    def method(self, *args, n_steps=None, **kwargs):
        if n_steps is not None:
            if args:
                raise TypeError(f"{fn.__name__}() got the horizon twice")
            args = (n_steps,)
        return fn(self, *args, **{k: v for k, v in kwargs.items() if k in takes})
    method._accepts_n_steps = True
    return method


class MfStrategy:
    """Protocol-like base: a factorisation ``A = B C`` described by its strategy matrix ``C``."""

    _HORIZON_METHODS = ("coefficients", "gram_matrix", "sensitivity", "streaming_matrix")

    def __init_subclass__(cls, **kwargs):
        super().__init_subclass__(**kwargs)
        for name in cls._HORIZON_METHODS:
            fn = cls.__dict__.get(name)
            if fn is not None and not getattr(fn, "_accepts_n_steps", False):
                setattr(cls, name, _accept_n_steps(fn))

    def coefficients(self, n: int) -> np.ndarray:
        raise NotImplementedError

    def gram_matrix(self, n: int) -> np.ndarray:
        return toeplitz_gram(self.coefficients(n), n)

    def sensitivity(self, n: int, min_sep: int = 1, max_participations: int | None = None) -> float:
        return math.sqrt(toeplitz_sensitivity_squared(self.coefficients(n), n, min_sep, max_participations))

    def streaming_matrix(self, n: int) -> StreamingMatrix:
        return toeplitz_inverse_streaming(self.coefficients(n))

    def row_norm(self, n: int, t: int) -> float:
        """``‖row_t(C⁻¹)‖``: factor between the base σ and the realised std of step ``t``."""
        rn = self.streaming_matrix(n).row_norms_squared(n)
        return float(math.sqrt(rn[min(t, n - 1)]))

    def fused_mechanism(self, n: int, step: int = 0) -> dict | None:
        c = self.coefficients(n)
        c = np.trim_zeros(np.asarray(c), "b")
        if len(c) <= 1:
            return None
        if len(c) > 64:
            raise ValueError("the fused kernel supports at most 63 history buffers; use fewer bands or the streaming path")
        return {"kind": "banded", "coef": c.tolist()}


for _name in MfStrategy._HORIZON_METHODS:
    setattr(MfStrategy, _name, _accept_n_steps(MfStrategy.__dict__[_name]))
del _name


@dataclasses.dataclass(frozen=True)
class IdentityStrategy(MfStrategy):
    """``C = I``: independent noise every step (DP-SGD as a degenerate factorisation)."""

    def coefficients(self, n):
        return np.array([1.0])

    def streaming_matrix(self, n):
        return identity_streaming()


@dataclasses.dataclass(frozen=True)
class BandMfStrategy(MfStrategy):
    bands: int
    momentum: float = 1.0
    lr_schedule: Any = None

    def __post_init__(self):
        if self.bands < 1:
            raise ValueError("bands must be >= 1")

    def coefficients(self, n):
        # optimised for one participation per band window (cyclic Poisson / b-min-sep use); more participations only rescale
        lr = _lr_weights(self.lr_schedule, n)
        return np.array(optimize_banded(n, min(self.bands, n), float(self.momentum), None if lr is None else tuple(lr.tolist())))


@dataclasses.dataclass(frozen=True)
class BltStrategy(MfStrategy):
    max_buffers: int = 10
    momentum: float = 1.0
    lr_schedule: Any = None
    min_sep_hint: int = 1
    max_participations_hint: int | None = 1

    def __post_init__(self):
        if not 1 <= self.max_buffers <= 16:
            raise ValueError("max_buffers must be in [1, 16]")

    def params(self, n: int) -> tuple[np.ndarray, np.ndarray]:
        s, d = optimize_blt(n, self.max_buffers, self.min_sep_hint, self.max_participations_hint)
        return np.array(s), np.array(d)

    def coefficients(self, n):
        s, d = self.params(n)
        return blt_coefs(s, d, n)

    def sensitivity(self, n, min_sep=1, max_participations=None):
        s, d = self.params(n)
        return math.sqrt(native.blt_sensitivity_squared(s.tolist(), d.tolist(), n, min_sep, max_participations))

    def streaming_matrix(self, n):
        s, d = self.params(n)
        return blt_inverse_streaming(s, d)

    def fused_mechanism(self, n, step=0):
        s, d = self.params(n)
        return {"kind": "blt", "scale": s.tolist(), "decay": d.tolist()}


@dataclasses.dataclass(frozen=True)
class BsrStrategy(MfStrategy):
    """Banded square root: ``C`` = first ``bandwidth`` coefficients of ``√A`` for the workload with
    weight decay ``alpha`` and momentum ``beta``: ``c_k = Σ_{j≤k} α^{k−j} r_{k−j} β^{j} r_j``."""
    bandwidth: int
    alpha: float = 1.0
    beta: float = 0.0

    def __post_init__(self):
        if self.bandwidth < 1 or not 0 < self.alpha <= 1 or not 0 <= self.beta < 1:
            raise ValueError("need bandwidth >= 1, alpha in (0, 1], beta in [0, 1)")

    def coefficients(self, n):
        b = min(self.bandwidth, n)
        r = sqrt_coefs(b)
        ar, br = r * self.alpha ** np.arange(b), r * self.beta ** np.arange(b)
        return np.convolve(ar, br)[:b]


@dataclasses.dataclass(frozen=True)
class BisrStrategy(MfStrategy):
    """Banded inverse square root: ``C⁻¹`` itself is banded (an FIR on the noise), ``C`` is dense."""
    bandwidth: int
    normalized: bool = True
    momentum: float = 0.0
    lr_schedule: Any = None
    inv_coefficients: tuple[float, ...] | None = None

    def __post_init__(self):
        if self.bandwidth < 2:
            raise ValueError("bandwidth must be >= 2")

    def inverse_taps(self, n: int) -> np.ndarray:
        if self.inv_coefficients is not None:
            return np.asarray(self.inv_coefficients, float)[: self.bandwidth]
        return inv_sqrt_coefs(min(self.bandwidth, n))

    def coefficients(self, n):
        return inverse_coef(self.inverse_taps(n), n)

    def sensitivity(self, n, min_sep=1, max_participations=None):
        s = math.sqrt(toeplitz_sensitivity_squared(self.coefficients(n), n, min_sep, max_participations))
        return s

    def streaming_matrix(self, n):
        return fir_streaming(self.inverse_taps(n))

    def fused_mechanism(self, n, step=0):
        return {"kind": "fir", "coef": self.inverse_taps(n).tolist()}


@dataclasses.dataclass(frozen=True)
class LambdaCgdStrategy(MfStrategy):
    """λ-CGD: ``n_t = d_t (z_t − λ z_{t−1})`` — anti-correlated noise with one step of memory.

    ``C⁻¹`` is bidiagonal ``(1, −λ)`` scaled per row by ``d_t`` (1 when not normalised, otherwise the
    column-norm normaliser that keeps the sensitivity at one).
    """
    lambda_: float
    normalized: bool = True
    lr_schedule: Any = None
    # z_t is drawn from fold_in(key, t), without the label the other strategies use (reference: dpftrl/noise/_lambda_cgd.py:279)
    step_key_labels = ()

    def __post_init__(self):
        if not 0 <= self.lambda_ < 1:
            raise ValueError("lambda_ must be in [0, 1)")

    def coefficients(self, n):
        return self.lambda_ ** np.arange(n)       # C = (I − λ S)⁻¹ has geometric columns

    def column_norm(self, n: int, t: int) -> float:
        """``d_t``: norm of column ``t`` of ``C = (I − λS)⁻¹`` truncated to ``n`` rows,
        ``sqrt((1 − λ^{2(n−t)}) / (1 − λ²))`` (reference: dpftrl/noise/_lambda_cgd.py:90-108)."""
        if not 0 <= t < n:
            raise ValueError(f"step {t} is outside the calibrated horizon [0, {n})")
        lam2 = self.lambda_ ** 2
        if lam2 == 0.0:
            return 1.0
        tail = lam2 ** (n - t)
        return math.sqrt((1.0 if tail < 1e-30 else 1.0 - tail) / (1.0 - lam2))

    def gram_matrix(self, n: int) -> np.ndarray:
        """``C'ᵀC'`` of the (column-normalised) strategy matrix: ``G_ij = λ^{|i−j|} d_max(i,j) / d_min(i,j)``."""
        if not self.normalized:
            return toeplitz_gram(self.coefficients(n), n)
        d = self.row_scales(n)
        i, j = np.meshgrid(np.arange(n), np.arange(n), indexing="ij")
        lo, hi = np.minimum(i, j), np.maximum(i, j)
        return (self.lambda_ ** (hi - lo)) * d[hi] / d[lo]

    def row_scales(self, n: int) -> np.ndarray:
        """Per-row factors of ``C⁻¹``: ``d_t`` when normalised (every column of the scaled ``C`` then has unit norm), else 1."""
        return np.array([self.column_norm(n, t) for t in range(n)]) if self.normalized else np.ones(n)

    def sensitivity(self, n, min_sep=1, max_participations=None):
        """Largest norm of a sum of participating columns of ``C·diag(d)⁻¹`` (all inner products are non-negative, so the
        worst record takes part as often as ``min_sep`` / ``max_participations`` allow): ``⟨c'_i, c'_j⟩ = λ^{j−i} d_j / d_i``."""
        fn = native.lambda_cgd_normalized_sensitivity_squared if self.normalized else native.lambda_cgd_sensitivity_squared
        return math.sqrt(float(fn(self.lambda_, int(n), int(min_sep), max_participations)))

    def streaming_matrix(self, n):
        base = fir_streaming(np.array([1.0, -self.lambda_]))
        if not self.normalized:
            return base
        sm = scale_rows_and_columns(base, row_scale=self.row_scales(n))
        d = self.row_scales(n)
        per_row = np.where(np.arange(n) == 0, 1.0, 1.0 + self.lambda_ ** 2) * d ** 2      # ‖row_t(C⁻¹)‖² (not cumulative)
        return StreamingMatrix(sm.init_multiply, sm.multiply_next, lambda m: per_row[:m])

    def row_norm(self, n: int, t: int) -> float:
        """``‖row_t(C⁻¹)‖ = d_t·sqrt(1 + λ²)`` (``d_0`` at the first step): factor between σ and the realised std."""
        t = min(t, n - 1)
        d = self.column_norm(n, t) if self.normalized else 1.0
        return d if (t == 0 or self.lambda_ == 0.0) else d * math.sqrt(1.0 + self.lambda_ ** 2)

    def fused_mechanism(self, n, step=0):
        """FIR taps ``(d_t, −λ d_t)`` of the current step; ``coef_fn`` gives the fused optimizer each later step's pair."""
        def taps(t):
            d = self.column_norm(n, min(t, n - 1)) if self.normalized else 1.0
            return [d, -self.lambda_ * d]
        return {"kind": "fir", "coef": taps(step), "coef_fn": taps}


def identity_strategy() -> IdentityStrategy:
    """``C = I``: independent noise per step (DP-SGD as a matrix-factorisation strategy)."""
    return IdentityStrategy()


def band_mf_strategy(*, bands: int, momentum: float = 1.0, lr_schedule=None) -> BandMfStrategy:
    """Banded Toeplitz strategy with ``bands`` diagonals whose coefficients are optimised numerically (one participation per band window)."""
    return BandMfStrategy(int(bands), float(momentum), lr_schedule)


def blt_strategy(*, max_buffers: int = 10, momentum: float = 1.0, lr_schedule=None) -> BltStrategy:
    """Buffered linear Toeplitz: ``C`` generated by a few (scale, decay) pairs; ``C^-1`` streams with one buffer per pair."""
    return BltStrategy(int(max_buffers), float(momentum), lr_schedule)


def bsr_strategy(*, bandwidth: int, alpha: float = 1.0, beta: float = 0.0) -> BsrStrategy:
    """Banded square root: the first ``bandwidth`` coefficients of the square root of the workload with weight decay ``alpha`` and momentum ``beta``."""
    return BsrStrategy(int(bandwidth), float(alpha), float(beta))


def bisr_strategy(*, bandwidth: int, normalized: bool = True, momentum: float = 0.0, lr_schedule=None,
                  inv_coefficients=None) -> BisrStrategy:
    """Banded inverse square root: ``C^-1`` itself is banded (an FIR filter on the noise), ``C`` is dense."""
    inv = None if inv_coefficients is None else tuple(float(x) for x in inv_coefficients)
    return BisrStrategy(int(bandwidth), bool(normalized), float(momentum), lr_schedule, inv)


def lambda_cgd_strategy(*, lambda_: float, normalized: bool = True, lr_schedule=None) -> LambdaCgdStrategy:
    """lambda-CGD: ``n_t = d_t (z_t - lambda z_{t-1})``, anti-correlated noise with one step of memory (``d_t`` normalises the sensitivity to one when ``normalized``)."""
    return LambdaCgdStrategy(float(lambda_), bool(normalized), lr_schedule)


_STRATEGIES: dict[str, type] = {c.__name__: c for c in (IdentityStrategy, BandMfStrategy, BltStrategy, BsrStrategy,
                                                         BisrStrategy, LambdaCgdStrategy)}


def register_strategy(cls: type) -> type:
    _STRATEGIES[cls.__name__] = cls
    return cls


def strategy_to_wire(s: MfStrategy) -> dict[str, Any]:
    """``{"type": ClassName, **factory_args}``; schedules become ``{"__opaque_recipe__": …}`` dicts."""
    out: dict[str, Any] = {"type": type(s).__name__}
    for f in dataclasses.fields(s):
        v = getattr(s, f.name)
        if f.name == "lr_schedule":
            v = schedule_to_wire(v)
        elif isinstance(v, tuple):
            v = list(v)
        out[f.name] = v
    return out


def strategy_from_wire(w: dict[str, Any]) -> MfStrategy:
    cls = _STRATEGIES[w["type"]]
    kw = {}
    for f in dataclasses.fields(cls):
        if f.name in w:
            v = w[f.name]
            if f.name == "lr_schedule":
                v = schedule_from_wire(v)
            elif isinstance(v, list):
                v = tuple(v)
            kw[f.name] = v
    return cls(**kw)


# =============================================================================== noise engine

@dataclasses.dataclass(frozen=True)
class MFNoiseState(NoiseState):
    _inner_state: Any
    _step_counter: int
    _rng_key: RngKey
    _first_max_norm: float | None = None


def _iid_normal_like(tree: Any, std: float, step_key: RngKey, compute_dtype: torch.dtype) -> Any:
    """Independent ``N(0, std²)`` for every leaf (device Philox where available, CPU generator otherwise)."""
    paths, leaves, td = tree_flatten_with_paths(tree)
    out, offset, gen = [], 0, None
    for x in leaves:
        if not isinstance(x, torch.Tensor):
            out.append(x)
            continue
        z = torch.zeros(x.shape, dtype=compute_dtype, device=x.device)
        if x.is_cuda and compute_dtype == torch.float32:
            from .. import ops
            ops.philox_normal_add_(z, seed=step_key.seed, offset=offset, std=std)
        else:
            if gen is None:
                gen = generator_from_key(step_key)
            z = (torch.randn(x.shape, generator=gen, dtype=compute_dtype) * std).to(x.device)
        out.append(z)
        offset += x.numel()
    return tree_unflatten(td, out)


def mf_gaussian_noise(grad_template: Any, strategy: MfStrategy, *, n_steps: int, min_sep: int = 1,
                      max_participations: int | None = None, noise_multiplier: float, key: RngKey,
                      compute_dtype: torch.dtype = torch.float32, second_moment_strategy: MfStrategy | None = None):
    """Correlated-noise mechanism: ``noise_fn(ClippedPytree, state) -> (NoisedPytree, state)``.

    Base σ is ``noise_multiplier · max_norm`` (the accountant divides the multiplier by
    ``sensitivity(C)``, see ``dpftrl.accounting.mf_gaussian``); step ``t`` adds row ``t`` of ``C⁻¹Z`` and
    publishes the realised std ``σ·‖row_t(C⁻¹)‖``.  The horizon ``n_steps`` is enforced, and ``max_norm``
    must stay constant across steps (the sensitivity analysis assumes one clipping bound).
    """
    if n_steps < 1:
        raise ValueError("n_steps must be >= 1")
    if not isinstance(key, RngKey):
        raise TypeError(f"key must be RngKey, got {type(key)}")
    if noise_multiplier < 0:
        raise ValueError("noise_multiplier must be >= 0")
    if min_sep < 1 or (max_participations is not None and max_participations < 1):
        raise ValueError("min_sep and max_participations must be >= 1")
    if second_moment_strategy is not None:
        return _paired_mf_gaussian_noise(grad_template, strategy, second_moment_strategy, n_steps=n_steps,
                                         noise_multiplier=noise_multiplier, key=key, compute_dtype=compute_dtype)
    sm = strategy.streaming_matrix(n_steps)
    row_sq = sm.row_norms_squared(n_steps) if sm.row_norms_squared is not None else np.ones(n_steps)
    inner0 = sm.init_multiply(grad_template.pytree if isinstance(grad_template, ClippedPytree) else grad_template)
    step_labels = getattr(strategy, "step_key_labels", ("mf_gaussian_column",))

    def noise_fn(grads: ClippedPytree, st: MFNoiseState):
        with torch.profiler.record_function("opaque::mf_gaussian_noise"):
            if isinstance(grads, SecondMomentClippingOutput):
                raise TypeError("mf_gaussian_noise was built without second_moment_strategy and expects ClippedPytree "
                                "inputs; rebuild it with second_moment_strategy=... for the paired form")
            if isinstance(grads, NoisedPytree) or not isinstance(grads, ClippedPytree):
                raise TypeError("mf_gaussian_noise expects ClippedPytree inputs")
            if isinstance(grads.max_norm, PerGroup):
                raise TypeError("mf_gaussian_noise supports a scalar max_norm")
            t = st._step_counter
            if t >= n_steps:
                raise RuntimeError(f"the mechanism was calibrated for {n_steps} steps; step {t} is past the horizon")
            mn = float(grads.max_norm)
            first = st._first_max_norm if st._first_max_norm is not None else mn
            if not math.isclose(first, mn, rel_tol=1e-9, abs_tol=0.0):
                raise ValueError(f"max_norm changed from {first} to {mn}; matrix-factorisation noise needs a constant bound")
            sigma = noise_multiplier * mn
            step_key = fold_in(st._rng_key, *step_labels, t)
            z = _iid_normal_like(grads.pytree, sigma, step_key, compute_dtype) if sigma > 0 else tree_map(
                lambda g: torch.zeros_like(g, dtype=compute_dtype), grads.pytree)
            x, inner = sm.multiply_next(z, st._inner_state)
            noisy = tree_map(lambda g, n: (g.to(compute_dtype) + n).to(g.dtype), grads.pytree, x)
            realised = sigma * math.sqrt(float(row_sq[t]))
            return NoisedPytree(noisy, grads.max_norm, realised), MFNoiseState(inner, t + 1, st._rng_key, first)

    return noise_fn, MFNoiseState(inner0, 0, key, None)


@dataclasses.dataclass(frozen=True)
class SecondMomentMFNoiseState(NoiseState):
    """Joint state of the paired form: one correlated-noise stream for ``Σg`` and one for ``Σg²``."""
    _first_state: MFNoiseState
    _second_state: MFNoiseState

    @property
    def _step_counter(self) -> int:
        return self._first_state._step_counter

    @property
    def _rng_key(self) -> RngKey:
        return self._first_state._rng_key


def _paired_mf_gaussian_noise(grad_template: Any, first: MfStrategy, second: MfStrategy, *, n_steps: int,
                              noise_multiplier: float, key: RngKey, compute_dtype: torch.dtype):
    """Two independent correlated-noise streams that share one privacy budget.

    With ``c1`` / ``c2`` the single-participation sensitivities (largest column norms) of the two strategies, the
    base deviations are ``paired_noise_stddev(max_norm·c1, squared_max_norm·c2, noise_multiplier / c1)``: the joint
    Mahalanobis budget is ``(c1 / noise_multiplier)²``, i.e. what the single-stream accountant charges for
    ``(noise_multiplier, first)``, and with a vanishing second stream the first deviation falls back to
    ``noise_multiplier · max_norm``.  Each stream then passes through its own ``C⁻¹``.
    Parity: packages/opaque-dpftrl/src/opaque/api/dpftrl/noise/_second_moment.py:56-190 of the reference.
    """
    from ..noise_allocation import FIRST_MOMENT_FOLD_TAG, SECOND_MOMENT_FOLD_TAG, paired_noise_stddev
    template = grad_template.pytree if isinstance(grad_template, ClippedPytree) else grad_template
    streams = []
    for strat, tag in ((first, FIRST_MOMENT_FOLD_TAG), (second, SECOND_MOMENT_FOLD_TAG)):
        sm = strat.streaming_matrix(n_steps)
        row_sq = sm.row_norms_squared(n_steps) if sm.row_norms_squared is not None else np.ones(n_steps)
        c = float(strat.sensitivity(n_steps, min_sep=n_steps, max_participations=1))
        streams.append((sm, row_sq, c, MFNoiseState(sm.init_multiply(template), 0, fold_in(key, tag), None)))
    (sm1, rows1, c1, st1), (sm2, rows2, c2, st2) = streams

    def one_stream(sm, rows, clipped: ClippedPytree, st: MFNoiseState, sigma: float, what: str):
        if isinstance(clipped.max_norm, PerGroup):
            raise TypeError("mf_gaussian_noise supports a scalar max_norm")
        mn = float(clipped.max_norm)
        first_mn = st._first_max_norm if st._first_max_norm is not None else mn
        if not math.isclose(first_mn, mn, rel_tol=1e-9, abs_tol=0.0):
            raise ValueError(f"{what}: max_norm changed from {first_mn} to {mn}; matrix-factorisation noise needs a constant bound")
        t = st._step_counter
        step_key = fold_in(st._rng_key, "mf_gaussian_column", t)
        z = _iid_normal_like(clipped.pytree, sigma, step_key, compute_dtype) if sigma > 0 else tree_map(
            lambda g: torch.zeros_like(g, dtype=compute_dtype), clipped.pytree)
        x, inner = sm.multiply_next(z, st._inner_state)
        noisy = tree_map(lambda g, n: (g.to(compute_dtype) + n).to(g.dtype), clipped.pytree, x)
        return (NoisedPytree(noisy, clipped.max_norm, sigma * math.sqrt(float(rows[t]))),
                MFNoiseState(inner, t + 1, st._rng_key, first_mn))

    def noise_fn(grads: Any, st: SecondMomentMFNoiseState):
        with torch.profiler.record_function("opaque::mf_gaussian_noise_paired"):
            if not isinstance(grads, SecondMomentClippingOutput):
                raise TypeError("mf_gaussian_noise was built with second_moment_strategy and expects "
                                "SecondMomentClippingOutput inputs: use clipped_grad(..., second_moment=True), or rebuild "
                                "the noise function without second_moment_strategy")
            g1, g2 = grads.grads, grads.squared_grads
            if not isinstance(g1, ClippedPytree) or not isinstance(g2, ClippedPytree):
                raise TypeError("both streams must be ClippedPytree")
            if st._step_counter >= n_steps:
                raise RuntimeError(f"the mechanism was calibrated for {n_steps} steps; step {st._step_counter} is past the horizon")
            if isinstance(g1.max_norm, PerGroup) or isinstance(g2.max_norm, PerGroup):
                raise TypeError("mf_gaussian_noise supports a scalar max_norm")
            s1, s2 = paired_noise_stddev(float(g1.max_norm) * c1, float(g2.max_norm) * c2, noise_multiplier / c1)
            n1, new1 = one_stream(sm1, rows1, g1, st._first_state, s1, "first stream")
            n2, new2 = one_stream(sm2, rows2, g2, st._second_state, s2, "squared stream")
            return SecondMomentNoiseOutput(n1, n2), SecondMomentMFNoiseState(new1, new2)

    return noise_fn, SecondMomentMFNoiseState(st1, st2)


def sync_mf_noise_state(state: MFNoiseState) -> MFNoiseState:
    from ..distributed import assert_scalar_equal, assert_string_equal, is_distributed
    if is_distributed():
        assert_scalar_equal(state._step_counter, name="MFNoiseState._step_counter")
        assert_string_equal(f"{state._rng_key.seed}:{state._first_max_norm}", name="MFNoiseState key/max_norm")
    return state


from ..distributed import register_sync_type as _rst  # noqa: E402

_rst(MFNoiseState, sync_mf_noise_state)
_rst(SecondMomentMFNoiseState, lambda st: SecondMomentMFNoiseState(sync_mf_noise_state(st._first_state),
                                                                   sync_mf_noise_state(st._second_state)))

__all__ = [
    "BandMfStrategy", "BisrStrategy", "BltStrategy", "BsrStrategy", "IdentityStrategy", "LambdaCgdStrategy",
    "MFNoiseState", "MfStrategy", "SecondMomentMFNoiseState", "StreamingMatrix", "band_mf_strategy", "bisr_strategy", "blt_coefs",
    "blt_inverse_coef", "blt_inverse_streaming", "blt_strategy", "bsr_strategy", "fir_streaming", "identity_strategy",
    "identity_streaming", "inv_sqrt_coefs", "inverse_coef", "lambda_cgd_strategy", "mf_gaussian_noise",
    "momentum_workload_coefs", "optimize_banded", "optimize_blt", "toeplitz_workload_error", "prefix_sum_streaming", "register_strategy", "sqrt_coefs", "strategy_from_wire",
    "strategy_to_wire", "toeplitz_gram", "toeplitz_inverse_streaming", "toeplitz_sensitivity_squared",
]

from ..utils.namespaces import submodule as _sub  # noqa: E402

_sub(__name__, "types", "Strategy and state types of the matrix-factorisation noise.",
     {n: globals()[n] for n in ("BandMfStrategy", "BisrStrategy", "BltStrategy", "BsrStrategy", "IdentityStrategy", "LambdaCgdStrategy",
                                "MFNoiseState", "MfStrategy", "SecondMomentMFNoiseState")}, bind=False)
