"""Empirical privacy auditing with one training run (Steinke, Nasr & Jagielski 2023).

Workflow: ``coin_flip`` marks ``num_canaries`` records as canaries and includes each with probability ½ (fair,
keyed coins); train once on the kept records; score every canary with ``loss_scores`` or ``gradient_scores``;
``one_run`` turns the scores into guesses (highest scores → "in", lowest → "out", the rest abstain) and returns
the largest ε that the number of correct guesses refutes at the requested confidence, by the (ε, δ) binomial
test and by the μ-GDP family test.

Everything here is host-side NumPy / PyTorch; it is diagnostic and never feeds back into private training.

Parity: packages/opaque-auditing/src/opaque/api/auditing/{_coin_flip.py, attacks/{_gradient,_loss}.py,
one_run/{_estimate,_eps_delta,_gdp,_roc,_stats}.py}.
"""
from __future__ import annotations

import dataclasses
import math
from collections.abc import Callable, Sequence
from typing import Any

import numpy as np
import torch
from scipy import stats

from ..random import RngKey, fold_in


@dataclasses.dataclass(frozen=True)
class CoinFlip:
    """Which records are canaries and which canaries were included in training."""
    canary_indices: np.ndarray        # [m] indices into the original dataset
    included: np.ndarray              # [m] bool
    dataset_size: int

    @property
    def num_canaries(self) -> int:
        return len(self.canary_indices)

    def kept_indices(self) -> np.ndarray:
        """Indices of the records to train on: all non-canaries plus the included canaries."""
        drop = np.zeros(self.dataset_size, dtype=bool)
        drop[self.canary_indices[~self.included]] = True
        return np.flatnonzero(~drop)


@dataclasses.dataclass(frozen=True)
class CanaryScores:
    """One membership score per canary (higher = more likely included), aligned with ``CoinFlip.canary_indices``."""
    scores: np.ndarray

    def __post_init__(self):
        object.__setattr__(self, "scores", np.asarray(self.scores, dtype=np.float64).reshape(-1))


def canary_scores(scores: Any) -> CanaryScores:
    """Wrap an array or tensor of per-canary scores as ``CanaryScores``."""
    if isinstance(scores, torch.Tensor):
        scores = scores.detach().float().cpu().numpy()
    return CanaryScores(np.asarray(scores))


def coin_flip(dataset: Any, *, num_canaries: int, key: RngKey) -> CoinFlip:
    """Choose ``num_canaries`` records uniformly and flip a fair coin for each."""
    n = len(dataset)
    if not 1 <= num_canaries <= n:
        raise ValueError("num_canaries must be in [1, len(dataset)]")
    rng = np.random.default_rng(fold_in(key, "audit_coin_flip").seed)
    idx = np.sort(rng.choice(n, size=num_canaries, replace=False))
    return CoinFlip(idx, rng.random(num_canaries) < 0.5, n)


def loss_scores(loss_fn: Callable[[Any], torch.Tensor], canaries: Sequence[Any], *, baseline_losses: Any = None) -> CanaryScores:
    """Score = −loss of the trained model on the canary (minus an optional pre-training baseline loss)."""
    with torch.no_grad():
        losses = np.array([float(loss_fn(c)) for c in canaries])
    if baseline_losses is not None:
        losses = losses - np.asarray(baseline_losses, dtype=np.float64)
    return CanaryScores(-losses)


def gradient_scores(canary_grads: Sequence[Any], released_updates: Sequence[Any]) -> CanaryScores:
    """Score = Σ_t ⟨g_canary,t , released_t⟩ : the canary's gradient direction shows up in the noisy sums it joined."""
    def flat(tree):
        from ..pytree import tree_leaves
        return torch.cat([x.detach().float().reshape(-1).cpu() for x in tree_leaves(tree) if isinstance(x, torch.Tensor)])
    out = []
    for per_canary in canary_grads:
        steps = per_canary if isinstance(per_canary, (list, tuple)) else [per_canary] * len(released_updates)
        out.append(sum(float(flat(g) @ flat(u)) for g, u in zip(steps, released_updates)))
    return CanaryScores(np.array(out))


# ------------------------------------------------------------------------------------------ estimators

def p_value_eps_delta(num_canaries: int, num_guesses: int, num_correct: int, epsilon: float, delta: float) -> float:
    """Probability of ≥ ``num_correct`` correct out of ``num_guesses`` guesses under (ε, δ)-DP (upper bound)."""
    q = 1.0 / (1.0 + math.exp(-epsilon))
    beta = float(stats.binom.sf(num_correct - 1, num_guesses, q))
    if delta <= 0:
        return min(beta, 1.0)
    alpha, acc = 0.0, 0.0
    for i in range(1, num_correct + 1):
        acc += float(stats.binom.pmf(num_correct - i, num_guesses, q))
        if acc > i * alpha:
            alpha = acc / i
    return min(beta + alpha * delta * 2 * num_canaries, 1.0)


def epsilon_lower_bound(num_canaries: int, num_guesses: int, num_correct: int, *, delta: float = 0.0,
                        confidence: float = 0.95, eps_max: float = 20.0) -> float:
    """Largest ε refuted at the given confidence (0 when nothing can be refuted)."""
    p = 1.0 - confidence
    if num_guesses == 0 or p_value_eps_delta(num_canaries, num_guesses, num_correct, 0.0, delta) >= p:
        return 0.0
    lo, hi = 0.0, eps_max
    if p_value_eps_delta(num_canaries, num_guesses, num_correct, hi, delta) < p:
        return hi
    for _ in range(60):
        mid = 0.5 * (lo + hi)
        if p_value_eps_delta(num_canaries, num_guesses, num_correct, mid, delta) < p:
            lo = mid
        else:
            hi = mid
    return lo


def _gdp_epsilon(mu: float, delta: float) -> float:
    """ε(δ) of a μ-GDP mechanism (inverse of δ(ε) = Φ(−ε/μ + μ/2) − e^ε Φ(−ε/μ − μ/2))."""
    f = lambda e: stats.norm.cdf(-e / mu + mu / 2) - math.exp(e) * stats.norm.cdf(-e / mu - mu / 2) - delta
    lo, hi = 0.0, 1.0
    if f(0.0) <= 0:
        return 0.0
    while f(hi) > 0 and hi < 1e3:
        hi *= 2
    for _ in range(80):
        mid = 0.5 * (lo + hi)
        lo, hi = (mid, hi) if f(mid) > 0 else (lo, mid)
    return hi


def gdp_mu_lower_bound(num_canaries: int, num_guesses: int, num_correct: int, *, confidence: float = 0.95,
                       deltas: Sequence[float] = (1e-2, 1e-3, 1e-4, 1e-5, 1e-6)) -> float:
    """Largest μ such that μ-GDP is refuted: some point (ε_μ(δ), δ) of its privacy profile fails the (ε, δ) test."""
    p = 1.0 - confidence

    def refuted(mu: float) -> bool:
        return any(p_value_eps_delta(num_canaries, num_guesses, num_correct, _gdp_epsilon(mu, d), d) < p for d in deltas)
    if num_guesses == 0 or not refuted(1e-3):
        return 0.0
    lo, hi = 1e-3, 1e-3
    while refuted(hi) and hi < 50:
        lo, hi = hi, hi * 2
    for _ in range(40):
        mid = 0.5 * (lo + hi)
        lo, hi = (mid, hi) if refuted(mid) else (lo, mid)
    return lo


def roc_curve(scores: CanaryScores, flips: CoinFlip):
    """(fpr, tpr, thresholds) of the membership score."""
    s, y = scores.scores, flips.included.astype(bool)
    order = np.argsort(-s)
    tp = np.cumsum(y[order])
    fp = np.cumsum(~y[order])
    return fp / max(1, (~y).sum()), tp / max(1, y.sum()), s[order]


def auc(scores: CanaryScores, flips: CoinFlip) -> float:
    """Area under the ROC curve of the canary scores against the coin flips."""
    fpr, tpr, _ = roc_curve(scores, flips)
    return float(np.trapezoid(np.concatenate([[0], tpr]), np.concatenate([[0], fpr])))


@dataclasses.dataclass(frozen=True)
class OneRunEstimate:
    epsilon_lower_bound: float
    gdp_mu_lower_bound: float
    num_canaries: int
    num_guesses: int
    num_correct: int
    accuracy: float
    confidence: float
    delta: float


def one_run(scores: CanaryScores, *, coin_flip: CoinFlip, num_guesses: int | None = None, delta: float = 0.0,
            confidence: float = 0.95, search: bool = True) -> OneRunEstimate:
    """Audit from one run: guess "in" for the top-k scores and "out" for the bottom-k, abstain elsewhere.

    With ``num_guesses=None`` and ``search=True`` a ladder of k values is tried and the confidence is split across
    them (union bound), so the reported bound stays valid.
    """
    s, y = scores.scores, coin_flip.included.astype(bool)
    m = len(s)
    if m != coin_flip.num_canaries:
        raise ValueError("one score per canary is required")
    order = np.argsort(s)

    def evaluate(k: int, conf: float):
        k = max(1, min(k, m // 2))
        correct = int((~y[order[:k]]).sum() + y[order[-k:]].sum())
        return (epsilon_lower_bound(m, 2 * k, correct, delta=delta, confidence=conf), 2 * k, correct)
    if num_guesses is not None:
        eps, r, v = evaluate(num_guesses // 2, confidence)
    else:
        ladder = sorted({max(1, m // d) for d in (2, 4, 8, 16, 32)}) if search else [m // 2]
        conf = 1.0 - (1.0 - confidence) / len(ladder)
        eps, r, v = max((evaluate(k, conf) for k in ladder), key=lambda t: t[0])
        confidence_used = conf
    mu = gdp_mu_lower_bound(m, r, v, confidence=confidence if num_guesses is not None else confidence_used)
    return OneRunEstimate(eps, mu, m, r, v, v / max(r, 1), confidence, delta)


__all__ = ["CanaryScores", "CoinFlip", "OneRunEstimate", "auc", "canary_scores", "coin_flip", "epsilon_lower_bound",
           "gdp_mu_lower_bound", "gradient_scores", "loss_scores", "one_run", "p_value_eps_delta", "roc_curve"]

from .. import __version__  # noqa: E402
from ..utils.namespaces import submodule as _sub  # noqa: E402

# import paths of the reference: opaque.auditing.attacks.{loss_scores, gradient_scores}, opaque.auditing.one_run.one_run.
# ``auditing.one_run`` stays callable: the namespace forwards a call to the function it holds.
_sub(__name__, "attacks", "Membership scores for canaries.", {"gradient_scores": gradient_scores, "loss_scores": loss_scores})
_sub(__name__, "one_run", "Privacy auditing with one training run.",
     {"one_run": one_run, "OneRunEstimate": OneRunEstimate, "epsilon_lower_bound": epsilon_lower_bound,
      "gdp_mu_lower_bound": gdp_mu_lower_bound, "p_value_eps_delta": p_value_eps_delta}, call=one_run)
_sub(__name__, "types", "Classes of the auditing façade.", {"CanaryScores": CanaryScores, "CoinFlip": CoinFlip, "OneRunEstimate": OneRunEstimate}, bind=False)
