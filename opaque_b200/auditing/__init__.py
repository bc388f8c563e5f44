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

    # the reference's names for the same partition
    @property
    def in_indices(self) -> np.ndarray:
        """Dataset indices of the canaries whose coin came up "in" (they are trained on)."""
        return self.canary_indices[self.included]

    @property
    def out_indices(self) -> np.ndarray:
        """Dataset indices of the canaries that are held out."""
        return self.canary_indices[~self.included]

    def train_indices(self, dataset_size: int | None = None) -> list[int]:
        """Dataset indices to train on (``dataset_size`` must agree with the partition's when given)."""
        if dataset_size is not None and int(dataset_size) != self.dataset_size:
            raise ValueError(f"the partition was drawn for {self.dataset_size} records, not {dataset_size}")
        return self.kept_indices().tolist()

    def train_subset(self, dataset: Any):
        """``torch.utils.data.Subset`` of ``dataset`` holding the records to train on."""
        return torch.utils.data.Subset(dataset, self.train_indices(len(dataset)))

    def split_scores(self, scores: "CanaryScores") -> tuple[np.ndarray, np.ndarray]:
        """``(scores of the included canaries, scores of the held-out canaries)``, joined by identifier when present."""
        s = scores.aligned_to(self)
        return s[self.included], s[~self.included]


@dataclasses.dataclass(frozen=True)
class CanaryScores:
    """One membership score per canary (higher = more likely included).  With ``canary_indices`` (the dataset index behind
    each score, any order) the scores are joined to a ``CoinFlip`` by identifier; without, they must already be in the
    order of ``CoinFlip.canary_indices``."""
    scores: np.ndarray
    canary_indices: np.ndarray | None = None

    def __post_init__(self):
        object.__setattr__(self, "scores", np.asarray(self.scores, dtype=np.float64).reshape(-1))
        if self.canary_indices is not None:
            ids = np.asarray(self.canary_indices)
            if ids.ndim != 1 or not np.issubdtype(ids.dtype, np.integer):
                raise ValueError("canary_indices must be a 1-D integer array")
            if len(ids) != len(self.scores) or len(np.unique(ids)) != len(ids):
                raise ValueError("one distinct canary index per score is required")
            object.__setattr__(self, "canary_indices", ids.astype(np.int64))

    def aligned_to(self, coin_flip: "CoinFlip") -> np.ndarray:
        """The scores in the order of ``coin_flip.canary_indices`` (joined by identifier when identifiers are attached)."""
        if self.canary_indices is None:
            return self.scores
        pos = {int(i): k for k, i in enumerate(self.canary_indices)}
        try:
            return self.scores[[pos[int(i)] for i in coin_flip.canary_indices]]
        except KeyError as exc:
            raise ValueError(f"no score for canary {exc.args[0]}") from None


def canary_scores(scores: Any, *, canary_indices: Any = None) -> CanaryScores:
    """Wrap an array or tensor of per-canary scores as ``CanaryScores``; ``canary_indices`` attests which dataset index
    each score belongs to (scores computed by another pipeline, in whatever order)."""
    if isinstance(scores, torch.Tensor):
        scores = scores.detach().float().cpu().numpy()
    if isinstance(canary_indices, torch.Tensor):
        canary_indices = canary_indices.cpu().numpy()
    return CanaryScores(np.asarray(scores), None if canary_indices is None else np.asarray(canary_indices))


def coin_flip(dataset: Any, *, num_canaries: int, key: RngKey) -> CoinFlip:
    """Choose ``num_canaries`` records uniformly and flip a fair coin for each."""
    n = len(dataset)
    if not 1 <= num_canaries <= n:
        raise ValueError("num_canaries must be in [1, len(dataset)]")
    rng = np.random.default_rng(fold_in(key, "audit_coin_flip").seed)
    idx = np.sort(rng.choice(n, size=num_canaries, replace=False))
    return CoinFlip(idx, rng.random(num_canaries) < 0.5, n)


def _dataset_scores(per_example, loss_fn, args, batch_argnums, coin_flip, dataset, reference_scores, batch_size, collate_fn) -> CanaryScores:
    """Shared driver of the dataset forms of ``loss_scores`` / ``gradient_scores``: batches of canaries through
    ``collate_fn``, one score per canary from ``per_example(call_args, in_dims)``, identifiers attached, reference subtracted."""
    argnums = tuple(batch_argnums)
    if not argnums or list(argnums) != sorted(set(argnums)) or min(argnums) < 0:
        raise ValueError("batch_argnums must be sorted, unique and non-negative")
    if not isinstance(batch_size, int) or isinstance(batch_size, bool):
        raise TypeError("batch_size must be an int")
    if batch_size < 1:
        raise ValueError("batch_size must be positive")
    if reference_scores is not None and reference_scores.canary_indices is None:
        raise TypeError("reference_scores must carry canary identifiers (scores returned by the dataset form do)")
    collate = collate_fn or torch.utils.data.default_collate
    ids = [int(i) for i in coin_flip.canary_indices]
    total = len(args) + len(argnums)
    out: list[torch.Tensor] = []
    for lo in range(0, len(ids), batch_size):
        chunk = ids[lo:lo + batch_size]
        batch = collate([dataset[i] for i in chunk])
        parts = [batch] if len(argnums) == 1 else list(batch)
        if len(parts) != len(argnums):
            raise ValueError(f"collate_fn returned {len(parts)} batch arguments for batch_argnums={argnums}")
        fixed = iter(args)
        call = [parts[argnums.index(p)] if p in argnums else next(fixed) for p in range(total)]
        in_dims = tuple(0 if p in argnums else None for p in range(total))
        vals = per_example(call, in_dims).detach().float().reshape(-1).cpu()
        if vals.numel() != len(chunk):
            raise ValueError("collate_fn changed the number of rows of a batch")
        out.append(vals)
    scores = -torch.cat(out).numpy() if out else np.zeros(0)
    result = CanaryScores(scores, np.asarray(ids, dtype=np.int64))
    if reference_scores is not None:
        result = CanaryScores(result.scores - reference_scores.aligned_to(coin_flip), result.canary_indices)
    return result


def loss_scores(loss_fn: Callable[..., torch.Tensor], *args: Any, batch_argnums: Sequence[int] | None = None,
                coin_flip: "CoinFlip | None" = None, dataset: Any = None, reference_scores: CanaryScores | None = None,
                batch_size: int = 32, collate_fn: Callable | None = None, baseline_losses: Any = None) -> CanaryScores:
    """Score = −loss of the trained model on the canary.

    Two forms.  ``loss_scores(loss_fn, canaries, baseline_losses=None)``: ``loss_fn(canary)`` for every element of a list,
    in the order of ``CoinFlip.canary_indices``.  Dataset form (the reference's):
    ``loss_scores(loss_fn, *fixed_args, batch_argnums=(1,), coin_flip=flips, dataset=data)`` — ``loss_fn`` is written for
    ONE example (as for ``clipped_grad``), the canaries of ``dataset`` are collated ``batch_size`` at a time and mapped
    with ``vmap``; the result carries each canary's dataset index, and ``reference_scores`` (the same call on the
    untrained model) is subtracted by identifier.

    Parity: packages/opaque-auditing/src/opaque/api/auditing/attacks/_loss.py:30."""
    if coin_flip is not None or dataset is not None or batch_argnums is not None:
        if coin_flip is None or dataset is None or batch_argnums is None:
            raise ValueError("the dataset form needs batch_argnums=, coin_flip= and dataset=")

        def per_example(call, in_dims):
            with torch.no_grad():
                return torch.func.vmap(loss_fn, in_dims=in_dims)(*call)
        return _dataset_scores(per_example, loss_fn, args, batch_argnums, coin_flip, dataset, reference_scores, batch_size, collate_fn)
    if len(args) != 1:
        raise TypeError("loss_scores(loss_fn, canaries) takes one list of canaries (or use the dataset form)")
    canaries = args[0]
    with torch.no_grad():
        losses = np.array([float(loss_fn(c)) for c in canaries])
    if baseline_losses is not None:
        losses = losses - np.asarray(baseline_losses, dtype=np.float64)
    return CanaryScores(-losses)


def gradient_scores(*args: Any, batch_argnums: Sequence[int] | None = None, coin_flip: "CoinFlip | None" = None,
                    dataset: Any = None, reference_scores: CanaryScores | None = None, batch_size: int = 32,
                    collate_fn: Callable | None = None) -> CanaryScores:
    """Two forms.  ``gradient_scores(canary_grads, released_updates)``: score = Σ_t ⟨g_canary,t , released_t⟩ — the canary's
    gradient direction shows up in the noisy sums it joined (white-box, needs the released updates).  Dataset form (the
    reference's): ``gradient_scores(loss_fn, params, *fixed_args, batch_argnums=(1,), coin_flip=flips, dataset=data)`` —
    score = −‖∇_params loss(example)‖², one example at a time (a member's gradient is smaller after training);
    ``reference_scores`` from the untrained model are subtracted by identifier.

    Parity: packages/opaque-auditing/src/opaque/api/auditing/attacks/_gradient.py:35."""
    if coin_flip is not None or dataset is not None or batch_argnums is not None:
        if coin_flip is None or dataset is None or batch_argnums is None or len(args) < 2:
            raise ValueError("the dataset form is gradient_scores(loss_fn, params, ..., batch_argnums=, coin_flip=, dataset=)")
        if 0 in tuple(batch_argnums):
            raise ValueError("position 0 is the parameters: it cannot be a batch argument")
        loss_fn, fixed = args[0], args[1:]
        from ..pytree import tree_leaves
        grad_fn = torch.func.grad(loss_fn, argnums=0)

        def per_example(call, in_dims):
            rows = next(len(tree_leaves(call[p])[0]) for p, d in enumerate(in_dims) if d == 0)
            vals = []
            for i in range(rows):
                one = [tree_map_index(c, i) if d == 0 else c for c, d in zip(call, in_dims)]
                g = grad_fn(*one)
                vals.append(sum(float((x.detach().float() ** 2).sum()) for x in tree_leaves(g) if isinstance(x, torch.Tensor)))
            return torch.tensor(vals)
        return _dataset_scores(per_example, loss_fn, fixed, batch_argnums, coin_flip, dataset, reference_scores, batch_size, collate_fn)
    if len(args) != 2:
        raise TypeError("gradient_scores(canary_grads, released_updates) takes two sequences (or use the dataset form)")
    canary_grads, released_updates = args

    def flat(tree):
        from ..pytree import tree_leaves
        return torch.cat([x.detach().float().reshape(-1).cpu() for x in tree_leaves(tree) if isinstance(x, torch.Tensor)])
    out = []
    for per_canary in canary_grads:
        steps = per_canary if isinstance(per_canary, (list, tuple)) else [per_canary] * len(released_updates)
        out.append(sum(float(flat(g) @ flat(u)) for g, u in zip(steps, released_updates)))
    return CanaryScores(np.array(out))


def tree_map_index(tree: Any, i: int) -> Any:
    """Row ``i`` of every tensor leaf of a batch."""
    from ..pytree import tree_map
    return tree_map(lambda x: x[i] if isinstance(x, torch.Tensor) else x, tree)


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


def _gdp_delta(mu: float, epsilon: float) -> float:
    """δ(ε) of μ-GDP: ``Φ(−ε/μ + μ/2) − e^ε Φ(−ε/μ − μ/2)``."""
    if mu <= 0:
        return 0.0
    return float(stats.norm.cdf(-epsilon / mu + mu / 2) - math.exp(epsilon) * stats.norm.cdf(-epsilon / mu - mu / 2))


def _gdp_epsilon(mu: float, delta: float) -> float:
    """The ε at which μ-GDP has exactly ``delta`` (0 when even ε = 0 needs less)."""
    if mu <= 0 or _gdp_delta(mu, 0.0) <= delta:
        return 0.0
    lo, hi = 0.0, 1.0
    while _gdp_delta(mu, hi) > delta and hi < 1e6:
        hi *= 2.0
    for _ in range(200):
        mid = 0.5 * (lo + hi)
        lo, hi = (mid, hi) if _gdp_delta(mu, mid) > delta else (lo, mid)
    return lo


@dataclasses.dataclass(frozen=True)
class EpsDeltaMethod:
    """(ε, δ) audit from ALL canaries at one threshold (order-statistics test of Xiang et al. 2025 for the (ε, δ) trade-off
    curve): every canary is guessed "in" when its score reaches the threshold, and under (ε, δ)-DP the number of wrong
    guesses among the ``m − round(m·δ)`` ranks outside the point mass dominates a Binomial with success probability
    ``1 / (1 + e^ε)``.  The largest ε whose p-value stays below ``significance`` is the lower bound.  Without
    ``threshold`` the one with the most correct guesses is taken, as the reference does
    (reference: auditing/one_run/_eps_delta.py, _estimate.py ``_best_r_u``)."""
    estimate: "OneRunEstimate"

    def guesses_and_errors(self, threshold: float | None = None) -> tuple[int, int]:
        a, b = np.asarray(self.estimate.in_scores, float), np.asarray(self.estimate.out_scores, float)
        m = len(a) + len(b)
        if threshold is not None:
            return m, m - int((a >= threshold).sum()) - int((b < threshold).sum())
        cuts = np.unique(np.r_[a, b, np.inf])                     # "in" iff score >= cut; +inf: everything "out"
        a_sorted, b_sorted = np.sort(a), np.sort(b)
        correct = (len(a) - np.searchsorted(a_sorted, cuts, "left")) + np.searchsorted(b_sorted, cuts, "left")
        return m, m - int(correct.max())

    @staticmethod
    def p_value(guesses: int, errors: int, epsilon: float, delta: float) -> float:
        trials = max(guesses - round(guesses * delta), 0)
        return 1.0 if trials == 0 else float(stats.binom.cdf(errors, trials, 1.0 / (1.0 + math.exp(max(epsilon, 0.0)))))

    @staticmethod
    def _check(significance: float, delta: float = 0.0) -> None:
        if not 0 < significance < 0.5:
            raise ValueError(f"significance must be in (0, 0.5), got {significance}")
        if not 0 <= delta <= 1:
            raise ValueError(f"delta must be in [0, 1], got {delta}")

    def epsilon_at(self, *, delta: float = 0.0, significance: float = 0.05, threshold: float | None = None) -> float:
        self._check(significance, delta)
        r, u = self.guesses_and_errors(threshold)
        trials = max(r - round(r * delta), 1)
        hi = max(1.1 * -math.log(significance ** (-1.0 / trials) - 1.0), 1.0)      # a perfect attack certifies no more
        lo = 0.0
        while hi - lo > 1e-4:
            mid = 0.5 * (lo + hi)
            lo, hi = (mid, hi) if self.p_value(r, u, mid, delta) < significance else (lo, mid)
        return lo

    def delta_at(self, *, epsilon: float, significance: float = 0.05, threshold: float | None = None) -> float:
        """Largest δ at which ``epsilon`` is still refuted (0 when it is not refuted even at δ = 0)."""
        self._check(significance)
        if epsilon < 0:
            raise ValueError(f"epsilon must be >= 0, got {epsilon}")
        r, u = self.guesses_and_errors(threshold)
        if self.p_value(r, u, epsilon, 0.0) >= significance:
            return 0.0
        lo, hi = 0.0, 1.0
        while hi - lo > 1e-6:
            mid = 0.5 * (lo + hi)
            lo, hi = (mid, hi) if self.p_value(r, u, epsilon, mid) < significance else (lo, mid)
        return lo


MAX_EXACT_RANKS = 2000      # ranks beyond this many get the trivial error probability 1/2 (keeps the rank × grid table small)


def gdp_rank_error_probabilities(num_canaries: int, ranks: int, mu: float, grid_size: int = 10_000) -> np.ndarray:
    """Under μ-GDP, the probability that the guess for the canary with the k-th smallest |privacy loss| is wrong, for the
    ``ranks`` LARGEST k of ``num_canaries``: ``v_k = E[sigmoid(−|L(Y_(k))|)]`` with ``Y`` drawn from the equal mixture of
    ``N(0, 1)`` and ``N(μ, 1)`` and ``L(z) = μ²/2 − μz`` (Xiang et al. 2025, eq. 12).  The expectation over the order
    statistic's density ``n!/((k−1)!(n−k)!) F^{k−1}(1−F)^{n−k} f`` is a sum over a grid in ``z`` sorted by ``|L|``, in logs."""
    from scipy import special
    n = int(num_canaries)
    z = np.linspace(-6.0, mu + 6.0, int(grid_size))
    mass = 0.5 * (stats.norm.pdf(z) + stats.norm.pdf(z - mu)) * (z[1] - z[0])
    loss = np.abs(0.5 * mu * mu - mu * z)
    order = np.argsort(loss, kind="stable")
    mass, loss = mass[order], loss[order]
    below = np.concatenate([[0.0], np.cumsum(mass)[:-1]])                   # mixture mass with a smaller |L|
    tiny = 1e-300
    log_f, log_lo, log_hi = np.log(np.maximum(mass, tiny)), np.log(np.maximum(below, tiny)), np.log(np.maximum(1.0 - below, tiny))
    k = np.arange(n - ranks + 1, n + 1, dtype=np.float64)[:, None]
    log_count = special.gammaln(n + 1) - special.gammaln(k) - special.gammaln(n - k + 1)
    table = (log_count + log_f[None, :] + np.where(k > 1, (k - 1) * log_lo[None, :], 0.0)
             + np.where(k < n, (n - k) * log_hi[None, :], 0.0) + special.log_expit(-loss)[None, :])
    return np.clip(np.exp(special.logsumexp(table, axis=1)), 0.0, 0.5)


def bernoulli_sum_lower_tail(probabilities: np.ndarray, num_fair: int, observed: int) -> float:
    """Chernoff bound on ``P(Σ X_i ≤ observed)`` for independent ``X_i ~ Bernoulli(p_i)`` plus ``num_fair`` fair coins:
    ``min_{λ ≤ 0} exp(−λ·observed + Σ log(1 − p_i + p_i e^λ))``; 1 when ``observed`` is not below the mean."""
    v = np.asarray(probabilities, float)
    if observed >= float(v.sum()) + 0.5 * num_fair:
        return 1.0
    if observed == 0:
        return min(math.exp(float(np.log(np.maximum(1.0 - v, 1e-300)).sum()) + num_fair * math.log(0.5)), 1.0)

    def slope(lam):                                                         # derivative of the exponent in λ (increasing)
        e = math.exp(lam)
        return -observed + float((v * e / (1.0 - v + v * e)).sum()) + num_fair * e / (1.0 + e)
    lo, hi = -50.0, 0.0
    if slope(lo) >= 0:
        lam = lo
    else:
        while hi - lo >= 1e-10:
            mid = 0.5 * (lo + hi)
            lo, hi = (lo, mid) if slope(mid) > 0 else (mid, hi)
        lam = 0.5 * (lo + hi)
    e = math.exp(lam)
    return min(math.exp(-lam * observed + float(np.log(1.0 - v + v * e).sum()) + num_fair * math.log(0.5 * (1.0 + e))), 1.0)


def gdp_order_statistics_p_value(num_canaries: int, guesses: int, errors: int, mu: float, grid_size: int = 10_000) -> float:
    """P-value of "the mechanism is μ-GDP" given ``errors`` wrong guesses among ``guesses`` (Xiang et al. 2025, theorems 2–3;
    reference: auditing/one_run/_gdp.py ``_p_value``)."""
    if not math.isfinite(mu) or mu <= 0.0:
        return 1.0
    exact = min(int(guesses), MAX_EXACT_RANKS)
    return bernoulli_sum_lower_tail(gdp_rank_error_probabilities(num_canaries, exact, mu, grid_size), int(guesses) - exact, int(errors))


@dataclasses.dataclass(frozen=True)
class GdpMethod:
    """μ-GDP audit from ALL canaries at one threshold: the largest μ whose order-statistics p-value stays below
    ``significance`` (bisection to 1 % of μ), and what μ-GDP at that level means as ε(δ), δ(ε), β(α) and advantage.
    Assumes the audited mechanism is Gaussian-DP-like (DP-SGD and its relatives); :class:`EpsDeltaMethod` assumes nothing."""
    estimate: "OneRunEstimate"
    grid_size: int = 10_000

    def mu_at(self, *, significance: float = 0.05, threshold: float | None = None) -> float:
        EpsDeltaMethod._check(significance)
        r, u = EpsDeltaMethod(self.estimate).guesses_and_errors(threshold)
        m = self.estimate.n_in + self.estimate.n_out
        hi = max(1.1 * -math.log(significance ** (-1.0 / max(m, 1)) - 1.0), 1.0)
        for _ in range(60):
            if gdp_order_statistics_p_value(m, r, u, hi, self.grid_size) >= significance:
                break
            hi *= 2.0
        else:
            raise RuntimeError(f"no finite mu explains {u} errors in {r} guesses at significance {significance}; "
                               f"use fewer canaries or a larger significance")
        lo = 0.0
        for _ in range(100):
            if hi - lo <= 0.01 * max(1.0, hi):
                break
            mid = 0.5 * (lo + hi)
            lo, hi = (mid, hi) if gdp_order_statistics_p_value(m, r, u, mid, self.grid_size) < significance else (lo, mid)
        return lo

    def epsilon_at(self, *, delta: float, significance: float = 0.05, threshold: float | None = None) -> float:
        if not 0 < delta <= 1:
            raise ValueError(f"mu-GDP has no pure-epsilon form: delta must be in (0, 1], got {delta}")
        return _gdp_epsilon(self.mu_at(significance=significance, threshold=threshold), delta)

    def delta_at(self, *, epsilon: float, significance: float = 0.05, threshold: float | None = None) -> float:
        if epsilon < 0:
            raise ValueError(f"epsilon must be >= 0, got {epsilon}")
        return max(0.0, _gdp_delta(self.mu_at(significance=significance, threshold=threshold), epsilon))

    def beta_at(self, *, alpha: float, significance: float = 0.05, threshold: float | None = None) -> float:
        """``Φ(Φ⁻¹(1 − α) − μ)``: the type-II error some attack reaches at false-positive rate ``alpha``."""
        if not 0 <= alpha <= 1:
            raise ValueError(f"alpha must be in [0, 1], got {alpha}")
        return float(stats.norm.cdf(stats.norm.ppf(1.0 - alpha) - self.mu_at(significance=significance, threshold=threshold)))

    def advantage(self, *, significance: float = 0.05, threshold: float | None = None) -> float:
        """Total-variation advantage ``2Φ(μ/2) − 1``."""
        return float(2.0 * stats.norm.cdf(self.mu_at(significance=significance, threshold=threshold) / 2.0) - 1.0)


@dataclasses.dataclass(frozen=True)
class OneRunEstimate:
    """Result of :func:`one_run`.  The fields are the guess-counting audit (Steinke et al. 2023) at the confidence and δ the
    call was given; ``epsilon_at`` / ``gdp_mu`` / ``delta_at`` / ``beta_at`` / ``advantage`` re-run that audit on the stored
    scores at another δ or significance level.  ``eps_delta()`` and ``gdp()`` give the all-canaries order-statistics audits
    (Xiang et al. 2025) that the reference's estimate object is built on, with the reference's numbers."""
    epsilon_lower_bound: float
    gdp_mu_lower_bound: float
    num_canaries: int
    num_guesses: int
    num_correct: int
    accuracy: float
    confidence: float
    delta: float
    in_scores: np.ndarray | None = None          # scores of the canaries that were trained on
    out_scores: np.ndarray | None = None         # scores of the held-out canaries
    canary_indices: np.ndarray | None = None

    def _audit(self, delta: float, significance: float) -> "OneRunEstimate":
        if self.in_scores is None or self.out_scores is None:
            raise ValueError("this estimate carries no scores; build it with one_run()")
        m = len(self.in_scores) + len(self.out_scores)
        flips = CoinFlip(np.arange(m), np.r_[np.ones(len(self.in_scores), bool), np.zeros(len(self.out_scores), bool)], m)
        return one_run(CanaryScores(np.r_[self.in_scores, self.out_scores]), coin_flip=flips, delta=delta, confidence=1.0 - significance)

    def eps_delta(self) -> EpsDeltaMethod:
        """The all-canaries (ε, δ) order-statistics audit on the stored scores; mechanism-agnostic."""
        if self.in_scores is None or self.out_scores is None:
            raise ValueError("this estimate carries no scores; build it with one_run()")
        return EpsDeltaMethod(self)

    def gdp(self, *, grid_size: int = 10_000) -> GdpMethod:
        """The μ-GDP questions as one object (``mu_at``, ``epsilon_at``, ``delta_at``, ``beta_at``, ``advantage``)."""
        if grid_size < 16:
            raise ValueError(f"grid_size must be >= 16, got {grid_size}")
        return GdpMethod(self, int(grid_size))

    @property
    def n_in(self) -> int:
        return 0 if self.in_scores is None else len(self.in_scores)

    @property
    def n_out(self) -> int:
        return 0 if self.out_scores is None else len(self.out_scores)

    def epsilon_at(self, *, delta: float, significance: float = 0.05, threshold: float | None = None) -> float:
        """Lower bound on ε at ``delta``, valid with probability ``1 − significance``."""
        return self._audit(delta, significance).epsilon_lower_bound

    def gdp_mu(self, *, significance: float = 0.05) -> float:
        """Lower bound on the μ of μ-GDP."""
        return self._audit(self.delta, significance).gdp_mu_lower_bound

    def delta_at(self, *, epsilon: float, significance: float = 0.05, threshold: float | None = None) -> float:
        """δ(ε) of the refuted μ-GDP level: the mechanism's δ at this ε is at least this."""
        return _gdp_delta(self.gdp_mu(significance=significance), epsilon)

    def beta_at(self, *, alpha: float, significance: float = 0.05, threshold: float | None = None) -> float:
        """Type-II error at false-positive rate ``alpha`` of the refuted μ-GDP level, ``Φ(Φ⁻¹(1 − α) − μ)``: some attack on
        the mechanism does at least this well."""
        return float(stats.norm.cdf(stats.norm.ppf(1.0 - alpha) - self.gdp_mu(significance=significance)))

    def advantage(self, *, significance: float = 0.05, threshold: float | None = None) -> float:
        """Total-variation advantage of the refuted μ-GDP level, ``2Φ(μ/2) − 1``."""
        return float(2.0 * stats.norm.cdf(self.gdp_mu(significance=significance) / 2.0) - 1.0)

    def attack_auc(self, *, confidence: float | None = None, num_samples: int = 1000, key: RngKey | None = None):
        """Area under the ROC curve of the scores (probability that an included canary outscores a held-out one); with
        ``confidence`` also a bootstrap interval ``(low, high)`` over ``num_samples`` resamples."""
        a, b = np.asarray(self.in_scores), np.asarray(self.out_scores)

        def area(x, y):
            return float(((x[:, None] > y[None, :]).mean() + 0.5 * (x[:, None] == y[None, :]).mean())) if len(x) and len(y) else 0.5
        point = area(a, b)
        if confidence is None:
            return point
        rng = np.random.default_rng(fold_in(key, "attack_auc").seed if key is not None else 0)
        draws = [area(rng.choice(a, len(a)), rng.choice(b, len(b))) for _ in range(int(num_samples))]
        lo, hi = np.quantile(draws, [(1 - confidence) / 2, 1 - (1 - confidence) / 2])
        return point, (float(lo), float(hi))

    def attack_beta_at(self, *, alpha):
        """Empirical attack error: ``1 − TPR`` at false-positive rate ``alpha`` (scalar or array), thresholding the scores."""
        a, b = np.asarray(self.in_scores), np.sort(np.asarray(self.out_scores))
        al = np.atleast_1d(np.asarray(alpha, dtype=float))
        out = []
        for x in al:
            k = int(np.floor(x * len(b)))                       # how many held-out canaries may be flagged
            thr = b[len(b) - k - 1] if k < len(b) else -np.inf  # flag scores strictly above this threshold
            out.append(1.0 - float((a > thr).mean()) if len(a) else 1.0)
        return out[0] if np.ndim(alpha) == 0 else np.asarray(out)


def one_run(scores: CanaryScores, *, coin_flip: CoinFlip, num_guesses: int | None = None, delta: float = 0.0,
            confidence: float = 0.95, search: bool = True) -> OneRunEstimate:
    """Audit from one run: guess "in" for the top-k scores and "out" for the bottom-k, abstain elsewhere.

    With ``num_guesses=None`` and ``search=True`` a ladder of k values is tried and the confidence is split across
    them (union bound), so the reported bound stays valid.
    """
    s, y = scores.aligned_to(coin_flip), coin_flip.included.astype(bool)
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
    return OneRunEstimate(eps, mu, m, r, v, v / max(r, 1), confidence, delta, s[y].copy(), s[~y].copy(),
                          np.asarray(coin_flip.canary_indices).copy())


__all__ = ["CanaryScores", "CoinFlip", "EpsDeltaMethod", "GdpMethod", "OneRunEstimate", "auc", "bernoulli_sum_lower_tail",
           "gdp_order_statistics_p_value", "gdp_rank_error_probabilities", "canary_scores", "coin_flip", "epsilon_lower_bound",
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
