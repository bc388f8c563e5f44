"""DP-FTRL accounting: the matrix mechanism as one Gaussian release, and its amplified variants.

``mf_gaussian(σ, strategy, n_steps=…)`` is a *whole-run* (horizon) process: the entire noisy prefix-sum
release is a single Gaussian mechanism whose effective noise multiplier is ``σ / sensitivity(C)``.  Use
``per_step(...)`` to record it step by step in an :class:`Accountant` (``per_step(h) * n`` evaluates
``h.pld_at(n)``).

Amplification:
  ``poisson(inner, q, n_steps=…)``     cyclic Poisson sampling with ``bands`` = the strategy's band count:
                                        each of the ``ceil(n/bands)`` rounds of a band is a Poisson-subsampled
                                        Gaussian at the band's effective multiplier (Choquette-Choo et al.)
  ``balls_in_bins(inner, num_bins=…, n_steps=…)``   Monte-Carlo PLD of the mixture over bins
  ``b_min_sep(inner, …)``              b-min-sep participation: sensitivity with ``min_sep = b`` (no extra
                                        amplification is claimed beyond the participation constraint)

Parity: packages/opaque-dpftrl/src/opaque/api/accounting/dpftrl/{mechanisms/_mf_gaussian,
amplification/_poisson,amplification/_balls_in_bins,amplification/_b_min_sep}.py.
"""
from __future__ import annotations

import dataclasses
import math

import numpy as np

from ..accounting.core import (DiscretizationConfig, DpHorizonProcess, DpProcess, PerStep, get_discretization, native,
                               per_step, register_process_codec)
from . import _transcripts
from .noise import MfStrategy, strategy_from_wire, strategy_to_wire


@dataclasses.dataclass(frozen=True)
class MfGaussian(DpHorizonProcess):
    noise_multiplier: float
    strategy: MfStrategy
    n_steps: int = 1
    min_sep: int = 1
    max_participations: int | None = None

    def __post_init__(self):
        if self.noise_multiplier < 0:
            raise ValueError(f"noise_multiplier must be non-negative, got {self.noise_multiplier}")
        if self.n_steps < 1 or self.min_sep < 1:
            raise ValueError("n_steps and min_sep must be >= 1")

    def effective_noise_multiplier(self, n_steps: int | None = None) -> float:
        n = n_steps or self.n_steps
        return self.noise_multiplier / self.strategy.sensitivity(n, self.min_sep, self.max_participations)

    def pld_at(self, n_steps: int, config: DiscretizationConfig | None = None):
        cfg = config or get_discretization()
        if self.noise_multiplier == 0:
            return native.nonprivate_pld(cfg.to_native())
        return native.gaussian_pld(self.effective_noise_multiplier(n_steps), cfg.to_native())

    def _build_pld(self, config):
        return self.pld_at(self.n_steps, config)


register_process_codec(
    MfGaussian,
    lambda p: {"noise_multiplier": p.noise_multiplier, "strategy": strategy_to_wire(p.strategy), "n_steps": p.n_steps,
               "min_sep": p.min_sep, "max_participations": p.max_participations},
    lambda w: MfGaussian(w["noise_multiplier"], strategy_from_wire(w["strategy"]), w.get("n_steps", 1),
                         w.get("min_sep", 1), w.get("max_participations")))


@dataclasses.dataclass(frozen=True)
class CyclicPoisson(DpHorizonProcess):
    """Banded MF under cyclic Poisson sampling (``bands`` partitions, rate ``q`` within the active one)."""
    inner: MfGaussian
    sample_rate: float
    n_steps: int
    bands: int = 1
    truncated_batch_size: int | None = None
    dataset_size: int | None = None

    @property
    def min_sep(self) -> int:
        return self.bands

    @property
    def max_participations(self) -> int:
        return -(-self.n_steps // self.bands)

    @property
    def atomic_unit(self) -> int:
        return self.bands

    def __post_init__(self):
        if not 0 < self.sample_rate <= 1:
            raise ValueError("sample_rate must be in (0, 1]")

    def pld_at(self, n_steps: int, config: DiscretizationConfig | None = None):
        cfg = config or get_discretization()
        b = self.bands
        # one record can only be hit in the steps of its own partition; with a b-banded C those steps'
        # columns are orthogonal, so each visit is an independent subsampled Gaussian with the column norm
        # as sensitivity; there are ceil(n / b) visits.
        col = math.sqrt(float(native.single_participation_sensitivity_squared(
            self.inner.strategy.gram_matrix(min(n_steps, 4 * b + 8)).reshape(-1).tolist(), min(n_steps, 4 * b + 8))))
        nm = self.inner.noise_multiplier / col
        visits = math.ceil(n_steps / b)
        if self.truncated_batch_size is not None and self.dataset_size is not None:
            base = native.truncated_poisson_gaussian_pld(nm, self.sample_rate, self.truncated_batch_size,
                                                         max(1, self.dataset_size // b), cfg.to_native())
        else:
            base = native.poisson_gaussian_pld(nm, self.sample_rate, cfg.to_native())
        return base if visits == 1 else base.self_compose(visits)

    def _build_pld(self, config):
        return self.pld_at(self.n_steps, config)


@dataclasses.dataclass(frozen=True)
class BallsInBins(DpHorizonProcess):
    inner: MfGaussian
    num_bins: int
    n_steps: int

    @property
    def min_sep(self) -> int:
        """Steps between two participations of a record: the number of bins."""
        return self.num_bins

    @property
    def max_participations(self) -> int:
        return -(-self.n_steps // self.num_bins)

    @property
    def num_epochs(self) -> float:
        return self.n_steps / self.num_bins

    @property
    def atomic_unit(self) -> int:
        """Steps after which the participation pattern repeats (one pass over the bins)."""
        return self.num_bins

    def pld_at(self, n_steps: int, config: DiscretizationConfig | None = None):
        cfg = config or get_discretization()
        g = self.inner.strategy.gram_matrix(n_steps)
        return native.balls_in_bins_mc_pld(np.asarray(g, float).reshape(-1).tolist(), n_steps, min(self.num_bins, n_steps),
                                           self.inner.noise_multiplier, cfg.to_native())

    def _build_pld(self, config):
        return self.pld_at(self.n_steps, config)


def _strategy_process_codec(cls):
    register_process_codec(
        cls,
        lambda p: {**{f.name: getattr(p, f.name) for f in dataclasses.fields(p) if f.name != "inner"},
                   "inner": {"type": "MfGaussian", "noise_multiplier": p.inner.noise_multiplier,
                             "strategy": strategy_to_wire(p.inner.strategy), "n_steps": p.inner.n_steps,
                             "min_sep": p.inner.min_sep, "max_participations": p.inner.max_participations}},
        lambda w: cls(inner=MfGaussian(w["inner"]["noise_multiplier"], strategy_from_wire(w["inner"]["strategy"]),
                                       w["inner"].get("n_steps", 1), w["inner"].get("min_sep", 1),
                                       w["inner"].get("max_participations")),
                      **{k: v for k, v in w.items() if k != "inner"}))


_strategy_process_codec(CyclicPoisson)
_strategy_process_codec(BallsInBins)


def mf_gaussian(noise_multiplier: float, strategy: MfStrategy, *, n_steps: int = 1, min_sep: int = 1,
                max_participations: int | None = None) -> MfGaussian:
    """A matrix-factorisation Gaussian mechanism: the noise multiplier is divided by the strategy's sensitivity under the participation pattern."""
    return MfGaussian(float(noise_multiplier), strategy, int(n_steps), int(min_sep), max_participations)


def poisson(inner: MfGaussian, sample_rate: float, *, n_steps: int, truncated_batch_size: int | None = None,
            dataset_size: int | None = None) -> CyclicPoisson:
    """Poisson subsampling of ``inner`` at ``sample_rate`` (optionally with a truncated batch size)."""
    bands = int(getattr(inner.strategy, "bands", getattr(inner.strategy, "bandwidth", 1)))
    return CyclicPoisson(inner, float(sample_rate), int(n_steps), bands, truncated_batch_size, dataset_size)


def balls_in_bins(inner: MfGaussian, *, num_bins: int, n_steps: int) -> BallsInBins:
    """Balls-in-bins participation (each record lands in one of ``num_bins`` steps per epoch) over a matrix-factorisation mechanism, Monte-Carlo PLD."""
    return BallsInBins(inner, int(num_bins), int(n_steps))


@dataclasses.dataclass(frozen=True)
class BMinSep(DpHorizonProcess):
    """Banded MF under b-min-sep subsampling: a free record joins a step with probability ``sampling_prob`` and is
    then barred for ``bands − 1`` steps.  Monte-Carlo PLD from the backward likelihood-ratio recursion (valid when the
    strategy has at most ``bands`` non-zero coefficients, so the columns of two participations never overlap)."""
    inner: MfGaussian
    bands: int
    n_steps: int
    sampling_prob: float
    warm_start: bool = False

    @property
    def min_sep(self) -> int:
        return self.bands

    @property
    def max_participations(self) -> int:
        return -(-self.n_steps // self.bands)

    @property
    def atomic_unit(self) -> int:
        return self.bands

    @property
    def p0(self) -> float:
        """Stationary per-example participation rate ``p / (1 + p·(bands − 1))``."""
        return self.sampling_prob / (1.0 + self.sampling_prob * max(0, self.bands - 1))

    def __post_init__(self):
        if self.bands < 1 or not 0 < self.sampling_prob <= 1:
            raise ValueError("need bands >= 1 and sampling_prob in (0, 1]")

    def pld_at(self, n_steps: int, config: DiscretizationConfig | None = None):
        cfg = config or get_discretization()
        coef = np.trim_zeros(np.asarray(self.inner.strategy.coefficients(n_steps), float), "b")
        if len(coef) > self.bands:
            raise ValueError(f"the strategy has {len(coef)} bands but the minimum separation is {self.bands}")
        ncfg = cfg.to_native()
        nm = self.inner.noise_multiplier
        # stored transcripts: every probe of a calibration search re-weights the same samples; when they would not fit
        # the registry's byte cap the streaming accountant draws the same samples without keeping them
        out = _transcripts.with_corpus(coef.tolist(), n_steps, self.bands, self.sampling_prob, self.warm_start,
                                       ncfg.num_mc_samples, ncfg.seed, lambda corpus: corpus.pld(nm, n_steps, ncfg))
        if out is not None:
            return out
        return native.b_min_sep_mc_pld(coef.tolist(), n_steps, self.bands, self.sampling_prob, nm, self.warm_start, ncfg)

    def _build_pld(self, config):
        return self.pld_at(self.n_steps, config)


_strategy_process_codec(BMinSep)


def b_min_sep(inner: MfGaussian, *, bands: int, n_steps: int, max_participations: int | None = None,
              sampling_prob: float | None = None, warm_start: bool = False, p0: float | None = None):
    """b-min-sep participation.  With ``sampling_prob`` the amplified Monte-Carlo accountant is used; without it the
    scheme is only a sensitivity constraint on the un-amplified mechanism (an upper bound for any sampling rate).

    ``p0`` states the rate the other way round: the STATIONARY per-example participation rate (expected batch size over
    the number of records).  A record that is available is then included with probability ``p0 / (1 − p0·(bands − 1))``,
    which is what ``sampling_prob`` means; give one of the two."""
    if p0 is not None:
        if sampling_prob is not None:
            raise ValueError("give sampling_prob or p0, not both")
        if not 0.0 < p0 < 1.0 or (bands > 1 and p0 * (bands - 1) >= 1.0):
            raise ValueError(f"p0={p0} is infeasible for bands={bands}: need 0 < p0 < 1/(bands-1)")
        sampling_prob = p0 / (1.0 - p0 * (bands - 1))
    if sampling_prob is not None:
        return BMinSep(inner, int(bands), int(n_steps), float(sampling_prob), bool(warm_start))
    return dataclasses.replace(inner, n_steps=int(n_steps), min_sep=int(bands), max_participations=max_participations)


__all__ = ["BMinSep", "BallsInBins", "CyclicPoisson", "MfGaussian", "b_min_sep", "balls_in_bins", "mf_gaussian", "per_step",
           "poisson"]

from ..utils.namespaces import submodule as _sub  # noqa: E402

_sub(__name__, "mechanisms", "DP-FTRL base mechanism.", {"mf_gaussian": mf_gaussian})
_sub(__name__, "amplification", "Amplified accounting for DP-FTRL samplers.",
     {"b_min_sep": b_min_sep, "balls_in_bins": balls_in_bins, "poisson": poisson})
_sub(__name__, "types", "Process classes of DP-FTRL accounting.", {"BMinSep": BMinSep, "BallsInBins": BallsInBins, "CyclicPoisson": CyclicPoisson,
                                                                   "MfGaussian": MfGaussian}, bind=False)
_sub(__name__ + ".mechanisms", "types", "Mechanism classes.", {"MfGaussian": MfGaussian}, bind=False)
_sub(__name__ + ".amplification", "types", "Amplification classes.", {"BMinSep": BMinSep, "BallsInBins": BallsInBins, "CyclicPoisson": CyclicPoisson}, bind=False)
