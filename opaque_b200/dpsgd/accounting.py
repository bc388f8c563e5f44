"""DP-SGD accounting front-ends: Gaussian mechanism, AdaClip transformation and sampling amplifications.

``poisson(gaussian(σ), q) * steps`` is the standard DP-SGD accountant.  Amplifications wrap a
``Gaussian`` (or ``AdaClip`` of a Gaussian) and lower to the matching native subsampled-Gaussian PLD.

Parity: packages/opaque-dpsgd/src/opaque/api/accounting/dpsgd/{mechanisms,amplification}/*.py.
"""
from __future__ import annotations

import dataclasses

from ..accounting.core import DpProcess, native


@dataclasses.dataclass(frozen=True)
class Gaussian(DpProcess):
    noise_multiplier: float

    def __post_init__(self):
        if not self.noise_multiplier > 0:
            raise ValueError(f"noise_multiplier must be > 0, got {self.noise_multiplier}")

    @property
    def effective_noise_multiplier(self) -> float:
        return self.noise_multiplier

    def _build_pld(self, config):
        return native.gaussian_pld(self.noise_multiplier, config.to_native())


@dataclasses.dataclass(frozen=True)
class AdaClip(DpProcess):
    """Gaussian step that also releases the noisy clipped-fraction of adaptive clipping.

    The pair is equivalent to one Gaussian with ``z_eff = (1/z² + K/(4σ_b²))^{-1/2}``,
    ``σ_b = expected_batch_size · fraction_noise_std`` and K groups.
    """
    inner: Gaussian
    fraction_noise_std: float
    expected_batch_size: float
    num_groups: int = 1

    @property
    def effective_noise_multiplier(self) -> float:
        return native.adaclip_effective_noise_multiplier(self.inner.noise_multiplier, self.fraction_noise_std,
                                                         self.expected_batch_size, self.num_groups)

    def _build_pld(self, config):
        return native.gaussian_pld(self.effective_noise_multiplier, config.to_native())


def _nm(inner: DpProcess) -> float:
    nm = getattr(inner, "effective_noise_multiplier", None)
    if nm is None:
        raise TypeError(f"amplification needs a Gaussian-type inner mechanism, got {type(inner).__name__}")
    return float(nm)


@dataclasses.dataclass(frozen=True)
class Poisson(DpProcess):
    inner: DpProcess
    sample_rate: float
    truncated_batch_size: int | None = None
    dataset_size: int | None = None

    def __post_init__(self):
        _nm(self.inner)
        if not 0 < self.sample_rate <= 1:
            raise ValueError(f"sample_rate must be in (0, 1], got {self.sample_rate}")
        if (self.truncated_batch_size is None) != (self.dataset_size is None):
            raise ValueError("truncated_batch_size and dataset_size must be given together")

    def _build_pld(self, config):
        if self.truncated_batch_size is not None:
            return native.truncated_poisson_gaussian_pld(_nm(self.inner), self.sample_rate, self.truncated_batch_size,
                                                         self.dataset_size, config.to_native())
        return native.poisson_gaussian_pld(_nm(self.inner), self.sample_rate, config.to_native())


@dataclasses.dataclass(frozen=True)
class ParallelPoisson(DpProcess):
    """W workers each Poisson-sample the SAME global dataset; a record can be hit by several of them."""
    inner: DpProcess
    sample_rate: float
    num_workers: int

    def __post_init__(self):
        _nm(self.inner)
        if not 0 < self.sample_rate < 1 or self.num_workers < 1:
            raise ValueError("need sample_rate in (0, 1) and num_workers >= 1")

    def _build_pld(self, config):
        return native.parallel_poisson_gaussian_pld(_nm(self.inner), self.sample_rate, self.num_workers, config.to_native())


@dataclasses.dataclass(frozen=True)
class RandomAllocation(DpProcess):
    """One epoch of ``num_bins`` steps in which each record takes part in exactly ``k`` of them."""
    inner: DpProcess
    num_bins: int
    k: int = 1

    def __post_init__(self):
        _nm(self.inner)
        if not 1 <= self.k <= self.num_bins:
            raise ValueError("need 1 <= k <= num_bins")

    def _build_pld(self, config):
        return native.random_allocation_gaussian_pld(_nm(self.inner), self.num_bins, self.k, config.to_native())

    # the reference's names: one epoch = ``num_bins`` steps in which a record takes part ``k`` times
    @property
    def steps_per_epoch(self) -> int:
        return self.num_bins

    @property
    def total_participations(self) -> int:
        return self.k

    @property
    def n_steps(self) -> int:
        return self.num_bins

    @property
    def num_epochs(self) -> int:
        return 1


def gaussian(noise_multiplier: float) -> Gaussian:
    """One Gaussian release with the given noise multiplier (sensitivity 1)."""
    return Gaussian(float(noise_multiplier))


def adaclip(inner: Gaussian, *, fraction_noise_std: float, expected_batch_size: float, num_groups: int = 1) -> AdaClip:
    """Gaussian release under AdaClip-style adaptive clipping: the effective noise multiplier accounts for the noised clip-fraction query."""
    return AdaClip(inner, float(fraction_noise_std), float(expected_batch_size), int(num_groups))


def poisson(inner: DpProcess, sample_rate: float, *, truncated_batch_size: int | None = None,
            dataset_size: int | None = None) -> Poisson:
    """Poisson subsampling of ``inner`` at ``sample_rate`` (optionally with a truncated batch size)."""
    return Poisson(inner, float(sample_rate), truncated_batch_size, dataset_size)


def parallel_poisson(inner: DpProcess, sample_rate: float, num_workers: int) -> ParallelPoisson:
    """``num_workers`` workers each Poisson-sample the SAME dataset at ``sample_rate``; a record can be hit by several of them in one step."""
    return ParallelPoisson(inner, float(sample_rate), int(num_workers))


def random_allocation(inner: DpProcess, num_bins: int, n_steps: int | None = None) -> DpProcess:
    """Whole-epoch process: do NOT multiply by the steps of the epoch, multiply by the number of epochs.

    With ``n_steps`` (the reference's horizon form) the result already covers ``ceil(n_steps / num_bins)`` epochs — a
    started epoch is charged in full, which bounds a run that stops inside it."""
    epoch = RandomAllocation(inner, int(num_bins), 1)
    if n_steps is None:
        return epoch
    epochs = max(-(-int(n_steps) // int(num_bins)), 1)
    return epoch if epochs == 1 else epoch * epochs


def k_out_of_t(inner: DpProcess, k: int | None = None, t: int | None = None, *, total_participations: int | None = None,
               n_steps: int | None = None) -> RandomAllocation:
    """Each record participates in exactly ``k`` of every ``t`` steps (fixed-participation sampling).  The reference's
    keywords name the whole-run form: ``total_participations`` of ``n_steps`` steps (``k = total_participations, t = n_steps``)."""
    if total_participations is not None or n_steps is not None:
        if k is not None or t is not None or total_participations is None or n_steps is None:
            raise ValueError("give (k, t) or (total_participations=, n_steps=)")
        k, t = total_participations, n_steps
    if k is None or t is None:
        raise ValueError("give (k, t) or (total_participations=, n_steps=)")
    return RandomAllocation(inner, int(t), int(k))


__all__ = ["AdaClip", "Gaussian", "ParallelPoisson", "Poisson", "RandomAllocation", "adaclip", "gaussian", "k_out_of_t",
           "parallel_poisson", "poisson", "random_allocation"]

from ..utils.namespaces import submodule as _sub  # noqa: E402

_sub(__name__, "mechanisms", "DP-SGD base mechanisms.", {"adaclip": adaclip, "gaussian": gaussian})
_sub(__name__, "amplification", "Amplification by sampling.",
     {"k_out_of_t": k_out_of_t, "parallel_poisson": parallel_poisson, "poisson": poisson, "random_allocation": random_allocation})
KOutOfT = RandomAllocation          # k-out-of-t participation is accounted as a random-allocation process
_sub(__name__, "types", "Process classes of DP-SGD accounting.", {"AdaClip": AdaClip, "Gaussian": Gaussian, "KOutOfT": KOutOfT,
                                                                  "ParallelPoisson": ParallelPoisson, "Poisson": Poisson, "RandomAllocation": RandomAllocation}, bind=False)
_sub(__name__ + ".mechanisms", "types", "Mechanism classes.", {"AdaClip": AdaClip, "Gaussian": Gaussian}, bind=False)
_sub(__name__ + ".amplification", "types", "Amplification classes.", {"KOutOfT": KOutOfT, "ParallelPoisson": ParallelPoisson, "Poisson": Poisson,
                                                                      "RandomAllocation": RandomAllocation}, bind=False)
