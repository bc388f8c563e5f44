"""Batch samplers for DP-FTRL: each guarantees the participation pattern its accountant assumes.

  CyclicPoissonSampler    the data is cut into ``bands`` parts; step t Poisson-samples part ``t mod bands``,
                           so a record takes part at most once every ``bands`` steps
  BMinSepSampler          Poisson sampling with a cool-down: a sampled record is unavailable for the next
                           ``bands − 1`` steps (b-min-sep participation)
  BallsInBinsSampler      every record is thrown into one of ``num_bins`` bins once; step t uses bin ``t mod num_bins``
  SequentialBatchSampler  fixed-size consecutive batches in a fixed order (deterministic participation)

All are resumable: state = key + ``consumed`` cursor (replayed on load).

Parity: packages/opaque-dpftrl/src/opaque/api/dpftrl/sampling/{_poisson,_b_min_sep,_balls_in_bins,
_sequential,_partitions}.py.
"""
from __future__ import annotations

import enum
from collections.abc import Sized

import numpy as np

from ..dpsgd.sampling import _load_common, _Resumable, _save_common, poisson_step_indices
from ..random import RngKey, fold_in
from ..serialization import register_serializer


class PartitionType(enum.Enum):
    EQUAL_SPLIT = "equal_split"          # contiguous blocks of (almost) equal size
    STRIDED = "strided"                  # record i belongs to part i mod bands


def partition_indices(n: int, parts: int, kind: PartitionType) -> list[np.ndarray]:
    idx = np.arange(n)
    if kind is PartitionType.STRIDED:
        return [idx[p::parts] for p in range(parts)]
    return [a for a in np.array_split(idx, parts)]


class CyclicPoissonSampler(_Resumable):
    def __init__(self, data_source: Sized, sample_rate: float, bands: int = 1, n_steps: int | None = 1,
                 partition_type: PartitionType = PartitionType.EQUAL_SPLIT, truncated_batch_size: int | None = None,
                 *, key: RngKey):
        if not 0 < sample_rate <= 1:
            raise ValueError(f"sample_rate must be in (0, 1], got {sample_rate}")
        if bands < 1:
            raise ValueError("bands must be >= 1")
        self.data_source, self.sample_rate, self.bands, self.n_steps = data_source, sample_rate, bands, n_steps
        self.partition_type, self.truncated_batch_size = partition_type, truncated_batch_size
        self._num_samples = len(data_source)
        if bands > self._num_samples:
            raise ValueError("more bands than records")
        self._parts = partition_indices(self._num_samples, bands, partition_type)
        self._key = key
        self._consumed = 0
        self._reset_generator()

    def _reset_generator(self):
        self.generator = np.random.default_rng(self._key.seed)

    def _draw(self):
        part = self._parts[self._consumed % self.bands]
        local = poisson_step_indices(self.generator, len(part), self.sample_rate, self.truncated_batch_size)
        return part[local].tolist()

    @property
    def expected_batch_size(self) -> float:
        return self._num_samples / self.bands * self.sample_rate

    @property
    def batch_size_variance(self) -> float:
        """Variance of one step's batch size: a Binomial over the records of the step's part (before any truncation)."""
        return self._num_samples / self.bands * self.sample_rate * (1.0 - self.sample_rate)


class BMinSepSampler(_Resumable):
    def __init__(self, data_source: Sized, bands: int, sampling_prob: float, n_steps: int | None, *, key: RngKey):
        if bands < 1 or not 0 < sampling_prob <= 1:
            raise ValueError("need bands >= 1 and sampling_prob in (0, 1]")
        self.data_source, self.bands, self.sampling_prob, self.n_steps = data_source, bands, sampling_prob, n_steps
        self._num_samples = len(data_source)
        self._key = key
        self._consumed = 0
        self._reset_generator()

    def _reset_generator(self):
        self.generator = np.random.default_rng(self._key.seed)
        self._free_at = np.zeros(self._num_samples, dtype=np.int64)   # first step at which a record may be drawn again

    def _draw(self):
        t = self._consumed
        free = self._free_at <= t
        hit = free & (self.generator.random(self._num_samples) < self.sampling_prob)
        self._free_at[hit] = t + self.bands
        return np.flatnonzero(hit).tolist()

    @property
    def stationary_rate(self) -> float:
        """Long-run fraction of steps in which a given record takes part: ``p / (1 + p·(bands − 1))``."""
        return self.sampling_prob / (1.0 + self.sampling_prob * max(0, self.bands - 1))

    @property
    def expected_batch_size(self) -> float:
        """Stationary expected batch size (the first ``bands`` steps, when every record is still free, are larger)."""
        return self._num_samples * self.stationary_rate

    @property
    def batch_size_variance(self) -> float:
        """Variance of the stationary batch size, treating records as independent: ``N·r·(1 − r)``."""
        r = self.stationary_rate
        return self._num_samples * r * (1.0 - r)


class BallsInBinsSampler(_Resumable):
    def __init__(self, data_source: Sized, num_bins: int, n_steps: int | None = None, *, key: RngKey):
        if num_bins < 1:
            raise ValueError("num_bins must be >= 1")
        self.data_source, self.num_bins, self.n_steps = data_source, num_bins, n_steps
        self._num_samples = len(data_source)
        self._key = key
        self._consumed = 0
        self._reset_generator()

    def _reset_generator(self):
        rng = np.random.default_rng(self._key.seed)
        self._bin = rng.integers(0, self.num_bins, size=self._num_samples)

    def _draw(self):
        return np.flatnonzero(self._bin == self._consumed % self.num_bins).tolist()

    @property
    def expected_batch_size(self) -> float:
        return self._num_samples / self.num_bins

    @property
    def sample_rate(self) -> float:
        """Per-step participation rate of a record: ``1 / num_bins``."""
        return 1.0 / self.num_bins

    @property
    def num_epochs(self) -> float | None:
        """Passes over the bins in ``n_steps`` steps (``None`` for an open-ended sampler)."""
        return None if self.n_steps is None else self.n_steps / self.num_bins


class SequentialBatchSampler(_Resumable):
    def __init__(self, data_source: Sized, batch_size: int, n_steps: int | None = None):
        if batch_size < 1:
            raise ValueError("batch_size must be >= 1")
        self.data_source, self.batch_size, self.n_steps = data_source, batch_size, n_steps
        self._num_samples = len(data_source)
        if batch_size > self._num_samples:
            raise ValueError("batch_size exceeds the dataset size")
        self._key = RngKey(0)
        self._consumed = 0

    def _reset_generator(self):
        pass

    @property
    def batches_per_epoch(self) -> int:
        return self._num_samples // self.batch_size

    def _draw(self):
        b = self._consumed % self.batches_per_epoch
        return list(range(b * self.batch_size, (b + 1) * self.batch_size))

    @property
    def expected_batch_size(self) -> float:
        return float(self.batch_size)

    @property
    def min_sep(self) -> int:
        return self.batches_per_epoch


register_serializer(CyclicPoissonSampler,
                    lambda s: {**_save_common(s), "sample_rate": s.sample_rate, "bands": s.bands,
                               "truncated_batch_size": s.truncated_batch_size, "partition_type": s.partition_type.value},
                    lambda t, sd: _load_common(t, sd, ("sample_rate", "bands", "truncated_batch_size")))
register_serializer(BMinSepSampler, lambda s: {**_save_common(s), "bands": s.bands, "sampling_prob": s.sampling_prob},
                    lambda t, sd: _load_common(t, sd, ("bands", "sampling_prob")))
register_serializer(BallsInBinsSampler, lambda s: {**_save_common(s), "num_bins": s.num_bins},
                    lambda t, sd: _load_common(t, sd, ("num_bins",)))
register_serializer(SequentialBatchSampler, lambda s: {**_save_common(s), "batch_size": s.batch_size},
                    lambda t, sd: _load_common(t, sd, ("batch_size",)))

__all__ = ["BMinSepSampler", "BallsInBinsSampler", "CyclicPoissonSampler", "PartitionType", "SequentialBatchSampler",
           "partition_indices"]

from ..utils.namespaces import submodule as _sub  # noqa: E402

_sub(__name__, "types", "Types of the DP-FTRL samplers.", {"PartitionType": PartitionType}, bind=False)
