"""Batch samplers whose randomness matches a DP-SGD amplification analysis.

Every sampler is a ``torch.utils.data.Sampler`` yielding *lists of indices*
(use as ``DataLoader(batch_sampler=…)``), is driven by an explicit ``RngKey``
and checkpoints as ``{key_seed, key_impl, consumed, …}``: restoring replays the
host generator ``consumed`` draws forward, so a resumed run sees the batches
the uninterrupted run would have seen.

Parity: packages/opaque-dpsgd/src/opaque/api/dpsgd/sampling/_poisson.py:33-240,
_k_out_of_t.py:16, _random_allocation.py:49, _helpers.py:13-33.
"""
from __future__ import annotations

from collections.abc import Iterator, Sized
from typing import Any

import numpy as np
from torch.utils.data import Sampler

from ..random import RngKey, fold_in
from ..serialization import register_serializer


def poisson_step_indices(rng: np.random.Generator, n: int, rate: float, cap: int | None) -> list[int]:
    """One Poisson draw over ``n`` items; with ``cap`` keep a uniform subset of that size."""
    picked = np.flatnonzero(rng.random(n) < rate)
    if cap is not None and picked.size > cap:
        picked = np.sort(rng.choice(picked, size=cap, replace=False))
    return picked.tolist()


class _Resumable(Sampler):
    """Shared cursor / replay machinery."""

    _consumed: int
    n_steps: int | None

    def _draw(self) -> list[int]:
        raise NotImplementedError

    def _reset_generator(self) -> None:
        raise NotImplementedError

    def __iter__(self) -> Iterator[list[int]]:
        while self.n_steps is None or self._consumed < self.n_steps:
            batch = self._draw()
            self._consumed += 1
            yield batch

    def __len__(self) -> int:
        if self.n_steps is None:
            raise TypeError("len() of unsized object (n_steps=None)")
        return self.n_steps - self._consumed

    @property
    def consumed(self) -> int:
        return self._consumed

    def _replay(self, consumed: int) -> None:
        self._reset_generator()
        self._consumed = 0
        for _ in range(consumed):
            self._draw()
            self._consumed += 1


class PoissonSampler(_Resumable):
    """Each example joins each batch independently with probability ``sample_rate``."""

    def __init__(self, data_source: Sized, sample_rate: float, n_steps: int | None = None,
                 truncated_batch_size: int | None = None, *, key: RngKey):
        if not 0 < sample_rate <= 1:
            raise ValueError(f"sample_rate must be in (0, 1], got {sample_rate}")
        if n_steps is not None and n_steps < 1:
            raise ValueError(f"n_steps must be >= 1 or None, got {n_steps}")
        if truncated_batch_size is not None and truncated_batch_size < 1:
            raise ValueError(f"truncated_batch_size must be >= 1, got {truncated_batch_size}")
        self.data_source = data_source
        self.sample_rate = sample_rate
        self.n_steps = n_steps
        self.truncated_batch_size = truncated_batch_size
        self._num_samples = len(data_source)
        self._key = key
        self._consumed = 0
        self._reset_generator()

    def _reset_generator(self) -> None:
        self.generator = np.random.default_rng(self._key.seed)

    def _draw(self) -> list[int]:
        return poisson_step_indices(self.generator, self._num_samples, self.sample_rate, self.truncated_batch_size)

    @property
    def expected_batch_size(self) -> float:
        return self._num_samples * self.sample_rate

    @property
    def batch_size_variance(self) -> float:
        return self._num_samples * self.sample_rate * (1 - self.sample_rate)


class KOutOfTSampler(_Resumable):
    """Every example takes part in exactly ``k`` of each window of ``t`` consecutive steps.

    At the start of a window each example draws its ``k`` participation slots
    uniformly without replacement; step ``s`` of the window yields the examples
    holding slot ``s``.  Windows use ``fold_in(key, window_index)``.
    """

    def __init__(self, data_source: Sized, k: int | None = None, t: int | None = None, n_steps: int | None = None, *, key: RngKey,
                 total_participations: int | None = None):
        if total_participations is not None:        # the reference's keywords: k of the WHOLE run of n_steps steps
            if k is not None or t is not None or n_steps is None:
                raise ValueError("give (k, t) or (total_participations=, n_steps=)")
            k, t = int(total_participations), int(n_steps)
        if k is None or t is None:
            raise ValueError("give (k, t) or (total_participations=, n_steps=)")
        if not 1 <= k <= t:
            raise ValueError(f"need 1 <= k <= t, got k={k}, t={t}")
        if n_steps is not None and n_steps < 1:
            raise ValueError(f"n_steps must be >= 1 or None, got {n_steps}")
        self.data_source, self.k, self.t, self.n_steps = data_source, k, t, n_steps
        self._num_samples = len(data_source)
        self._key = key
        self._consumed = 0
        self._window = -1
        self._slots: np.ndarray | None = None

    def _reset_generator(self) -> None:
        self._window, self._slots = -1, None

    def _draw(self) -> list[int]:
        w, s = divmod(self._consumed, self.t)
        if w != self._window:
            rng = np.random.default_rng(fold_in(self._key, w).seed)
            ranks = rng.random((self._num_samples, self.t)).argsort(axis=1)
            self._slots = ranks[:, : self.k]
            self._window = w
        return np.flatnonzero((self._slots == s).any(axis=1)).tolist()

    @property
    def expected_batch_size(self) -> float:
        return self._num_samples * self.k / self.t


class RandomAllocationSampler(_Resumable):
    """Balls-into-bins: per epoch each example lands in exactly one of ``num_bins`` steps."""

    def __init__(self, data_source: Sized, num_bins: int, n_steps: int | None = None, *, key: RngKey):
        if num_bins < 1:
            raise ValueError(f"num_bins must be >= 1, got {num_bins}")
        if n_steps is not None and n_steps < 1:
            raise ValueError(f"n_steps must be >= 1 or None, got {n_steps}")
        self.data_source, self.num_bins, self.n_steps = data_source, num_bins, n_steps
        self._num_samples = len(data_source)
        self._key = key
        self._consumed = 0
        self._epoch = -1
        self._assign: np.ndarray | None = None

    def _reset_generator(self) -> None:
        self._epoch, self._assign = -1, None

    def _draw(self) -> list[int]:
        e, b = divmod(self._consumed, self.num_bins)
        if e != self._epoch:
            rng = np.random.default_rng(fold_in(self._key, e).seed)
            self._assign = rng.integers(0, self.num_bins, size=self._num_samples)
            self._epoch = e
        return np.flatnonzero(self._assign == b).tolist()

    @property
    def num_epochs(self) -> float | None:
        """Passes over the bins in ``n_steps`` steps (``None`` for an open-ended sampler)."""
        return None if self.n_steps is None else self.n_steps / self.num_bins

    @property
    def expected_batch_size(self) -> float:
        return self._num_samples / self.num_bins


def _save_common(s: Any) -> dict[str, Any]:
    return {"key_seed": str(s._key.seed), "key_impl": s._key.impl, "consumed": s._consumed,
            "num_samples": s._num_samples, "n_steps": s.n_steps}


def _load_common(template: Any, sd: dict[str, Any], extra: tuple[str, ...]) -> Any:
    if int(sd.get("num_samples", template._num_samples)) != template._num_samples:
        raise ValueError(f"sampler was saved over {sd['num_samples']} examples but the template has {template._num_samples}")
    for name in extra:
        if name in sd and sd[name] != getattr(template, name):
            raise ValueError(f"sampler field {name!r} changed: saved {sd[name]!r}, template {getattr(template, name)!r}")
    template._key = RngKey(int(sd.get("key_seed", template._key.seed)), sd.get("key_impl", template._key.impl))
    if "n_steps" in sd:
        template.n_steps = sd["n_steps"]
    template._replay(int(sd.get("consumed", 0)))
    return template


register_serializer(
    PoissonSampler,
    lambda s: {**_save_common(s), "sample_rate": s.sample_rate, "truncated_batch_size": s.truncated_batch_size},
    lambda t, sd: _load_common(t, sd, ("sample_rate", "truncated_batch_size")))
register_serializer(KOutOfTSampler, lambda s: {**_save_common(s), "k": s.k, "t": s.t},
                    lambda t, sd: _load_common(t, sd, ("k", "t")))
register_serializer(RandomAllocationSampler, lambda s: {**_save_common(s), "num_bins": s.num_bins},
                    lambda t, sd: _load_common(t, sd, ("num_bins",)))


class BalancedRankSampler(Sampler):
    """Deal ONE global sample out evenly over the data-parallel ranks.

    Every rank builds the same ``inner`` sampler (same key, the GLOBAL index range) and keeps positions
    ``rank, rank + world, ...`` of the sorted draw, so per-rank batch sizes differ by at most one example.  The union
    over ranks is exactly the inner sampler's draw, so the privacy analysis is that of the inner sampler on the whole
    dataset — while the step time no longer follows the unluckiest rank (independent per-rank Poisson draws of
    expected size b have a spread of about ±sqrt(b), and every rank waits for the largest).  Each rank must be able
    to read any record.  No counterpart in the reference, which samples per rank
    (packages/opaque-dpsgd/src/opaque/api/dpsgd/sampling).
    """

    def __init__(self, inner: Sampler, rank: int, world: int):
        if not 0 <= rank < world:
            raise ValueError("need 0 <= rank < world")
        self.inner, self.rank, self.world = inner, rank, world

    def __iter__(self) -> Iterator[list[int]]:
        for batch in self.inner:
            yield sorted(batch)[self.rank::self.world]

    def __len__(self) -> int:
        return len(self.inner)

    def __getattr__(self, name: str):            # sample_rate, num_bins, consumed, ... of the global sampler
        if name in ("inner", "rank", "world"):
            raise AttributeError(name)
        return getattr(self.inner, name)



def _load_balanced(template: "BalancedRankSampler", sd: dict[str, Any]) -> "BalancedRankSampler":
    from ..serialization import from_state_dict
    if int(sd.get("world", template.world)) != template.world:
        raise ValueError(f"sampler was saved for {sd['world']} ranks but the job has {template.world}")
    template.inner = from_state_dict(template.inner, sd["inner"])
    return template


def _save_balanced(s: "BalancedRankSampler") -> dict[str, Any]:
    from ..serialization import state_dict
    return {"inner": state_dict(s.inner), "world": s.world}


register_serializer(BalancedRankSampler, _save_balanced, _load_balanced)


__all__ = ["BalancedRankSampler", "KOutOfTSampler", "PoissonSampler", "RandomAllocationSampler", "poisson_step_indices"]
