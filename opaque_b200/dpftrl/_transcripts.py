"""Registry of stored b-min-sep Monte-Carlo transcripts.

A calibration search evaluates the amplified b-min-sep accountant at many noise multipliers (and, for step searches, at
many horizons).  The samples do not depend on the noise multiplier, so they are drawn ONCE per
``(coefficients, min_sep, sampling_prob, warm_start, num_samples, seed)`` and kept in a C++ ``BMinSepCorpus``; every probe
re-weights the same transcripts.  A stored corpus also serves any shorter horizon (a prefix of its columns is exactly
the shorter run's corpus), so the registry keeps, per key, the longest horizon asked for so far.

The registry is bounded: at most ``MAX_ENTRIES`` corpora and ``max_bytes()`` bytes (environment variable
``OPAQUE_B200_B_MIN_SEP_TRANSCRIPT_CACHE_MAX_BYTES``, default 4 GiB).  A corpus that would not fit is not stored and the
caller falls back to the streaming accountant, which draws the same samples without keeping them — the result is the
same either way.

Parity: packages/opaque-dpftrl/src/opaque/api/accounting/dpftrl/amplification/_b_min_sep/_transcript_cache.py and
packages/opaque-accounting/src/amplification/b_min_sep/registry.rs of the reference.
"""
from __future__ import annotations

import os
import threading
from collections import OrderedDict
from typing import Any, Callable, TypeVar

from ..accounting.core import native

T = TypeVar("T")

ENV_MAX_BYTES = "OPAQUE_B200_B_MIN_SEP_TRANSCRIPT_CACHE_MAX_BYTES"
DEFAULT_MAX_BYTES = 4 * 1024 ** 3
MAX_ENTRIES = 4

_lock = threading.RLock()
_entries: "OrderedDict[tuple, Any]" = OrderedDict()      # key (without the horizon) -> BMinSepCorpus
_stats = {"hits": 0, "misses": 0, "evictions": 0, "too_large": 0}


def max_bytes() -> int:
    raw = os.environ.get(ENV_MAX_BYTES)
    if raw is None or raw == "":
        return DEFAULT_MAX_BYTES
    value = int(raw)
    if value < 0:
        raise ValueError(f"{ENV_MAX_BYTES} must be >= 0")
    return value


def estimate_nbytes(n_steps: int, num_samples: int) -> int:
    """One byte for the participation bit and two doubles (P- and Q-branch normals) per (sample, step)."""
    return int(num_samples) * int(n_steps) * 17


def _key(coef, min_sep: int, sampling_prob: float, warm_start: bool, num_samples: int, seed: int) -> tuple:
    return (tuple(float(c) for c in coef), int(min_sep), float(sampling_prob), bool(warm_start), int(num_samples), int(seed))


def _total_bytes() -> int:
    return sum(int(c.nbytes) for c in _entries.values())


def with_corpus(coef, n_steps: int, min_sep: int, sampling_prob: float, warm_start: bool, num_samples: int, seed: int,
                use: Callable[[Any], T]) -> T | None:
    """Run ``use(corpus)`` with a stored corpus that covers ``n_steps`` (creating or extending it first), holding the
    registry lock so that a concurrent ``clear()`` cannot free the corpus in mid-use.  Returns ``None`` without calling
    ``use`` when the corpus would exceed the byte cap."""
    key = _key(coef, min_sep, sampling_prob, warm_start, num_samples, seed)
    with _lock:
        corpus = _entries.get(key)
        if corpus is not None and corpus.n_steps >= n_steps:
            _entries.move_to_end(key)
            _stats["hits"] += 1
            return use(corpus)
        cap = max_bytes()
        need = estimate_nbytes(n_steps, num_samples)
        if need > cap:
            _stats["too_large"] += 1
            return None
        _stats["misses"] += 1
        _entries.pop(key, None)                                    # a shorter corpus of the same key is replaced
        while _entries and (len(_entries) >= MAX_ENTRIES or _total_bytes() + need > cap):
            _entries.popitem(last=False)
            _stats["evictions"] += 1
        corpus = native.BMinSepCorpus(list(key[0]), int(n_steps), int(min_sep), float(sampling_prob), bool(warm_start),
                                      int(num_samples), int(seed))
        _entries[key] = corpus
        return use(corpus)


def clear() -> None:
    with _lock:
        _entries.clear()


def info() -> dict[str, int]:
    with _lock:
        return {"entries": len(_entries), "bytes": _total_bytes(), **_stats}


__all__ = ["DEFAULT_MAX_BYTES", "ENV_MAX_BYTES", "MAX_ENTRIES", "clear", "estimate_nbytes", "info", "max_bytes", "with_corpus"]
