"""Immutable JAX-style RNG keys plus the Philox counter derivation used on device.

Key algebra (bit-compatible with the reference so checkpoints and seeds carry
over): ``key(seed)`` keeps the low 64 bits; ``fold_in(k, d)`` hashes
``(k.seed, d)`` with BLAKE2b-64 — integers as 16-byte little-endian signed,
anything else as UTF-8, each part followed by ``|`` — and reads the digest as a
little-endian unsigned 64-bit seed; ``split(k, n)[i] = fold_in(k, i)``.

Device noise does not consume a stateful generator: the 64-bit seed of the
per-step key is the Philox-4x32 key and the counter is the coordinate's global
flat index, so any sharding of the coordinates yields the same realisation.

Parity: packages/opaque-engine/src/opaque/api/engine/random/_engine.py:23-101,
_helpers.py.
"""
from __future__ import annotations

import dataclasses
import hashlib
import os
import random as _pyrandom

import numpy as np
import torch

_U64 = (1 << 64) - 1
_TORCH_SEED_MOD = (1 << 63) - 1
DEFAULT_IMPL = "opaque_threefry_like"


@dataclasses.dataclass(frozen=True)
class RngKey:
    """Key material: a 64-bit seed and the name of the derivation scheme."""

    seed: int
    impl: str = DEFAULT_IMPL


def key(seed: int) -> RngKey:
    """A root ``RngKey`` from an integer seed."""
    if isinstance(seed, bool) or not isinstance(seed, int):
        raise TypeError(f"seed must be int, got {type(seed)}")
    return RngKey(seed & _U64)


def _mix(seed: int, item: int | str) -> int:
    digest = hashlib.blake2b(digest_size=8)
    for part in (seed, item):
        if isinstance(part, int):
            digest.update(part.to_bytes(16, "little", signed=True))
        else:
            digest.update(str(part).encode("utf-8"))
        digest.update(b"|")
    return int.from_bytes(digest.digest(), "little", signed=False)


def fold_in(rng_key: RngKey, *data: int | str) -> RngKey:
    """Derive a child key; several items fold left to right."""
    if not data:
        raise ValueError("fold_in requires at least one data argument")
    seed = rng_key.seed
    for item in data:
        if not isinstance(item, (int, str)):
            raise TypeError(f"data must be int or str, got {type(item)}")
        seed = _mix(seed, item)
    return RngKey(seed, rng_key.impl)


def split(rng_key: RngKey, num: int = 2) -> tuple[RngKey, ...]:
    """``num`` independent child keys of ``key``."""
    if num < 1:
        raise ValueError(f"num must be >= 1, got {num}")
    return tuple(fold_in(rng_key, i) for i in range(num))


def generator_from_key(rng_key: RngKey, device: str | torch.device = "cpu") -> torch.Generator:
    """A ``torch.Generator`` seeded with ``seed mod (2**63 - 1)`` (CPU by default)."""
    return torch.Generator(device=device).manual_seed(rng_key.seed % _TORCH_SEED_MOD)


def philox_key(rng_key: RngKey) -> tuple[int, int]:
    """The two 32-bit Philox key words ``(lo, hi)`` of a key's seed."""
    return rng_key.seed & 0xFFFFFFFF, (rng_key.seed >> 32) & 0xFFFFFFFF


def random_key() -> RngKey:
    """A key from OS entropy (non-reproducible runs)."""
    return key(int.from_bytes(os.urandom(8), "little"))


def set_reproducible_pytorch_seed(key_val: "RngKey | int", *, deterministic: bool = True) -> RngKey:
    """Seed the python, numpy and torch (CPU and every CUDA device) global generators from one key (or integer seed) and
    return the key.  With ``deterministic`` also asks cuDNN for deterministic algorithms and sets the cuBLAS workspace
    variable that deterministic GEMMs need.  Global state: call once at the start of a script.

    Parity: packages/opaque-engine/src/opaque/api/engine/random/_helpers.py:39."""
    k = key_val if isinstance(key_val, RngKey) else key(int(key_val))
    seed = int(k.seed)
    _pyrandom.seed(seed)
    np.random.seed(seed % (1 << 32))
    torch.manual_seed(seed % _TORCH_SEED_MOD)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed % _TORCH_SEED_MOD)
    if deterministic:
        import os
        torch.backends.cudnn.deterministic = True
        torch.backends.cudnn.benchmark = False
        os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":4096:8")
    return k


from ..serialization import register_serializer as _reg  # noqa: E402

_reg(RngKey, lambda k: {"seed": str(k.seed), "impl": k.impl},
     lambda t, sd: RngKey(int(sd.get("seed", t.seed)), sd.get("impl", t.impl)))

__all__ = ["RngKey", "fold_in", "generator_from_key", "key", "philox_key", "random_key",
           "set_reproducible_pytorch_seed", "split"]

from ..utils.namespaces import submodule as _sub  # noqa: E402

_sub(__name__, "types", "Classes of the random façade.", {"RngKey": RngKey}, bind=False)
