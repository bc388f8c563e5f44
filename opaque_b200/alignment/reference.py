"""Reference-policy helpers for preference optimisation: which parameters play the reference, and scoring a dataset once.

* :func:`with_disabled_adapter` / :func:`null_ref_context` — run the reference forward through the POLICY object: a LoRA
  model with its adapters switched off is the base model.  Works for this package's models (``add_lora``), for models
  wrapped by the PEFT library (``disable_adapter()`` / a frozen ``"ref"`` adapter clone), and is a no-op otherwise.
* :func:`ema_update_reference` — the TR-DPO update ``ref ← (1 − α)·ref + α·policy`` on parameter pytrees.
* :func:`compute_ref_logprobs_for_dataset` — one pass of a reference callable over a dataset: rank-sharded, gathered back
  in dataset order, cached on disk under a fingerprint of the data and of the reference's identity.  The cache holds
  per-example values of private data, so its directory and files are readable by the owner only.

All of these change module state or touch the file system: call them outside ``vmap`` / ``torch.func`` transforms.

Parity: packages/opaque-alignment/src/opaque/api/alignment/dpo/reference/{_adapter,_sync,_precompute}.py.
"""
from __future__ import annotations

import contextlib
import hashlib
import json
import os
import tempfile
from collections.abc import Callable, Mapping, Sequence
from typing import Any

import torch

from ..distributed import gather_tensors, get_rank, get_world_size, is_distributed
from ..pytree import tree_map


def _is_peft_model(model: Any) -> bool:
    return isinstance(getattr(model, "peft_config", None), dict) and hasattr(model, "disable_adapter")


def _has_own_lora(model: Any) -> bool:
    return isinstance(model, torch.nn.Module) and any(getattr(m, "lora_A", None) is not None and isinstance(m.lora_A, torch.nn.Parameter)
                                                      for m in model.modules())


@contextlib.contextmanager
def with_disabled_adapter(model: Any):
    """Inside the block ``model`` computes with its adapters off (the base model); restored on exit.  No-op for a model
    without adapters."""
    if _is_peft_model(model):
        with model.disable_adapter():
            yield
    elif _has_own_lora(model):
        from ..models.layers import adapters_disabled
        with adapters_disabled():
            yield
    else:
        yield


@contextlib.contextmanager
def null_ref_context(model: Any, ref_model: Any | None = None):
    """Turn ``model`` into its own reference inside the block.

    ``ref_model`` given → nothing to do (the caller uses it).  A PEFT model with an adapter named ``"ref"`` (a frozen
    clone of the initial adapter) → that adapter is selected and the previous selection restored.  Any other model with
    adapters → adapters off.  No adapters → no-op (the caller supplies frozen parameters itself).
    """
    if ref_model is not None:
        yield
        return
    if _is_peft_model(model) and "ref" in model.peft_config and hasattr(model, "set_adapter"):
        previous = getattr(model, "active_adapters", None) or getattr(model, "active_adapter", None)
        model.set_adapter("ref")
        try:
            yield
        finally:
            if previous is not None:
                model.set_adapter(previous if isinstance(previous, str) or len(previous) != 1 else previous[0])
        return
    with with_disabled_adapter(model):
        yield


def ema_update_reference(ref_params: Any, policy_params: Any, alpha: float) -> Any:
    """``(1 − alpha)·ref + alpha·policy`` leaf by leaf (new tensors; the inputs are not modified).  ``alpha = 0`` keeps the
    reference, ``alpha = 1`` copies the policy."""
    if not 0.0 <= alpha <= 1.0:
        raise ValueError(f"alpha must be in [0, 1], got {alpha}")
    return tree_map(lambda r, p: torch.lerp(r.detach(), p.detach().to(r.dtype), float(alpha)), ref_params, policy_params)


# ---------------------------------------------------------------------------------------------------- precompute

def _canonical(value: Any, path: str = "cache_identity") -> Any:
    """JSON-able form with sorted mappings; anything that has no stable text form is refused."""
    if value is None or isinstance(value, (bool, int, float, str)):
        return value
    if isinstance(value, Mapping):
        return {str(k): _canonical(v, f"{path}.{k}") for k, v in sorted(value.items(), key=lambda kv: str(kv[0]))}
    if isinstance(value, (list, tuple)):
        return [_canonical(v, f"{path}[{i}]") for i, v in enumerate(value)]
    raise TypeError(f"{path}: values of type {type(value).__name__} cannot identify a cache entry")


def _dataset_fingerprint(dataset: Any) -> str:
    fp = getattr(dataset, "_fingerprint", None)
    if isinstance(fp, str):
        return fp
    h = hashlib.sha256()
    h.update(str(len(dataset)).encode())
    for i in range(len(dataset)):
        row = dataset[i]
        h.update(json.dumps(_canonical({k: (v.tolist() if isinstance(v, torch.Tensor) else v) for k, v in row.items()}, "row"),
                            sort_keys=True).encode())
    return h.hexdigest()[:32]


def _cache_file(cache_dir: str | None, dataset: Any, identity: Any, columns: Sequence[str]) -> str:
    base = cache_dir or os.path.join(tempfile.gettempdir(), "opaque_b200_ref_cache")
    key = json.dumps({"data": _dataset_fingerprint(dataset), "identity": _canonical(identity), "columns": list(columns)}, sort_keys=True)
    return os.path.join(base, hashlib.sha256(key.encode()).hexdigest()[:40] + ".safetensors")


def _add_columns(dataset: Any, columns: Mapping[str, torch.Tensor]) -> Any:
    if hasattr(dataset, "add_column"):                      # datasets.Dataset
        for name, values in columns.items():
            if name in getattr(dataset, "column_names", ()):
                dataset = dataset.remove_columns(name)
            dataset = dataset.add_column(name, values.tolist())
        return dataset
    return [{**dict(dataset[i]), **{name: float(values[i]) for name, values in columns.items()}} for i in range(len(dataset))]


def compute_ref_logprobs_for_dataset(dataset: Any, ref: Callable[[dict], Mapping[str, torch.Tensor]],
                                     collator: Callable[[list], dict], output_columns: Sequence[str], *, cache_identity: Any,
                                     batch_size: int = 8, cache_dir: str | None = None, use_cache: bool = True,
                                     shard: bool | None = None) -> Any:
    """Score every row with ``ref(collator(rows)) -> {column: [B] tensor}`` (under ``no_grad``) and return the dataset with
    ``output_columns`` added (a ``datasets.Dataset`` through ``add_column``; a list of dict rows otherwise).

    With a live process group each rank scores its own contiguous slice and the results are gathered back in dataset
    order (``shard=None`` / ``True``; ``False``: every rank scores everything).  With ``use_cache`` the columns are stored
    in ``cache_dir`` (default: ``<tmp>/opaque_b200_ref_cache``) as a ``.safetensors`` file named after a hash of the
    dataset fingerprint, ``cache_identity`` (JSON-like; what the reference IS) and the column names; directory and file
    are owner-only.  All ranks must pass the same arguments.
    """
    columns = list(output_columns)
    if not columns:
        raise ValueError("output_columns is empty")
    live = is_distributed()
    if shard is True and not live:
        raise RuntimeError("shard=True needs an initialised process group")
    sharded = live if shard is None else bool(shard)
    path = _cache_file(cache_dir, dataset, cache_identity, columns) if use_cache else None
    n = len(dataset)
    cached = None
    if path is not None and os.path.exists(path):
        from safetensors.torch import load_file
        loaded = load_file(path)
        if all(c in loaded and loaded[c].shape == (n,) for c in columns):
            cached = {c: loaded[c] for c in columns}
    if live:                                               # a rank with a stale or missing file makes everybody recompute
        from ..distributed import reduce_scalar
        if not bool(reduce_scalar(int(cached is not None), "min")):
            cached = None
    if cached is None:
        rank, world = (get_rank(), get_world_size()) if sharded else (0, 1)
        per = n // world
        lo, hi = rank * per, (n if rank == world - 1 else (rank + 1) * per)
        parts: dict[str, list[torch.Tensor]] = {c: [] for c in columns}
        with torch.no_grad():
            for start in range(lo, hi, batch_size):
                out = ref(collator([dataset[i] for i in range(start, min(hi, start + batch_size))]))
                for c in columns:
                    parts[c].append(out[c].detach().float().reshape(-1).cpu())
        local = {c: (torch.cat(v) if v else torch.zeros(0)) for c, v in parts.items()}
        cached = {c: (gather_tensors(v).cpu() if sharded and live else v) for c, v in local.items()}
        for c in columns:
            if cached[c].shape != (n,):
                raise RuntimeError(f"reference column {c!r}: expected {n} values, got {tuple(cached[c].shape)}")
        if path is not None and (not live or get_rank() == 0):
            from safetensors.torch import save_file
            os.makedirs(os.path.dirname(path), mode=0o700, exist_ok=True)
            os.chmod(os.path.dirname(path), 0o700)
            tmp = path + f".{os.getpid()}.tmp"
            save_file({c: v.contiguous() for c, v in cached.items()}, tmp)
            os.chmod(tmp, 0o600)
            os.replace(tmp, path)
    return _add_columns(dataset, cached)


__all__ = ["compute_ref_logprobs_for_dataset", "ema_update_reference", "null_ref_context", "with_disabled_adapter"]
