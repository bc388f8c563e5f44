"""Hugging Face ``transformers.TrainingArguments`` → :class:`TrainingArguments`.

Every field of the Hugging Face dataclass falls into exactly one bucket:

* **direct** — same name and meaning here; copied.
* **renamed** — same meaning, other name (``lr_scheduler_type`` → ``lr_scheduler``).
* **derived** — several fields combine into one setting.  The important one: Hugging Face's effective batch
  (``per_device_train_batch_size × gradient_accumulation_steps``) is the privacy-relevant batch, so it becomes the
  LOGICAL Poisson batch here and the per-device size becomes the microbatch — dropping the accumulation factor would
  understate the sampling rate and report a too small ε.
* **refused** — set to a non-default value it has no safe meaning under per-example clipping (model sharding, paged /
  quantised optimizers, embedding-noise tricks): ``ValueError`` with the reason and what to use instead.
* **ignored** — irrelevant to this trainer (process plumbing, evaluation gather flags); dropped with a
  ``RuntimeWarning`` when set away from its default, so nothing is swallowed silently.

``tests/test_trainers.py`` checks that the installed ``transformers`` version's fields are all classified.

Parity: packages/opaque-transformers/src/opaque/api/transformers/trainer/_hf_convert.py (manifest, batch / optimizer /
warm-up collapse, max_grad_norm and Liger mappings) and _convert.py (the shared manifest engine).
"""
from __future__ import annotations

import dataclasses
import warnings
from collections.abc import Mapping
from typing import Any, Callable

RENAMED: dict[str, str] = {"lr_scheduler_type": "lr_scheduler"}

PAGED_OR_QUANTISED_OPTIMS = frozenset({
    "adamw_apex_fused", "adamw_bnb_8bit", "adamw_8bit", "paged_adamw_8bit", "paged_adamw_32bit", "lion_8bit",
    "paged_lion_8bit", "paged_lion_32bit", "rmsprop_bnb", "rmsprop_bnb_8bit", "rmsprop_bnb_32bit", "adamw_torch_xla",
    "adamw_torch_npu_fused", "adamw_anyprecision"})

# field -> reason; refused when the value differs from the Hugging Face default / is truthy
REFUSED: dict[str, str] = {
    "fsdp": "parameters are replicated and the DP state (noise, optimizer) is sharded ZeRO-1 style; model sharding is not supported",
    "fsdp_config": "see fsdp",
    "deepspeed": "see fsdp: the sharded DP optimizer replaces ZeRO stages",
    "parallelism_config": "tensor / pipeline parallel layouts are not supported; data parallelism only",
    "neftune_noise_alpha": "NEFTune adds data-dependent noise to embeddings outside the privacy analysis",
    "optim_target_modules": "layer-wise optimizers (GaLore, APOLLO) are not supported under per-example clipping",
    "fp16": "use bf16: fp16 loss scaling interacts with the clipping threshold",
    "fp16_full_eval": "use bf16_full_eval",
    "train_sampling_strategy": "batches are drawn by the DP sampler (sampling_mode); length grouping would break the sampling analysis",
}

# combined into other settings by the transforms below
DERIVED = frozenset({"per_device_train_batch_size", "gradient_accumulation_steps", "auto_find_batch_size", "optim",
                     "warmup_steps", "warmup_ratio", "max_grad_norm", "use_liger_kernel", "liger_kernel_config"})

IGNORED = frozenset({
    "use_cache", "logging_nan_inf_filter", "eval_use_gather_object", "batch_eval_metrics", "hub_strategy", "hub_always_push",
    "accelerator_config", "length_column_name", "ddp_find_unused_parameters", "ddp_bucket_cap_mb", "ddp_broadcast_buffers",
    "do_train", "do_eval", "do_predict"})


def _as_dict(hf_args: Any) -> dict[str, Any]:
    if isinstance(hf_args, Mapping):
        return dict(hf_args)
    if dataclasses.is_dataclass(hf_args):
        return {f.name: getattr(hf_args, f.name) for f in dataclasses.fields(hf_args)}
    return {k: v for k, v in vars(hf_args).items() if not k.startswith("_")}


def _hf_defaults() -> dict[str, Any]:
    """Defaults of the installed ``transformers.TrainingArguments`` (empty when the package is absent)."""
    try:
        import transformers
    except Exception:      # noqa: BLE001
        return {}
    out = {}
    for f in dataclasses.fields(transformers.TrainingArguments):
        if f.default is not dataclasses.MISSING:
            out[f.name] = f.default
        elif f.default_factory is not dataclasses.MISSING:      # type: ignore[misc]
            try:
                out[f.name] = f.default_factory()               # type: ignore[misc]
            except Exception:      # noqa: BLE001
                pass
    return out


def _is_set(name: str, value: Any, defaults: Mapping[str, Any]) -> bool:
    """True when ``value`` says something: differs from the Hugging Face default and is not an empty container / None."""
    if value is None or value == "" or value == [] or value == {} or value is False:
        return False
    if name in defaults:
        d = defaults[name]
        if value == d or str(getattr(value, "value", value)) == str(getattr(d, "value", d)):
            return False
    return True


def classify(name: str, own_fields: set[str]) -> str:
    """Bucket of one Hugging Face field: ``derived`` / ``renamed`` / ``refused`` / ``ignored`` / ``direct`` / ``unknown``."""
    if name in DERIVED:
        return "derived"
    if name in RENAMED:
        return "renamed"
    if name in REFUSED:
        return "refused"
    if name in IGNORED:
        return "ignored"
    if name in own_fields:
        return "direct"
    return "unknown"


# ---- derived settings ------------------------------------------------------------------------------------------------

def _batch(hf: Mapping[str, Any]) -> dict[str, Any]:
    per_device = int(hf.get("per_device_train_batch_size") or 8)
    accum = int(hf.get("gradient_accumulation_steps") or 1)
    out: dict[str, Any] = {"per_device_train_batch_size": per_device * accum,
                           "auto_find_microbatch_size": bool(hf.get("auto_find_batch_size", False))}
    if accum > 1:
        out["microbatch_size"] = per_device
    return out


def _optim(hf: Mapping[str, Any]) -> dict[str, Any]:
    raw = hf.get("optim")
    if raw is None:
        return {}
    name = str(getattr(raw, "value", raw)).lower()
    if name in PAGED_OR_QUANTISED_OPTIMS:
        raise ValueError(f"optim={name!r}: paged / quantised / vendor-fused optimizers have no counterpart; use optim='adamw' "
                         "(or 'adamw-bc' for the noise-aware second moment)")
    if name in ("adamw_torch", "adamw_hf", "adamw_torch_fused", "adamw_torch_4bit"):
        return {"optim": "adamw"}
    return {"optim": name}


def _warmup(hf: Mapping[str, Any]) -> dict[str, Any]:
    steps = hf.get("warmup_steps") or 0
    return {"warmup_steps": steps if steps else (hf.get("warmup_ratio") or 0)}      # a value below 1 is a fraction of the run


def _clip(hf: Mapping[str, Any]) -> dict[str, Any]:
    v = hf.get("max_grad_norm")
    return {"clipping_norm": float(v)} if v else {}         # closest knob: the global clip becomes the per-example bound


def _kernels(hf: Mapping[str, Any]) -> dict[str, Any]:
    return {"use_performance_kernels": True} if hf.get("use_liger_kernel") else {}


TRANSFORMS: tuple[Callable[[Mapping[str, Any]], dict[str, Any]], ...] = (_batch, _optim, _warmup, _clip, _kernels)


def convert_hf_training_arguments(hf_args: Any, own_fields: set[str], **overrides: Any) -> dict[str, Any]:
    """Keyword arguments for :class:`TrainingArguments` from a Hugging Face arguments object / mapping.

    ``overrides`` (DP settings: ``privacy_noise_multiplier``, ``clipping_norm``, ``sampling_mode`` …) win over everything
    derived from ``hf_args``.
    """
    hf = _as_dict(hf_args)
    defaults = _hf_defaults()
    out: dict[str, Any] = {}
    for name, value in hf.items():
        bucket = classify(name, own_fields)
        if bucket == "refused":
            if _is_set(name, value, defaults):
                raise ValueError(f"{name}={value!r} is not supported: {REFUSED[name]}")
        elif bucket == "ignored":
            if _is_set(name, value, defaults):
                warnings.warn(f"TrainingArguments.from_hf: {name}={value!r} has no effect in this trainer and is dropped",
                              RuntimeWarning, stacklevel=3)
        elif bucket == "renamed":
            if value is not None:
                out[RENAMED[name]] = str(getattr(value, "value", value))
        elif bucket == "direct":
            if value is not None:
                out[name] = getattr(value, "value", value) if not isinstance(value, (dict, list, tuple)) else value
        elif bucket == "unknown" and _is_set(name, value, defaults):
            warnings.warn(f"TrainingArguments.from_hf: unknown field {name}={value!r} is dropped", RuntimeWarning, stacklevel=3)
    for fn in TRANSFORMS:
        out.update(fn(hf))
    out.update(overrides)
    return {k: v for k, v in out.items() if k in own_fields}


__all__ = ["DERIVED", "IGNORED", "REFUSED", "RENAMED", "classify", "convert_hf_training_arguments"]
