"""``TrainingArguments``: a standalone dataclass shaped like Hugging Face's, with the DP-specific fields.

Differences from HF semantics: ``per_device_train_batch_size`` is the EXPECTED Poisson batch per device (sample
rate = global batch / dataset size); there is no ``gradient_accumulation_steps`` (microbatching is internal to a
DP step: ``microbatch_size``); ``clipping_norm`` (per example) replaces ``max_grad_norm``; dict-valued fields
accept a mapping, a JSON string or ``"k=v,k2=v2"``; FSDP / DeepSpeed arguments are rejected by ``from_hf``.
``dp_engine`` selects the gradient engine: ``"fused"`` (B200 kernels, ghost clipping, sharded optimizer),
``"reference"`` (vmap per-example gradients + all-reduce) or ``"auto"``.

Parity: packages/opaque-transformers/src/opaque/api/transformers/trainer/_training_arguments.py:143-527,
_convert.py, _hf_convert.py:353-413.
"""
from __future__ import annotations

import dataclasses
import json
import os
from collections.abc import Mapping
from typing import Any

MECHANISMS_DPFTRL = frozenset({"mf_band", "mf_blt", "mf_bisr", "mf_bsr", "mf_lambda_cgd", "mf_identity"})
MECHANISMS = frozenset({"gaussian", *MECHANISMS_DPFTRL})
SAMPLING_MODES = frozenset({"poisson", "random_allocation", "k_out_of_t", "b_min_sep", "balls_in_bins",
                            "cyclic_poisson", "sequential"})
SAMPLER_BY_MECHANISM = {"gaussian": "poisson", "mf_identity": "poisson", "mf_band": "b_min_sep",
                        "mf_blt": "balls_in_bins", "mf_bisr": "balls_in_bins", "mf_bsr": "balls_in_bins",
                        "mf_lambda_cgd": "balls_in_bins"}
ALLOWED_SAMPLERS = {"gaussian": frozenset({"poisson", "random_allocation", "k_out_of_t"}),
                    "mf_identity": frozenset({"poisson", "balls_in_bins"}),
                    "mf_band": frozenset({"b_min_sep", "poisson", "cyclic_poisson", "sequential"}),
                    "mf_blt": frozenset({"balls_in_bins", "sequential"}), "mf_bisr": frozenset({"balls_in_bins", "sequential"}),
                    "mf_bsr": frozenset({"balls_in_bins", "sequential"}), "mf_lambda_cgd": frozenset({"balls_in_bins", "sequential"})}
MECH_DEFAULTS: dict[str, dict[str, Any]] = {"mf_band": {"bands": 16}, "mf_blt": {"max_buffers": 10},
                                            "mf_bisr": {"bandwidth": 4},
                                            "mf_bsr": {"bandwidth": 8, "alpha": 1.0, "beta": 0.9},
                                            "mf_lambda_cgd": {"lambda_": 0.5}, "mf_identity": {}, "gaussian": {}}
CALIBRATION_DEFAULTS = {"min": 0.11, "max": 10.0, "tol": 1e-3}
OPTIMIZER_ALIASES = {"adamw_torch": "adamw", "adamw_torch_fused": "adamw", "adamw_hf": "adamw", "adamw": "adamw",
                     "adamw-bc": "adamw-bc", "adamw_bc": "adamw-bc", "adam": "adam", "sgd": "sgd", "lion": "lion",
                     "lion_32bit": "lion", "adagrad": "adagrad", "rmsprop": "rmsprop", "radam": "radam",
                     "adadelta": "adadelta", "adafactor": "adafactor", "ademamix": "ademamix",
                     "schedule_free_adamw": "schedule_free_adamw", "schedule_free_sgd": "schedule_free_sgd"}


def parse_dict_field(value: Any, name: str) -> dict[str, Any]:
    """Accept a mapping, a JSON object string or ``k=v,k2=v2`` (values parsed as JSON scalars when possible)."""
    if value is None or value == "":
        return {}
    if isinstance(value, Mapping):
        return dict(value)
    if isinstance(value, str):
        text = value.strip()
        if text.startswith("{"):
            out = json.loads(text)
            if not isinstance(out, dict):
                raise ValueError(f"{name}: expected a JSON object")
            return out
        out = {}
        for part in text.split(","):
            if "=" not in part:
                raise ValueError(f"{name}: expected k=v pairs, got {part!r}")
            k, v = part.split("=", 1)
            try:
                out[k.strip()] = json.loads(v.strip())
            except json.JSONDecodeError:
                out[k.strip()] = v.strip()
        return out
    raise TypeError(f"{name}: expected a mapping or a string, got {type(value).__name__}")


@dataclasses.dataclass
class TrainingArguments:
    output_dir: str | None = None
    overwrite_output_dir: bool = False
    per_device_train_batch_size: int = 8
    per_device_eval_batch_size: int | None = None
    eval_accumulation_steps: int | None = None
    eval_delay: float = 0.0
    microbatch_size: int | None = None
    auto_find_microbatch_size: bool = False
    learning_rate: float = 5e-5
    weight_decay: float = 0.0
    adam_beta1: float = 0.9
    adam_beta2: float = 0.999
    adam_epsilon: float = 1e-8
    clipping_norm: Any = 1.0
    optim: str = "adamw"
    optim_args: Any = None
    lr_scheduler: str = "linear"
    lr_scheduler_kwargs: Any = dataclasses.field(default_factory=dict)
    warmup_steps: int = 0
    num_train_epochs: float = 3.0
    max_steps: int = -1
    log_level: str = "passive"
    log_level_replica: str = "warning"
    log_on_each_node: bool = True
    logging_dir: str | None = None
    logging_strategy: str = "steps"
    logging_first_step: bool = False
    logging_steps: int = 500
    save_strategy: str = "steps"
    save_steps: int = 500
    save_total_limit: int | None = None
    save_safetensors: bool = True
    save_on_each_node: bool = False
    save_only_model: bool = False
    restore_callback_states_from_checkpoint: bool = False
    seed: int = 42
    data_seed: int | None = None
    full_determinism: bool = False
    use_cpu: bool = False
    use_mps_device: bool = False
    bf16: bool = False
    bf16_full_eval: bool = False
    tf32: bool | None = None
    local_rank: int = -1
    ddp_backend: str | None = None
    ddp_timeout: int = 1800
    eval_strategy: str = "no"
    eval_steps: int | None = None
    eval_on_start: bool = False
    eval_do_concat_batches: bool = True
    prediction_loss_only: bool = False
    include_for_metrics: list = dataclasses.field(default_factory=list)
    average_tokens_across_devices: bool = True
    metric_for_best_model: str | None = None
    greater_is_better: bool | None = None
    load_best_model_at_end: bool = False
    ignore_data_skip: bool = False
    dataloader_num_workers: int = 0
    dataloader_persistent_workers: bool = False
    dataloader_pin_memory: bool = True
    dataloader_prefetch_factor: int | None = None
    dataloader_multiprocessing_context: str | None = None
    dataloader_in_order: bool = True
    dataloader_drop_last: bool = False
    remove_unused_columns: bool = True
    torch_empty_cache_steps: int | None = None
    label_names: list | None = None
    label_smoothing_factor: float = 0.0
    report_to: Any = None
    disable_tqdm: bool | None = None
    run_name: str | None = None
    project: str | None = None
    trackio_space_id: str | None = None
    trackio_bucket_id: str | None = None
    trackio_static_space_id: str | None = None
    push_to_hub: bool = False
    hub_model_id: str | None = None
    hub_token: str | None = None
    hub_private_repo: bool | None = None
    hub_revision: str | None = None
    torch_compile: bool = False
    torch_compile_backend: str | None = None
    torch_compile_mode: str | None = None
    use_performance_kernels: bool = False
    performance_kernels_config: Any = None
    use_compat_patches: bool = True
    gradient_checkpointing: bool = False
    gradient_checkpointing_kwargs: Any = None
    skip_memory_metrics: bool = True
    include_tokens_per_second: bool = False
    include_sync_metrics: bool = False      # fused engine: log the gradient-barrier / shard-step / parameter-barrier times per step
    include_num_input_tokens_seen: bool = False
    debug: str = ""
    resume_from_checkpoint: str | None = None
    activation_offloading: bool = False
    privacy_target_epsilon: float | None = None
    privacy_target_delta: float | None = None
    clipping_mode: str = "fixed"
    clipping_kwargs: Any = dataclasses.field(default_factory=dict)
    privacy_noise_mechanism: str = "gaussian"
    privacy_noise_multiplier: float | None = None
    privacy_noise_mechanism_kwargs: Any = dataclasses.field(default_factory=dict)
    sampling_mode: str = "auto"
    sampling_kwargs: Any = dataclasses.field(default_factory=dict)
    noise_calibration_kwargs: Any = dataclasses.field(default_factory=dict)
    enable_jit_checkpoint: bool = False
    dp_engine: str = "auto"
    dp_cuda_graph: bool = False          # fused engine: replay each microbatch (forward, backward, clip GEMMs) as one CUDA graph
    _n_gpu: int = dataclasses.field(default=-1, repr=False)

    def __post_init__(self) -> None:
        for name in ("lr_scheduler_kwargs", "clipping_kwargs", "privacy_noise_mechanism_kwargs", "sampling_kwargs",
                     "noise_calibration_kwargs", "optim_args", "performance_kernels_config",
                     "gradient_checkpointing_kwargs"):
            setattr(self, name, parse_dict_field(getattr(self, name), name))
        if isinstance(self.include_for_metrics, str):
            self.include_for_metrics = [x for x in self.include_for_metrics.replace(",", " ").split() if x]
        unknown = sorted(set(self.include_for_metrics or []) - {"inputs", "loss"})
        if unknown:
            raise ValueError(f"include_for_metrics takes 'inputs' and / or 'loss'; got {unknown}")
        if self.eval_accumulation_steps is not None and int(self.eval_accumulation_steps) < 1:
            raise ValueError("eval_accumulation_steps must be a positive number of batches")
        if isinstance(self.clipping_norm, str):
            try:
                self.clipping_norm = float(self.clipping_norm)
            except ValueError:
                self.clipping_norm = parse_dict_field(self.clipping_norm, "clipping_norm")
        if isinstance(self.clipping_norm, Mapping):
            self.clipping_norm = {k: float(v) for k, v in self.clipping_norm.items()}
        elif not float(self.clipping_norm) > 0:
            raise ValueError("clipping_norm must be > 0")
        if self.clipping_mode not in ("fixed", "adaptive", "auto"):
            raise ValueError(f"clipping_mode must be fixed|adaptive|auto, got {self.clipping_mode!r}")
        if self.privacy_noise_mechanism not in MECHANISMS:
            raise ValueError(f"privacy_noise_mechanism must be one of {sorted(MECHANISMS)}")
        if self.sampling_mode == "auto":
            self.sampling_mode = SAMPLER_BY_MECHANISM[self.privacy_noise_mechanism]
        elif self.sampling_mode not in SAMPLING_MODES:
            raise ValueError(f"sampling_mode must be 'auto' or one of {sorted(SAMPLING_MODES)}")
        elif self.sampling_mode not in ALLOWED_SAMPLERS[self.privacy_noise_mechanism]:
            raise ValueError(f"sampling_mode={self.sampling_mode!r} is not valid for {self.privacy_noise_mechanism!r}; "
                             f"allowed: {sorted(ALLOWED_SAMPLERS[self.privacy_noise_mechanism])}")
        self.privacy_noise_mechanism_kwargs = {**MECH_DEFAULTS[self.privacy_noise_mechanism], **self.privacy_noise_mechanism_kwargs}
        self.noise_calibration_kwargs = {**CALIBRATION_DEFAULTS, **self.noise_calibration_kwargs}
        if self.privacy_target_epsilon is not None and self.privacy_noise_multiplier is not None:
            raise ValueError("give either privacy_target_epsilon (calibrated) or privacy_noise_multiplier, not both")
        if self.privacy_target_epsilon is not None and self.privacy_target_epsilon <= 0:
            raise ValueError("privacy_target_epsilon must be > 0")
        if self.optim.lower() not in OPTIMIZER_ALIASES:
            raise ValueError(f"unknown optimizer {self.optim!r}")
        self.optim = OPTIMIZER_ALIASES[self.optim.lower()]
        if self.dp_engine not in ("auto", "fused", "reference"):
            raise ValueError("dp_engine must be auto|fused|reference")
        if self.per_device_train_batch_size < 1:
            raise ValueError("per_device_train_batch_size must be >= 1")
        if self.microbatch_size is not None and self.microbatch_size < 1:
            raise ValueError("microbatch_size must be >= 1")

    # ---- derived -------------------------------------------------------------------------------
    @property
    def world_size(self) -> int:
        return int(os.environ.get("WORLD_SIZE", "1"))

    @property
    def process_index(self) -> int:
        return int(os.environ.get("RANK", "0"))

    @property
    def local_process_index(self) -> int:
        return int(os.environ.get("LOCAL_RANK", "0"))

    @property
    def train_batch_size(self) -> int:
        """Expected GLOBAL batch size."""
        return self.per_device_train_batch_size * self.world_size

    @property
    def eval_batch_size(self) -> int:
        return self.per_device_eval_batch_size or self.per_device_train_batch_size

    @property
    def should_log(self) -> bool:
        return self.process_index == 0

    @property
    def should_save(self) -> bool:
        return self.process_index == 0

    def to_dict(self) -> dict[str, Any]:
        return {f.name: getattr(self, f.name) for f in dataclasses.fields(self) if not f.name.startswith("_")}

    # ---- read-only names that Hugging Face callbacks and integrations look up on an arguments object ----------------
    @property
    def parallel_mode(self) -> str:
        """``"distributed"`` with several processes, else ``"not_distributed"`` (values of Hugging Face's ``ParallelMode``)."""
        return "distributed" if self.world_size > 1 else "not_distributed"

    @property
    def gradient_accumulation_steps(self) -> int:
        """Always 1: one optimizer step per sampled batch (``microbatch_size`` only splits its evaluation)."""
        return 1

    @property
    def lr_scheduler_type(self) -> str:
        return self.lr_scheduler

    @property
    def fp16(self) -> bool:
        """The trainers compute in bf16 or fp32; fp16 with a loss scaler is a functional-API feature."""
        return False

    @property
    def warmup_ratio(self) -> float:
        """The fractional form of ``warmup_steps`` (a value below 1 IS the fraction), else 0."""
        return float(self.warmup_steps) if 0 < self.warmup_steps < 1 else 0.0

    @property
    def device(self) -> "Any":
        import torch
        if self.use_cpu or not torch.cuda.is_available():
            return torch.device("cpu")
        return torch.device("cuda", self.local_process_index)

    @property
    def n_gpu(self) -> int:
        """GPUs driven by THIS process: one (a process per GPU) or none."""
        return 0 if self.device.type == "cpu" else 1

    @classmethod
    def from_hf(cls, hf_args: Any, **overrides: Any) -> "TrainingArguments":
        """Build from a Hugging Face ``TrainingArguments`` (object or mapping); ``overrides`` carry the DP settings.

        The conversion is manifest-driven (:mod:`opaque_b200.transformers.hf_convert`): the effective Hugging Face batch
        (per-device × accumulation) becomes the logical Poisson batch and the per-device size the microbatch,
        ``max_grad_norm`` becomes the per-example clipping norm, optimizer aliases collapse onto ``adamw``, sharded-model /
        quantised-optimizer options are refused, fields without meaning here are dropped with a warning."""
        from .hf_convert import convert_hf_training_arguments
        own = {f.name for f in dataclasses.fields(cls) if not f.name.startswith("_")}
        return cls(**convert_hf_training_arguments(hf_args, own, **overrides))


__all__ = ["ALLOWED_SAMPLERS", "MECHANISMS", "MECH_DEFAULTS", "SAMPLER_BY_MECHANISM", "SAMPLING_MODES",
           "TrainingArguments", "parse_dict_field"]
