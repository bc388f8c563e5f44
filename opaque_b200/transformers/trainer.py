"""``DPTrainer``: a Hugging-Face-shaped training loop over the DP primitives.

One step = sample (Poisson / DP-FTRL sampler) → per-example clipped gradients → cross-rank reduction → noise →
optimizer, with the accountant charged once per step.  Two gradient engines share the loop:

  ``fused``      (B200) :class:`opaque_b200.engine.fused.FusedDPEngine` — ghost clipping, clip-weighted tcgen05
                 weight-gradient GEMMs that reduce-scatter into sharded state, Philox / correlated noise fused
                 with AdamW-BC.  The model must expose ``per_example_loss(**batch) -> [B]``.
  ``reference``  the functional pipeline ``clipped_grad`` (vmap) → ``sum_gradients_`` → ``gaussian_noise`` /
                 ``mf_gaussian_noise`` → functional optimizer; runs anywhere (CPU / gloo included) and is the
                 numerical baseline of the fused engine.

Checkpoints are atomic directories ``checkpoint-N`` (written as ``checkpoint-N.tmp`` then renamed) holding
``model.safetensors`` (or adapter weights), ``dp_optimizer.pt``, ``dp_state.pt`` (runtime bundle, version 3:
clip / noise / sampler state, DP hyper-parameters for drift detection), ``accountant.json``,
``trainer_state.json`` and ``rng_state.pth`` (``rng_state_{rank}.pth`` with several ranks); resuming uses the saved accountant as a prefix so
calibration and stop-at-ε account for budget already spent.

A retryable OOM on any rank is turned into a cluster-wide decision (one MAX all-reduce of a flag): every rank
halves its microbatch and replays the step, so nobody is left waiting in a collective.

Parity: packages/opaque-transformers/src/opaque/api/transformers/trainer/{_dp_trainer,_checkpoint,_distributed,
_dpftrl,_optim,_scheduler,_eval,_callback,_state}.py.
"""
from __future__ import annotations

import dataclasses
import json
import math
import os
import pickle
import random
import re
import shutil
import time
from collections.abc import Callable, Mapping, Sequence
from typing import Any

import numpy as np
import torch
import torch.distributed as dist

from .. import accounting as acc
from .. import optimizers as optim_lib
from .. import scheduling as sched
from ..distributed import (gather_tensors, get_rank, get_world_size, is_distributed, local_shard, reduce_scalar, sum_gradients_,
                           sync)
from ..dpftrl import accounting as ftrl_acc
from ..dpftrl import noise as ftrl_noise
from ..dpftrl.sampling import BallsInBinsSampler, BMinSepSampler, CyclicPoissonSampler, SequentialBatchSampler
from ..dpsgd import accounting as sgd_acc
from ..dpsgd.clipping import adaptive_clipped_grad, auto_clipped_grad, clipped_grad, per_group
from ..dpsgd.noise import gaussian_noise
from ..dpsgd.sampling import KOutOfTSampler, PoissonSampler, RandomAllocationSampler
from ..functional import make_functional
from ..profiling import perf_tracker
from ..random import RngKey, fold_in, key
from ..serialization import from_state_dict, state_dict
from .evaluation import (EvalPrediction, EvaluationResult, PredictionAccumulator, PredictionOutput, TrainOutput, speed_metrics, to_python,
                         with_metric_prefix)
from .training_args import MECHANISMS_DPFTRL, TrainingArguments

DP_STATE_BUNDLE_VERSION = 3
CHECKPOINT_RE = re.compile(r"^checkpoint-(\d+)$")
FILES = {"optimizer": "dp_optimizer.pt", "state": "dp_state.pt", "accountant": "accountant.json",
         "trainer_state": "trainer_state.json", "args": "training_args.bin", "weights": "model.safetensors"}


# ------------------------------------------------------------------------------------------ small pieces

@dataclasses.dataclass
class DPTrainerState:
    global_step: int = 0
    epoch: float = 0.0
    max_steps: int = 0
    num_input_tokens_seen: int = 0
    log_history: list = dataclasses.field(default_factory=list)
    best_metric: float | None = None
    best_model_checkpoint: str | None = None
    epsilon: float | None = None

    def to_json(self) -> str:
        return json.dumps(dataclasses.asdict(self), indent=1)


class TrainerCallback:
    """Override any hook; every hook receives ``(args, state, control, **kwargs)``."""

    def on_train_begin(self, args, state, control, **kw): ...
    def on_step_begin(self, args, state, control, **kw): ...
    def on_pre_optimizer_step(self, args, state, control, **kw): ...
    def on_optimizer_step(self, args, state, control, **kw): ...
    def on_step_end(self, args, state, control, **kw): ...
    def on_log(self, args, state, control, logs=None, **kw): ...
    def on_evaluate(self, args, state, control, metrics=None, **kw): ...
    def on_save(self, args, state, control, **kw): ...
    def on_train_end(self, args, state, control, **kw): ...


@dataclasses.dataclass
class TrainerControl:
    should_training_stop: bool = False
    should_save: bool = False
    should_evaluate: bool = False
    should_log: bool = False


class PrinterCallback(TrainerCallback):
    def on_log(self, args, state, control, logs=None, **kw):
        if args.should_log and logs:
            print({k: (round(v, 5) if isinstance(v, float) else v) for k, v in logs.items()}, flush=True)


class JsonlLoggerCallback(TrainerCallback):
    """``report_to="jsonl"``: append every log record to ``output_dir/metrics.jsonl`` (rank 0 only)."""

    def on_log(self, args, state, control, logs=None, **kw):
        if args.should_log and logs and args.output_dir:
            os.makedirs(args.output_dir, exist_ok=True)
            with open(os.path.join(args.output_dir, "metrics.jsonl"), "a") as f:
                f.write(json.dumps({"step": state.global_step, **{k: v for k, v in logs.items() if isinstance(v, (int, float, str))}}) + "\n")


class TensorBoardCallback(TrainerCallback):
    """``report_to="tensorboard"``: scalars under ``logging_dir`` (or ``output_dir/runs``); privacy metrics keep their names."""

    def __init__(self):
        self.writer = None

    def on_train_begin(self, args, state, control, **kw):
        if not args.should_log:
            return
        from torch.utils.tensorboard import SummaryWriter
        self.writer = SummaryWriter(log_dir=getattr(args, "logging_dir", None) or os.path.join(args.output_dir or ".", "runs"))

    def on_log(self, args, state, control, logs=None, **kw):
        if self.writer is not None and logs:
            for k, v in logs.items():
                if isinstance(v, (int, float)):
                    self.writer.add_scalar(k if "/" in k else f"train/{k}", v, state.global_step)

    def on_train_end(self, args, state, control, **kw):
        if self.writer is not None:
            self.writer.close()
            self.writer = None


class WandbCallback(TrainerCallback):
    """``report_to="wandb"``: forwards log records to an existing or new W&B run (offline mode works without a network)."""

    def __init__(self):
        self.run = None

    def on_train_begin(self, args, state, control, **kw):
        if not args.should_log:
            return
        import wandb
        self.run = wandb.run or wandb.init(project=os.environ.get("WANDB_PROJECT", "opaque_b200"), name=getattr(args, "run_name", None),
                                          config={k: v for k, v in dataclasses.asdict(args).items() if isinstance(v, (int, float, str, bool))})

    def on_log(self, args, state, control, logs=None, **kw):
        if self.run is not None and logs:
            self.run.log({k: v for k, v in logs.items() if isinstance(v, (int, float))}, step=state.global_step)


REPORTERS = {"jsonl": JsonlLoggerCallback, "tensorboard": TensorBoardCallback, "wandb": WandbCallback}


def reporting_callbacks(report_to: Any) -> list[TrainerCallback]:
    """Callbacks for ``report_to`` (a name, a list of names, ``"none"`` / ``None``, or ``"all"`` = every importable one)."""
    if report_to in (None, "none", [], ()):
        return []
    names = [report_to] if isinstance(report_to, str) else list(report_to)
    if names == ["all"]:
        names = ["jsonl"]
        for mod, name in (("torch.utils.tensorboard", "tensorboard"), ("wandb", "wandb")):
            try:
                __import__(mod)
                names.append(name)
            except Exception:      # noqa: BLE001 — an optional integration that is not installed is skipped
                pass
    out = []
    for n in names:
        if n not in REPORTERS:
            raise ValueError(f"report_to={n!r} is not supported; choose from {sorted(REPORTERS)}")
        out.append(REPORTERS[n]())
    return out


class BestModelSaveCallback(TrainerCallback):
    """Track ``metric_for_best_model`` on every evaluation and remember the best checkpoint."""

    def on_evaluate(self, args, state, control, metrics=None, **kw):
        name = args.metric_for_best_model
        if not name or not metrics:
            return
        keyname = name if name in metrics else f"eval_{name}"
        if keyname not in metrics:
            return
        better = (lambda a, b: a > b) if args.greater_is_better else (lambda a, b: a < b)
        if state.best_metric is None or better(metrics[keyname], state.best_metric):
            state.best_metric = float(metrics[keyname])
            control.should_save = True
            if args.output_dir:            # the training loop writes this checkpoint right after the evaluation
                state.best_model_checkpoint = os.path.join(args.output_dir, f"checkpoint-{state.global_step}")


@dataclasses.dataclass
class RuntimeCheckpoint:
    """Everything besides weights / optimizer needed to continue a DP run bit-for-bit (``dp_state.pt``).

    The first block carries the field names of the reference's bundle
    (packages/opaque-transformers/src/opaque/api/transformers/trainer/_checkpoint.py:198-290); ``extras`` holds what
    this trainer checks in addition (sampling mode, clipping settings, mechanism arguments, engine).  The file is a
    ``torch.save`` of a plain dict with these keys, never a pickled class instance, so reading it needs neither
    this package nor the reference: ``torch.load(path)["noise_multiplier"]``.  A bundle written by the reference (a
    pickled instance of ITS dataclass) loads through :func:`load_runtime_checkpoint`, which resolves that class name to
    this one.
    """
    version: int
    clip_state: dict
    noise_state: dict
    sampler_state: dict | None
    sample_rate: float
    target_delta: float
    noise_multiplier: float
    expected_steps_per_epoch: int
    expected_batch_size: float
    total_steps: int
    mechanism_kind: str = "gaussian"
    mf_n_steps: int | None = None
    mf_min_sep: int | None = None
    mf_max_participations: int | None = None
    lr_scheduler: str | None = None
    learning_rate: float | None = None
    warmup_steps: float | None = None
    lr_scheduler_kwargs: dict | None = None
    extras: dict = dataclasses.field(default_factory=dict)

    # names used elsewhere in this trainer
    @property
    def max_steps(self) -> int:
        return self.total_steps

    @property
    def mechanism(self) -> str:
        return self.mechanism_kind

    def to_dict(self) -> dict:
        return {"format": "opaque dp_state bundle", **{f.name: getattr(self, f.name) for f in dataclasses.fields(self)}}

    @classmethod
    def from_dict(cls, d: Mapping) -> "RuntimeCheckpoint":
        names = {f.name for f in dataclasses.fields(cls)}
        missing = {"version", "clip_state", "noise_state", "sample_rate", "target_delta", "noise_multiplier", "total_steps"} - set(d)
        if missing:
            raise ValueError(f"dp_state bundle lacks {sorted(missing)}")
        return cls(**{k: v for k, v in d.items() if k in names})


def save_runtime_checkpoint(bundle: RuntimeCheckpoint, path: str) -> None:
    """Write ``dp_state.pt``: ``torch.save`` of the bundle as a plain dict."""
    torch.save(bundle.to_dict(), path)


class _BundleUnpickler(pickle.Unpickler):
    """Resolves the reference's ``RuntimeCheckpoint`` class (and nothing else of its packages) to this module's."""

    def find_class(self, module, name):
        if name == "RuntimeCheckpoint" and module.endswith("trainer._checkpoint"):
            return _ForeignBundle
        return super().find_class(module, name)


class _ForeignBundle:
    """Receives the attribute dict of a pickled foreign dataclass instance."""

    def __setstate__(self, state):
        self.__dict__.update(state)


class _BundlePickle:
    """``pickle_module`` for ``torch.load`` with the class resolution above."""
    __name__ = "pickle"
    Unpickler = _BundleUnpickler
    load = staticmethod(lambda f, **kw: _BundleUnpickler(f, **kw).load())
    loads = staticmethod(pickle.loads)
    dumps = staticmethod(pickle.dumps)
    dump = staticmethod(pickle.dump)
    Pickler = pickle.Pickler
    HIGHEST_PROTOCOL = pickle.HIGHEST_PROTOCOL
    DEFAULT_PROTOCOL = pickle.DEFAULT_PROTOCOL
    PickleError = pickle.PickleError
    UnpicklingError = pickle.UnpicklingError
    PicklingError = pickle.PicklingError


def load_runtime_checkpoint(path: str) -> RuntimeCheckpoint:
    """Read ``dp_state.pt`` written by this trainer (a dict) or by the reference's trainer (its dataclass instance)."""
    obj = torch.load(path, map_location="cpu", weights_only=False, pickle_module=_BundlePickle)
    if isinstance(obj, _ForeignBundle):
        obj = dict(obj.__dict__)
    if not isinstance(obj, Mapping):
        raise TypeError(f"{path} does not hold a dp_state bundle (got {type(obj).__name__})")
    bundle = RuntimeCheckpoint.from_dict(obj)
    if bundle.version != DP_STATE_BUNDLE_VERSION:
        raise ValueError(f"unsupported dp_state bundle version {bundle.version} (expected {DP_STATE_BUNDLE_VERSION})")
    return bundle


def build_lr_schedule(args: TrainingArguments, max_steps: int):
    """HF scheduler names → schedule recipes (multiplied into ``learning_rate``)."""
    lr, w, kw = args.learning_rate, args.warmup_steps, dict(args.lr_scheduler_kwargs)
    decay = max(1, max_steps - w)
    name = args.lr_scheduler
    if name == "constant":
        base = sched.constant_schedule(lr)
    elif name in ("linear", "polynomial"):
        power = kw.get("power", 1.0) if name == "polynomial" else 1.0
        base = sched.polynomial_schedule(lr, kw.get("lr_end", 0.0), power, decay, transition_begin=w)
    elif name in ("cosine", "cosine_with_min_lr"):
        base = sched.cosine_schedule(lr, kw.get("min_lr", 0.0), decay, transition_begin=w, num_cycles=kw.get("num_cycles", 0.5))
    elif name == "cosine_with_restarts":
        cycles = int(kw.get("num_cycles", 1))
        base = sched.with_restarts(sched.cosine_schedule(lr, 0.0, max(1, decay // cycles)), decay, cycles, transition_begin=w)
    elif name == "inverse_sqrt":
        base = sched.inverse_sqrt_schedule(lr, kw.get("timescale", max(w, 1)), transition_begin=w)
    elif name in ("warmup_stable_decay", "wsd"):
        nd = int(kw.get("num_decay_steps", max(1, max_steps // 10)))
        return sched.warmup_stable_decay(lr, kw.get("min_lr", 0.0), num_warmup_steps=max(w, 1),
                                         num_stable_steps=max(0, max_steps - max(w, 1) - nd), num_decay_steps=nd,
                                         decay_shape=kw.get("decay_shape", "1-sqrt"))
    elif name == "exponential":
        base = sched.exponential_schedule(lr, kw.get("decay_rate", 0.99), transition_begin=w)
    else:
        raise ValueError(f"unknown lr_scheduler {name!r}")
    return sched.with_warmup(base, w) if w > 0 else base


def build_optimizer(args: TrainingArguments, lr) -> optim_lib.GradientTransformation:
    """Canonical optimizer names → functional optimizers; ``adamw-bc`` = AdamW with noise bias correction."""
    betas = (args.adam_beta1, args.adam_beta2)
    extra = dict(args.optim_args)
    name = args.optim
    if name == "adamw-bc":
        return optim_lib.adamw(lr, betas, args.adam_epsilon, args.weight_decay, noise_bias_correction=True, **extra)
    if name == "adamw":
        return optim_lib.adamw(lr, betas, args.adam_epsilon, args.weight_decay, **extra)
    if name == "adam":
        return optim_lib.adam(lr, betas, args.adam_epsilon, args.weight_decay, **extra)
    if name == "sgd":
        return optim_lib.sgd(lr, weight_decay=args.weight_decay, **extra)
    if name == "lion":
        return optim_lib.lion(lr, (args.adam_beta1, extra.pop("beta2", 0.99)), args.weight_decay, **extra)
    if name in ("adagrad", "rmsprop", "radam", "adadelta", "adafactor", "ademamix", "schedule_free_adamw", "schedule_free_sgd"):
        return getattr(optim_lib, name)(lr, weight_decay=args.weight_decay, **extra)
    raise ValueError(f"unknown optimizer {name!r}")


def build_strategy(mechanism: str, kwargs: Mapping[str, Any]) -> ftrl_noise.MfStrategy:
    table = {"mf_band": ftrl_noise.band_mf_strategy, "mf_blt": ftrl_noise.blt_strategy, "mf_bisr": ftrl_noise.bisr_strategy,
             "mf_bsr": ftrl_noise.bsr_strategy, "mf_lambda_cgd": ftrl_noise.lambda_cgd_strategy,
             "mf_identity": lambda **k: ftrl_noise.identity_strategy()}
    return table[mechanism](**dict(kwargs))


def list_checkpoints(output_dir: str) -> list[str]:
    if not output_dir or not os.path.isdir(output_dir):
        return []
    found = [(int(m.group(1)), d) for d in os.listdir(output_dir) if (m := CHECKPOINT_RE.match(d))]
    return [os.path.join(output_dir, d) for _, d in sorted(found)]


def rotate_checkpoints(output_dir: str, limit: int | None, keep: str | None = None) -> None:
    if not limit or limit <= 0:
        return
    ckpts = [c for c in list_checkpoints(output_dir) if c != keep]
    excess = len(ckpts) + (1 if keep else 0) - limit
    for c in ckpts[:max(0, excess)]:
        shutil.rmtree(c, ignore_errors=True)


def _is_retryable_oom(exc: BaseException) -> bool:
    return isinstance(exc, torch.OutOfMemoryError) or (isinstance(exc, RuntimeError) and "out of memory" in str(exc).lower())


def default_per_example_loss(model_call: Callable[..., Any], example: Mapping[str, torch.Tensor],
                             label_smoothing: float = 0.0) -> torch.Tensor:
    """Mean next-token NLL of ONE example (no batch axis), labels already aligned; with ``label_smoothing`` the target
    distribution is ``(1 − s)·one-hot + s·uniform`` (mean over the scored tokens, as ``torch.nn.functional.cross_entropy``)."""
    from ..alignment.sft import nll_loss
    ids = example["input_ids"].unsqueeze(0)
    logits = model_call(ids)
    logits = getattr(logits, "logits", logits)
    if label_smoothing:
        return torch.nn.functional.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), example["labels"].reshape(-1),
                                                 ignore_index=-100, label_smoothing=float(label_smoothing))
    return nll_loss(logits, example["labels"].unsqueeze(0)).squeeze(0)


# ------------------------------------------------------------------------------------------ trainer

class DPTrainer:
    """Differentially private trainer with the call surface of the Hugging Face ``Trainer``.

    Owns sampling (Poisson and the DP-FTRL participation schemes), per-example clipping, noise, the privacy
    accountant, evaluation, callbacks and checkpoints (resume replays batches and noise exactly).  Gradients come from
    the fused B200 engine or from the functional reference engine (``args.dp_engine``; ``engine_kind`` tells which).
    Parity: packages/opaque-transformers/src/opaque/api/transformers/trainer/_dp_trainer.py of the reference.
    """

    def __init__(self, model: torch.nn.Module | None = None, args: TrainingArguments | None = None,
                 data_collator: Callable | None = None, train_dataset: Any = None, eval_dataset: Any = None,
                 processing_class: Any = None, compute_loss_func: Callable | None = None,
                 compute_metrics: Callable | None = None, callbacks: Sequence[TrainerCallback] | None = None,
                 optimizers: tuple = (None, None), optimizer_cls_and_kwargs: tuple | None = None,
                 preprocess_logits_for_metrics: Callable | None = None):
        if model is None:
            raise ValueError("DPTrainer needs a model")
        self.model = model
        self.args = args or TrainingArguments()
        self.train_dataset, self.eval_dataset = train_dataset, eval_dataset
        self.processing_class = processing_class
        self.compute_loss_func = compute_loss_func
        self.compute_metrics = compute_metrics
        self.preprocess_logits_for_metrics = preprocess_logits_for_metrics
        self.optimizers = optimizers
        self.optimizer_cls_and_kwargs = optimizer_cls_and_kwargs
        self.state = DPTrainerState()
        self.control = TrainerControl()
        self.callbacks: list[TrainerCallback] = [PrinterCallback(), BestModelSaveCallback(), *reporting_callbacks(self.args.report_to),
                                                 *(callbacks or [])]
        if data_collator is None:
            from ..alignment.data import language_modeling_collator
            pad = getattr(processing_class, "pad_token_id", None) or 0
            data_collator = lambda rows: language_modeling_collator(rows, pad_token_id=pad)
        self.data_collator = data_collator
        self.accountant: acc.Accountant | None = None
        self.perf = None
        self._ddp_init()

    # ---- distributed bootstrap ----------------------------------------------------------------
    def _ddp_init(self) -> None:
        a = self.args
        if a.world_size > 1 and not dist.is_initialized():
            backend = a.ddp_backend or ("nccl" if torch.cuda.is_available() and not a.use_cpu else "gloo")
            if backend not in ("nccl", "gloo", "mpi"):
                raise ValueError(f"unsupported ddp_backend {backend!r} (nccl, gloo, mpi)")
            import datetime
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group(backend, init_method="env://", timeout=datetime.timedelta(seconds=a.ddp_timeout))
        if torch.cuda.is_available() and not a.use_cpu:
            torch.cuda.set_device(a.local_process_index)
            self.device = torch.device("cuda", a.local_process_index)
        else:
            self.device = torch.device("cpu")
        self.model.to(self.device)

    # ---- small parts of the Hugging Face Trainer surface that user scripts rely on -----------------------------
    def is_world_process_zero(self) -> bool:
        return self.args.process_index == 0

    def is_local_process_zero(self) -> bool:
        return self.args.local_process_index == 0

    def add_callback(self, callback: "TrainerCallback | type") -> None:
        self.callbacks.append(callback() if isinstance(callback, type) else callback)

    def pop_callback(self, callback: "TrainerCallback | type") -> "TrainerCallback | None":
        for i, cb in enumerate(self.callbacks):
            if cb is callback or (isinstance(callback, type) and isinstance(cb, callback)):
                return self.callbacks.pop(i)
        return None

    def remove_callback(self, callback: "TrainerCallback | type") -> None:
        self.pop_callback(callback)

    def num_examples(self, dataset: Any = None) -> int:
        return len(dataset if dataset is not None else self.train_dataset)

    def create_model_card(self, model_name: str | None = None, **fields: Any) -> str:
        """Write ``README.md`` into ``output_dir`` with the privacy statement of the run (ε, δ, mechanism, sampling)."""
        a = self.args
        eps = self.epsilon() if self.accountant is not None else float("nan")
        lines = [f"# {model_name or os.path.basename(a.output_dir.rstrip('/')) or 'model'}", "",
                 "Trained with differential privacy.", "",
                 f"- privacy guarantee: ({eps:.4g}, {getattr(self, 'target_delta', a.privacy_target_delta)})-DP",
                 f"- mechanism: {a.privacy_noise_mechanism}; sampling: {a.sampling_mode}; clipping: {a.clipping_mode} at {a.clipping_norm}",
                 f"- noise multiplier: {getattr(self, 'noise_multiplier', a.privacy_noise_multiplier)}; steps: {self.state.global_step}"]
        lines += [f"- {k}: {v}" for k, v in fields.items()]
        text = "\n".join(lines) + "\n"
        if a.output_dir and self.is_world_process_zero():
            os.makedirs(a.output_dir, exist_ok=True)
            with open(os.path.join(a.output_dir, "README.md"), "w") as f:
                f.write(text)
        return text

    def push_to_hub(self, commit_message: str | None = "End of training", blocking: bool = True, token: str | None = None,
                    revision: str | None = None, **kwargs: Any) -> Any:
        """Save the model and its model card into ``output_dir`` and upload that folder to the Hub in one commit
        (``hub_model_id`` / ``hub_token`` / ``hub_private_repo`` / ``hub_revision``).  Checkpoint folders and run-state files
        (noise and sampler keys) are never uploaded; see :mod:`opaque_b200.transformers.hub`.  ``self.hub_client`` (or
        ``client=``) replaces ``huggingface_hub.HfApi``."""
        from . import hub
        return hub.push_to_hub(self, commit_message, blocking, token, revision, **kwargs)

    # ---- Hugging Face Trainer conveniences -----------------------------------------------------------------------
    @property
    def callback_handler(self) -> "DPTrainer":
        """The object that owns ``callbacks`` / ``add_callback`` / ``pop_callback`` / ``remove_callback`` (this trainer)."""
        return self

    def init_hf_repo(self, token: str | None = None) -> str:
        """Create the Hub repository named by ``hub_model_id`` (or ``output_dir``) if needed; returns its id."""
        from . import hub
        return hub.init_hub_repo(self, token=token)

    def create_scheduler(self, num_training_steps: int | None = None, optimizer: Any = None):
        """The learning-rate schedule of this run (a ``scheduling`` recipe, ``schedule(step) -> lr``)."""
        steps = int(num_training_steps or self.state.max_steps or self.args.max_steps or 1)
        self.lr_schedule = build_lr_schedule(self.args, steps)
        return self.lr_schedule

    def create_optimizer(self):
        """The functional optimizer chain for ``args.optim`` (what the reference engine steps with)."""
        schedule = getattr(self, "lr_schedule", None) or self.create_scheduler()
        return build_optimizer(self.args, schedule)

    def get_eval_dataloader(self, eval_dataset: Any = None):
        """Collated evaluation batches of THIS rank's shard, ``eval_batch_size`` rows each (an iterable with ``len``)."""
        data = eval_dataset if eval_dataset is not None else self.eval_dataset
        if data is None:
            raise ValueError("evaluation needs an eval_dataset")
        shard = local_shard(data, rank=self.args.process_index, world_size=self.args.world_size)
        bs, collate = self.args.eval_batch_size, self.data_collator

        class _Batches:
            def __len__(_):
                return (len(shard) + bs - 1) // bs

            def __iter__(_):
                for lo in range(0, len(shard), bs):
                    yield collate([shard[i] for i in range(lo, min(len(shard), lo + bs))])
        return _Batches()

    @torch.no_grad()
    def prediction_step(self, model: Any, inputs: Mapping[str, torch.Tensor], prediction_loss_only: bool,
                        ignore_keys: Any = None) -> tuple[torch.Tensor | None, Any, Any]:
        """``(mean loss, logits, labels)`` of one collated batch (logits and labels ``None`` with ``prediction_loss_only``)."""
        batch = self._to_device(inputs)
        loss = self.compute_batch_per_example_loss(batch).float().mean() if "labels" in batch else None
        if prediction_loss_only or "input_ids" not in batch:
            return loss, None, None
        logits = model(batch["input_ids"])
        return loss, getattr(logits, "logits", logits), batch.get("labels")

    def compute_per_example_loss_and_metrics(self, model_call: Callable[..., Any], example: Mapping[str, torch.Tensor]):
        """``(loss, metrics)`` of ONE record; the default has no extra metrics.  Override together with
        :meth:`compute_per_example_loss` when a task wants to log per-record quantities of NON-private evaluation data."""
        return self.compute_per_example_loss(model_call, example), {}

    def log_metrics(self, split: str, metrics: Mapping[str, Any]) -> None:
        """Print a metrics block the way the Hugging Face trainer does (rank 0 only)."""
        if not self.is_world_process_zero():
            return
        rows = {k: (f"{v:.4f}" if isinstance(v, float) else str(v)) for k, v in sorted(metrics.items())}
        width = max((len(k) for k in rows), default=0)
        print(f"***** {split} metrics *****")
        for k, v in rows.items():
            print(f"  {k:<{width}} = {v:>10}")

    def save_metrics(self, split: str, metrics: Mapping[str, Any], combined: bool = True) -> None:
        """Write ``{split}_results.json`` into ``output_dir`` and (``combined``) merge into ``all_results.json``."""
        if not self.is_world_process_zero() or not self.args.output_dir:
            return
        os.makedirs(self.args.output_dir, exist_ok=True)
        plain = to_python(dict(metrics))
        with open(os.path.join(self.args.output_dir, f"{split}_results.json"), "w") as f:
            json.dump(plain, f, indent=4, sort_keys=True)
        if combined:
            path = os.path.join(self.args.output_dir, "all_results.json")
            merged = json.load(open(path)) if os.path.exists(path) else {}
            merged.update(plain)
            with open(path, "w") as f:
                json.dump(merged, f, indent=4, sort_keys=True)

    def save_state(self) -> None:
        """Write ``trainer_state.json`` (step, log history, best metric) into ``output_dir``."""
        if not self.is_world_process_zero() or not self.args.output_dir:
            return
        os.makedirs(self.args.output_dir, exist_ok=True)
        with open(os.path.join(self.args.output_dir, FILES["trainer_state"]), "w") as f:
            f.write(self.state.to_json())

    def save_accountant(self, output_dir: str | None = None) -> str | None:
        """Write the accountant (process tree + budget) as ``accountant.json``; returns the path (rank 0), else ``None``."""
        out = output_dir or self.args.output_dir
        if not self.is_world_process_zero() or not out or getattr(self, "accountant", None) is None:
            return None
        os.makedirs(out, exist_ok=True)
        path = os.path.join(out, FILES["accountant"])
        with open(path, "w") as f:
            f.write(self.accountant.to_json())
        return path

    def _call(self, hook: str, **kw: Any) -> None:
        for cb in self.callbacks:
            getattr(cb, hook)(self.args, self.state, self.control, model=self.model, **kw)

    # ---- overridable task hooks -----------------------------------------------------------------
    def compute_per_example_loss(self, model_call: Callable[..., Any], example: Mapping[str, torch.Tensor]) -> torch.Tensor:
        """Loss of ONE record (reference engine; runs under ``vmap``)."""
        if self.compute_loss_func is not None:
            return self.compute_loss_func(model_call, example)
        return default_per_example_loss(model_call, example, self.args.label_smoothing_factor)

    def compute_batch_per_example_loss(self, batch: Mapping[str, torch.Tensor]) -> torch.Tensor:
        """One loss per record of a batch (fused engine, evaluation)."""
        if hasattr(self.model, "per_example_loss"):
            return self.model.per_example_loss(batch["input_ids"], batch["labels"])
        out = [self.compute_per_example_loss(self.model, {k: v[i] for k, v in batch.items()}) for i in range(len(batch["input_ids"]))]
        return torch.stack(out) if out else torch.zeros(0, device=self.device)

    # ---- set-up -----------------------------------------------------------------------------------
    def _fused_blockers(self) -> list[str]:
        """Reasons why this run cannot use the fused engine (empty list: it can)."""
        why = []
        if self.device.type != "cuda":
            why.append("no CUDA device")
        if not hasattr(self.model, "per_example_loss"):
            why.append("the model has no per_example_loss (convert it with opaque_b200.patches)")
        if self.compute_loss_func is not None:
            why.append("compute_loss_func is set")
        if self.args.label_smoothing_factor:        # label smoothing lives in the trainer's default loss (reference engine)
            why.append("label_smoothing_factor is set")
        if not why:
            from ..device import fused_kernels_available
            if not fused_kernels_available():
                why.append("the sm_100a kernel library is not available")
        return why

    def _resolve_engine(self) -> str:
        want = self.args.dp_engine
        why = self._fused_blockers()
        if want == "fused" and why:
            raise RuntimeError("dp_engine='fused' is not possible here: " + "; ".join(why))
        if want == "auto" and why and self.device.type == "cuda":
            # the vmap engine is several times slower on a GPU: never take it silently
            import warnings
            warnings.warn("dp_engine='auto' falls back to the reference (vmap) engine: " + "; ".join(why), RuntimeWarning,
                          stacklevel=3)
        return "fused" if (want in ("auto", "fused") and not why) else "reference"

    def _fused_loss_fn(self):
        """Per-example loss the fused engine differentiates (keyword arguments = the entries of :meth:`_fused_payload`)."""
        return self.model.per_example_loss

    def _fused_payload(self, batch) -> dict[str, torch.Tensor]:
        """Tensors of one local batch, leading dimension = privacy units."""
        return {"input_ids": batch["input_ids"], "labels": batch["labels"]}

    def _build_sampler(self, n_local: int, steps: int, data_key: RngKey):
        a = self.args
        ranks = a.world_size if getattr(self, "_balanced", False) else 1        # a global draw covers all ranks' batches
        q = min(1.0, a.per_device_train_batch_size * ranks / max(n_local, 1))
        kw = dict(a.sampling_kwargs)
        mode = a.sampling_mode
        rng = range(n_local)
        cap = self._truncation_cap()
        self._sampled_records = n_local          # the population one draw runs over (the accountant's dataset_size)
        if mode == "poisson":
            return PoissonSampler(rng, q, n_steps=steps, truncated_batch_size=cap, key=data_key), q
        if mode == "random_allocation":
            bins = int(kw.get("num_bins", max(1, round(1 / q))))
            return RandomAllocationSampler(rng, bins, n_steps=steps, key=data_key), 1.0 / bins
        if mode == "k_out_of_t":
            t = int(kw.get("t", max(1, round(1 / q))))
            return KOutOfTSampler(rng, int(kw.get("k", 1)), t, n_steps=steps, key=data_key), kw.get("k", 1) / t
        bands = int(a.privacy_noise_mechanism_kwargs.get("bands", a.privacy_noise_mechanism_kwargs.get("bandwidth", kw.get("bands", 1))))
        if mode == "cyclic_poisson":
            return CyclicPoissonSampler(rng, min(1.0, q * bands), bands=bands, n_steps=steps, key=data_key,
                                        **({"truncated_batch_size": cap} if cap is not None else {})), min(1.0, q * bands)
        if mode == "b_min_sep":
            return BMinSepSampler(rng, bands, q, steps, key=data_key), q
        if mode == "balls_in_bins":
            bins = int(kw.get("num_bins", max(1, round(1 / q))))
            return BallsInBinsSampler(rng, bins, n_steps=steps, key=data_key), 1.0 / bins
        if mode == "sequential":
            return SequentialBatchSampler(rng, min(a.per_device_train_batch_size, n_local), n_steps=steps), q
        raise ValueError(mode)

    def _truncation_cap(self) -> int | None:
        """``sampling_kwargs['truncated_batch_size']`` (alias ``max_batch_size``): a hard cap on the Poisson batch.

        Truncation changes the mechanism, so the cap is also handed to the accountant; sampling modes that cannot
        truncate refuse the key instead of ignoring it (reference: trainer/_dp_trainer.py:4238-4296).
        """
        kw = self.args.sampling_kwargs if isinstance(self.args.sampling_kwargs, Mapping) else {}
        raw = kw.get("truncated_batch_size", kw.get("max_batch_size"))
        if raw is None:
            return None
        if self.args.sampling_mode not in ("poisson", "cyclic_poisson"):
            raise ValueError(f"sampling_kwargs['truncated_batch_size'] applies to Poisson sampling only, not to "
                             f"sampling_mode={self.args.sampling_mode!r}")
        cap = int(raw)
        if cap < 1:
            raise ValueError("truncated_batch_size must be >= 1")
        return cap

    def _participation(self, sampler, steps: int) -> tuple[int, int | None]:
        """(min_sep, max_participations) implied by the sampler for MF sensitivity."""
        sampler = getattr(sampler, "inner", sampler)           # BalancedRankSampler wraps the global sampler
        if isinstance(sampler, BallsInBinsSampler):
            return sampler.num_bins, math.ceil(steps / sampler.num_bins)
        if isinstance(sampler, SequentialBatchSampler):
            return sampler.min_sep, math.ceil(steps / sampler.min_sep)
        if isinstance(sampler, (CyclicPoissonSampler, BMinSepSampler)):
            return sampler.bands, math.ceil(steps / sampler.bands)
        return 1, None

    def _step_process(self, nm: float, q: float, steps: int, sampler) -> acc.DpProcess:
        """The accountant's description of ONE step at noise multiplier ``nm``."""
        a = self.args
        sampler = getattr(sampler, "inner", sampler)
        W = a.world_size
        if a.privacy_noise_mechanism == "gaussian":
            g: acc.DpProcess = sgd_acc.gaussian(nm)
            if a.clipping_mode == "adaptive":
                g = sgd_acc.adaclip(g, fraction_noise_std=float(a.clipping_kwargs.get("fraction_noise_std", 0.05)),
                                    expected_batch_size=float(a.train_batch_size),
                                    num_groups=len(a.clipping_norm) if isinstance(a.clipping_norm, Mapping) else 1)
            if a.sampling_mode == "poisson":
                # disjoint shards: each record is sampled by one rank at rate q; with a cap the truncated mechanism is
                # accounted over the population that one draw runs over
                cap = self._truncation_cap()
                if cap is not None:
                    return sgd_acc.poisson(g, q, truncated_batch_size=cap, dataset_size=int(self._sampled_records))
                return sgd_acc.poisson(g, q)
            if a.sampling_mode == "random_allocation":
                return acc.per_step(_EpochProcess(sgd_acc.random_allocation(g, sampler.num_bins), sampler.num_bins))
            if a.sampling_mode == "k_out_of_t":
                return acc.per_step(_EpochProcess(sgd_acc.k_out_of_t(g, sampler.k, sampler.t), sampler.t))
            return g
        strat = self._strategy
        ms, mp = self._participation(sampler, steps)
        inner = ftrl_acc.mf_gaussian(nm, strat, n_steps=steps, min_sep=ms, max_participations=mp)
        if a.sampling_mode in ("cyclic_poisson",):
            cap = self._truncation_cap()
            extra = dict(truncated_batch_size=cap, dataset_size=int(self._sampled_records)) if cap is not None else {}
            return ftrl_acc.per_step(ftrl_acc.poisson(inner, q, n_steps=steps, **extra))
        if a.sampling_mode == "b_min_sep" and a.sampling_kwargs.get("amplified", False):
            n_coef = len(np.trim_zeros(np.asarray(strat.coefficients(steps), float), "b"))
            if n_coef <= sampler.bands:          # Monte-Carlo accountant for the subsampled banded mechanism
                return ftrl_acc.per_step(ftrl_acc.b_min_sep(ftrl_acc.mf_gaussian(nm, strat, n_steps=steps), bands=sampler.bands,
                                                           n_steps=steps, sampling_prob=sampler.sampling_prob))
        if a.sampling_mode == "poisson" and a.privacy_noise_mechanism == "mf_identity":
            cap = self._truncation_cap()
            if cap is not None:
                return sgd_acc.poisson(sgd_acc.gaussian(nm), q, truncated_batch_size=cap, dataset_size=int(self._sampled_records))
            return sgd_acc.poisson(sgd_acc.gaussian(nm), q)
        return ftrl_acc.per_step(inner)

    def _calibrate(self, q: float, steps: int, sampler, prefix: acc.DpProcess | None) -> float:
        a = self.args
        if a.privacy_noise_multiplier is not None:
            return float(a.privacy_noise_multiplier)
        if a.privacy_target_epsilon is None:
            raise ValueError("set privacy_target_epsilon (calibrated noise) or privacy_noise_multiplier")
        budget = acc.epsilon_budget(a.privacy_target_epsilon, self.target_delta)
        kw = a.noise_calibration_kwargs
        res = acc.calibrate(budget, lambda nm: self._step_process(nm, q, steps, sampler) * steps, kw["min"], kw["max"],
                            tolerance=kw["tol"], prefix=prefix)
        return float(res.param)

    # fields that exist for call-compatibility with Hugging Face argument sets and have no effect here
    _INERT_FIELDS = ("overwrite_output_dir", "log_level_replica", "log_on_each_node",
                     "save_on_each_node", "restore_callback_states_from_checkpoint", "use_mps_device", "bf16_full_eval",
                     "local_rank", "average_tokens_across_devices",
                     "ignore_data_skip", "dataloader_num_workers", "dataloader_persistent_workers",
                     "dataloader_prefetch_factor", "dataloader_multiprocessing_context", "dataloader_in_order",
                     "dataloader_drop_last", "remove_unused_columns", "label_names", "disable_tqdm", "trackio_space_id",
                     "trackio_bucket_id", "trackio_static_space_id", "hub_model_id", "hub_token", "hub_private_repo",
                     "hub_revision", "torch_compile", "torch_compile_backend", "torch_compile_mode",
                     "performance_kernels_config", "use_compat_patches")

    def inert_arguments(self) -> dict[str, Any]:
        """Arguments that were set away from their default but change nothing in this trainer (data loading is
        index-based inside the DP sampler, the hub fields act only with ``push_to_hub``, no tracing compiler on the hot
        path)."""
        defaults = {f.name: (f.default if f.default is not dataclasses.MISSING else f.default_factory())
                    for f in dataclasses.fields(type(self.args)) if f.name in self._INERT_FIELDS}
        acting = {"hub_model_id", "hub_token", "hub_private_repo", "hub_revision"} if self.args.push_to_hub else set()
        return {k: getattr(self.args, k) for k, d in defaults.items()
                if k not in acting and getattr(self.args, k) != d and (getattr(self.args, k) or d)}       # None and {} both mean unset

    def _apply_runtime_flags(self) -> None:
        a = self.args
        if a.log_level not in ("passive", None, ""):
            import logging
            level = getattr(logging, str(a.log_level).upper(), None)
            if isinstance(level, int):
                logging.getLogger("opaque_b200").setLevel(level)
        if a.tf32 is not None:
            torch.backends.cuda.matmul.allow_tf32 = bool(a.tf32)
            torch.backends.cudnn.allow_tf32 = bool(a.tf32)
        if a.full_determinism:
            torch.use_deterministic_algorithms(True, warn_only=True)
            os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":4096:8")
        inert = self.inert_arguments()
        # settings that would change WHAT is trained if they were honoured are refused, not ignored
        refused = {k: v for k, v in inert.items() if k in ("torch_compile", "dataloader_drop_last", "use_mps_device", "label_names")}
        if refused:
            raise ValueError("these TrainingArguments cannot be honoured by this trainer (no tracing compiler on the hot path, batches "
                             "come from the DP sampler, CUDA / CPU devices only, labels are derived from input_ids): "
                             + ", ".join(f"{k}={v!r}" for k, v in sorted(refused.items())))
        if inert and self.is_world_process_zero():
            import warnings
            warnings.warn("these TrainingArguments are accepted for compatibility and have NO effect here: "
                          + ", ".join(f"{k}={v!r}" for k, v in sorted(inert.items())), RuntimeWarning, stacklevel=3)

    def _setup(self, resume: str | None) -> None:
        a = self.args
        self._apply_runtime_flags()
        torch.manual_seed(a.seed)
        if self.train_dataset is None:
            raise ValueError("training needs a train_dataset")
        W, rank = a.world_size, a.process_index
        n_total = len(self.train_dataset)
        per = n_total // W                                   # equal shards; the tail is trimmed
        # sampling_kwargs={"balance": True}: ONE global draw per step dealt out evenly over the ranks (every rank reads
        # any record); default: disjoint shards with an independent draw per rank, as in the reference
        self._balanced = bool(a.sampling_kwargs.get("balance", False)) and W > 1 and a.sampling_mode != "sequential"
        if self._balanced:
            self._local_data = _Trimmed(self.train_dataset, per * W)
            n_local = per * W
        else:
            self._local_data = local_shard(_Trimmed(self.train_dataset, per * W), rank=rank, world_size=W)
            n_local = per
        q_nominal = min(1.0, a.per_device_train_batch_size / max(per, 1))
        if a.max_steps > 0:
            steps = a.max_steps
        else:
            steps = max(1, math.ceil(a.num_train_epochs / q_nominal))
        self.state.max_steps = steps
        self.target_delta = a.privacy_target_delta if a.privacy_target_delta is not None else 1.0 / (n_total ** 1.1)
        data_key = fold_in(key(a.data_seed if a.data_seed is not None else a.seed), "global" if self._balanced else rank)
        self.sampler, self.sample_rate = self._build_sampler(n_local, steps, data_key)
        if self._balanced:
            from ..dpsgd.sampling import BalancedRankSampler
            self.sampler = BalancedRankSampler(self.sampler, rank, W)
        self._strategy = build_strategy(a.privacy_noise_mechanism, a.privacy_noise_mechanism_kwargs) \
            if a.privacy_noise_mechanism in MECHANISMS_DPFTRL else None
        self.engine_kind = self._resolve_engine()
        if self.engine_kind == "reference":
            # torch.func.grad under vmap supports neither saved-tensor hooks (offloading, torch.utils.checkpoint) nor the
            # checkpoint autograd node.  The framework's own models switch to functional_checkpoint there; anything else
            # is refused with the way out
            if a.activation_offloading:
                raise ValueError("activation_offloading needs the fused engine (dp_engine='fused' on a B200); on the "
                                 "reference engine lower microbatch_size or use gradient_checkpointing")
            if a.gradient_checkpointing and not hasattr(self.model, "activation_checkpointing"):
                raise ValueError("gradient_checkpointing on the reference engine needs a model of opaque_b200.models (or a "
                                 "converted Hugging Face model); lower microbatch_size instead")
        prefix = None
        runtime = None
        if resume:
            runtime, prefix = self._load_checkpoint_meta(resume)
        self.noise_multiplier = runtime.noise_multiplier if runtime else self._calibrate(self.sample_rate, steps, self.sampler, prefix)
        self.step_process = self._step_process(self.noise_multiplier, self.sample_rate, steps, self.sampler)
        self.accountant = acc.Accountant(
            acc.epsilon_budget(a.privacy_target_epsilon, self.target_delta) if a.privacy_target_epsilon else None, prefix)
        self.lr_schedule = build_lr_schedule(a, steps)
        self.expected_batch = float(a.train_batch_size)
        noise_key = key(a.seed + 1)
        mb = a.microbatch_size or a.per_device_train_batch_size
        self._microbatch = mb
        if self.engine_kind == "fused":
            self._setup_fused(noise_key, steps)
        else:
            self._setup_reference(noise_key, steps)
        if resume:
            self._load_checkpoint_state(resume, runtime)
        self.perf = perf_tracker(self.device, warmup_steps=1)

    def _clip_bound(self):
        a = self.args
        if isinstance(a.clipping_norm, Mapping):
            pats = {k: v for k, v in a.clipping_norm.items() if k != "fallback"}
            return per_group(self._trainable, pats, fallback=a.clipping_norm.get("fallback"))
        return float(a.clipping_norm)

    def _setup_reference(self, noise_key: RngKey, steps: int) -> None:
        a = self.args
        self._fmodel, self._trainable, self._frozen = make_functional(self.model, disable_autograd_tracking=True,
                                                                    partition_trainable=True)
        frozen, fmodel = self._frozen, self._fmodel

        def loss_fn(trainable, example):
            call = lambda *x, **k: fmodel({**frozen, **trainable}, *x, **k)
            return self.compute_per_example_loss(call, example)
        common = dict(normalize_by=self.expected_batch, batch_argnums=1, return_aux=True, microbatch_size=self._microbatch)
        bound = self._clip_bound()
        if a.clipping_mode == "fixed":
            self._grad_fn, self._clip_state = clipped_grad(loss_fn, clipping_norm=bound, **common)
        elif a.clipping_mode == "auto":
            self._grad_fn, self._clip_state = auto_clipped_grad(loss_fn, R=bound, gamma=float(a.clipping_kwargs.get("gamma", 0.01)), **common)
        else:
            kw = {k: v for k, v in a.clipping_kwargs.items()}
            self._grad_fn, self._clip_state = adaptive_clipped_grad(
                loss_fn, initial_clipping_norm=bound, key=fold_in(key(a.seed), "adaclip"), return_aux=True,
                normalize_by=self.expected_batch, batch_argnums=1, microbatch_size=self._microbatch, **kw)
        if self._strategy is None:
            self._noise_fn, self._noise_state = gaussian_noise(noise_multiplier=self.noise_multiplier, key=noise_key)
        else:
            ms, mp = self._participation(self.sampler, steps)
            from ..types import clipped
            self._noise_fn, self._noise_state = ftrl_noise.mf_gaussian_noise(
                clipped(self._trainable, 1.0), self._strategy, n_steps=steps, min_sep=ms, max_participations=mp,
                noise_multiplier=self.noise_multiplier, key=noise_key)
        self._optimizer = self.optimizers[0] or build_optimizer(a, self.lr_schedule)
        self._opt_state = self._optimizer.init(self._trainable)

    def _setup_fused(self, noise_key: RngKey, steps: int) -> None:
        from ..engine.fused import FusedDPEngine
        from ..parallel.sharded import DPStepConfig
        a = self.args
        extra = dict(a.optim_args)
        if a.optim in ("adamw", "adamw-bc", "adam"):
            cfg = DPStepConfig(lr=self.lr_schedule, betas=(a.adam_beta1, a.adam_beta2), eps=a.adam_epsilon,
                               weight_decay=a.weight_decay, decoupled_weight_decay=a.optim != "adam",
                               noise_bias_correction=a.optim == "adamw-bc")
        elif a.optim == "sgd" and not extra.get("dampening") and not extra.get("maximize"):
            # PyTorch semantics as in the functional optimizer: L2 weight decay folded into the gradient, optional momentum
            cfg = DPStepConfig(lr=self.lr_schedule, betas=(float(extra.get("momentum", 0.0)), 0.0), weight_decay=a.weight_decay,
                               decoupled_weight_decay=False, noise_bias_correction=False, optimizer="sgd",
                               nesterov=bool(extra.get("nesterov", False)))
        elif a.optim == "lion":
            cfg = DPStepConfig(lr=self.lr_schedule, betas=(a.adam_beta1, float(extra.get("beta2", 0.99))), weight_decay=a.weight_decay,
                               decoupled_weight_decay=bool(extra.get("decoupled_weight_decay", True)),
                               noise_bias_correction=False, optimizer="lion")
        else:
            raise ValueError("the fused engine implements Adam / AdamW / AdamW-BC, SGD (momentum, Nesterov) and Lion; use "
                             "dp_engine='reference' for other optimizers")
        mech = self._strategy.fused_mechanism(steps) if self._strategy is not None else None
        bound: Any = float(a.clipping_norm) if not isinstance(a.clipping_norm, Mapping) else None
        group_of = None
        if bound is None:                      # {"substring": C, ..., "fallback": C}: first matching pattern wins
            pats = [k for k in a.clipping_norm if k != "fallback"]

            def group_of(name: str) -> str:
                hit = next((p for p in pats if p in name), None)
                if hit is None and "fallback" not in a.clipping_norm:
                    raise ValueError(f"parameter {name!r} matches no group pattern and no fallback was given")
                return hit or "fallback"
            used = {group_of(n) for n, p in self.model.named_parameters() if p.requires_grad}
            bound = {g: float(a.clipping_norm[g]) for g in used}
        adaptive = None
        if a.clipping_mode == "adaptive":
            from ..dpsgd.clipping import AdaptiveClipState
            kw = dict(a.clipping_kwargs)
            adaptive = AdaptiveClipState(bound if not isinstance(bound, Mapping) else per_group(
                {n: p for n, p in self.model.named_parameters() if p.requires_grad},
                {k: v for k, v in a.clipping_norm.items() if k != "fallback"}, fallback=a.clipping_norm.get("fallback")),
                0, float(kw.get("target_quantile", 0.5)), float(kw.get("learning_rate", 0.2)),
                float(kw.get("clipping_norm_min", 0.01)), float(kw.get("clipping_norm_max", 100.0)),
                float(kw.get("fraction_noise_std", 0.05)), fold_in(key(a.seed), "adaclip"))
        self._fused = FusedDPEngine(self.model, clipping_norm=bound, noise_multiplier=self.noise_multiplier,
                                    normalize_by=self.expected_batch, key=noise_key, step_config=cfg,
                                    microbatch_size=self._microbatch, mechanism=mech,
                                    clipping_mode="auto" if a.clipping_mode == "auto" else "clip",
                                    gamma=float(a.clipping_kwargs.get("gamma", 0.01)), group_of=group_of, adaptive=adaptive,
                                    cuda_graph=a.dp_cuda_graph)
        self._graphs_ready = not a.dp_cuda_graph
        if a.include_sync_metrics:          # CUDA events around barrier / shard step / barrier, read where the step's metrics are read
            self._fused.opt.timing = []
        # host-side leave notices: a rank that stops between steps tells the others through the rendezvous store, so they
        # raise before their next device barrier instead of waiting for its flag until the bounded wait runs out
        self._liveness = None
        if is_distributed() and self._fused.group.world > 1:
            from ..parallel.peer import Liveness
            self._liveness = Liveness(self._fused.group.rank, self._fused.group.world)

    # ---- data -----------------------------------------------------------------------------------
    def get_train_dataloader(self):
        """Iterator of collated local batches (possibly EMPTY under Poisson sampling)."""
        data, collate = self._local_data, self.data_collator
        for idx in self.sampler:
            yield collate([data[i] for i in idx])

    def _to_device(self, batch: Mapping[str, torch.Tensor]) -> dict[str, torch.Tensor]:
        pin = self.args.dataloader_pin_memory and self.device.type == "cuda"
        out = {}
        for k, v in batch.items():
            if isinstance(v, torch.Tensor):
                out[k] = (v.pin_memory() if pin and v.numel() else v).to(self.device, non_blocking=True)
            else:
                out[k] = v
        return out

    # ---- one step ---------------------------------------------------------------------------------
    def training_step(self, batch: Mapping[str, torch.Tensor]) -> dict[str, float]:
        """One DP optimizer step on this rank's batch; returns scalar metrics (global where meaningful)."""
        a = self.args
        self._call("on_step_begin")
        batch = self._to_device(batch)
        n_local = int(next(v for v in batch.values() if isinstance(v, torch.Tensor)).shape[0])
        with self.perf.step("train", batch_size=n_local, track_memory=not a.skip_memory_metrics) as sp:
            if self.engine_kind == "fused":
                metrics = self._fused_step(batch, sp)
            else:
                metrics = self._reference_step(batch, sp)
        self.state.global_step += 1
        self.accountant |= self.step_process
        self._call("on_step_end")
        return metrics

    def _cluster_flag(self, flag: bool) -> bool:
        return bool(reduce_scalar(int(flag), "max")) if is_distributed() else flag

    def _reference_step(self, batch, sp) -> dict[str, float]:
        a = self.args
        payload = {"input_ids": batch["input_ids"], "labels": batch["labels"]}
        payload.update({k: v for k, v in batch.items() if k not in payload and isinstance(v, torch.Tensor) and v.shape[:1] == batch["input_ids"].shape[:1]})
        while True:
            oom = False
            try:
                from ..ops.functional import plain_torch_ops
                with plain_torch_ops():          # vmap needs plain PyTorch ops (no custom autograd nodes)
                    (grads, aux), clip_state = self._grad_fn(self._trainable, payload, state=self._clip_state)
            except Exception as exc:      # noqa: BLE001 — only OOM is swallowed, and only with auto_find_microbatch_size
                if not (self.args.auto_find_microbatch_size and _is_retryable_oom(exc)):
                    raise
                oom = True
            if not (self.args.auto_find_microbatch_size and self._cluster_flag(oom)):
                break
            if self._microbatch <= 1:
                raise torch.OutOfMemoryError("out of memory at microbatch size 1")
            self._microbatch = max(1, self._microbatch // 2)      # every rank steps down together and replays
            self._setup_reference_grad_only()
        sp.mark("clip")
        grads = sum_gradients_(grads)
        self._clip_state = sync(clip_state)
        aux = sync(aux)
        self._call("on_pre_optimizer_step")
        noisy, self._noise_state = self._noise_fn(grads, self._noise_state)
        sp.mark("noise")
        updates, self._opt_state = self._optimizer.update(noisy, self._opt_state, params=self._trainable)
        self._trainable = optim_lib.apply_updates(self._trainable, updates)
        self._write_back()
        sp.mark("optimizer")
        self._call("on_optimizer_step")
        n = aux.batch_size
        out = {"loss": float(aux.loss_values.mean()) if n else 0.0, "grad_norm": float(aux.grad_norms.mean()) if n else 0.0,
               "clip_rate": float(aux.clipping_rate) if isinstance(aux.clipping_rate, (int, float)) else 0.0,
               "batch_size": float(n), "noise_std": float(noisy.noise_stddev) if isinstance(noisy.noise_stddev, (int, float)) else 0.0,
               "clipping_norm": float(getattr(self._clip_state, "clipping_norm", a.clipping_norm)) if not isinstance(a.clipping_norm, Mapping) else 0.0}
        if "labels" in batch:
            self.state.num_input_tokens_seen += int(reduce_scalar(int((batch["labels"] != -100).sum()), "sum"))
        return out

    def _setup_reference_grad_only(self) -> None:
        saved = (self._noise_fn, self._noise_state, self._optimizer, self._opt_state, self._trainable)
        self._setup_reference(key(self.args.seed + 1), self.state.max_steps)
        self._noise_fn, self._noise_state, self._optimizer, self._opt_state, self._trainable = saved

    @torch.no_grad()
    def _write_back(self) -> None:
        named = dict(self.model.named_parameters())
        for n, v in self._trainable.items():
            named[n].copy_(v)

    def _fused_step(self, batch, sp) -> dict[str, float]:
        if getattr(self, "_liveness", None) is not None:
            self._liveness.check()
        self._call("on_pre_optimizer_step")
        payload = self._fused_payload(batch)
        loss_fn = self._fused_loss_fn()
        if not self._graphs_ready and payload["input_ids"].shape[0]:
            self._fused.prepare_graphs(loss_fn, payload)
            self._graphs_ready = True
        while True:                                   # cluster-wide agreement on out-of-memory, then a smaller microbatch
            oom = False
            try:
                res = self._fused.accumulate(loss_fn, payload)
            except Exception as exc:      # noqa: BLE001 — only OOM is swallowed, and only with auto_find_microbatch_size
                if not (self.args.auto_find_microbatch_size and _is_retryable_oom(exc)):
                    raise
                oom = True
            if not (self.args.auto_find_microbatch_size and self._cluster_flag(oom)):
                break
            if self._fused.microbatch_size <= 1:
                raise torch.OutOfMemoryError("out of memory at microbatch size 1")
            torch.cuda.empty_cache()
            self._fused.reset_gradients()
            self._fused.microbatch_size = self._microbatch = max(1, self._fused.microbatch_size // 2)
        res = self._fused.apply(res)
        sp.mark("optimizer")
        self._call("on_optimizer_step")
        n = int(reduce_scalar(res.batch_size, "sum")) if is_distributed() else res.batch_size
        if "labels" in batch:
            self.state.num_input_tokens_seen += int(reduce_scalar(int((batch["labels"] != -100).sum()), "sum"))
        sync_ms = {}
        if self._fused.opt.timing is not None:
            sync_ms = {f"sync/{k}": v for k, v in self._fused.opt.timing_ms().items()}
            sync_ms["sync/exposed_wait_ms"] = sync_ms["sync/grad_barrier_ms"] + sync_ms["sync/param_barrier_ms"]
            self._fused.opt.timing = []
        return {**sync_ms, "loss": res.loss if res.batch_size else 0.0, "grad_norm": res.grad_norm_mean if res.batch_size else 0.0,
                "clip_rate": res.clip_rate if res.batch_size else 0.0, "batch_size": float(n),
                "noise_std": self.noise_multiplier * self._fused.sensitivity() / self.expected_batch,
                "clipping_norm": self._fused.sensitivity()}

    _preempted = False

    def _install_preemption_handler(self) -> None:
        """``enable_jit_checkpoint``: on SIGTERM finish the current step, save ``checkpoint-N`` and leave the loop."""
        if not self.args.enable_jit_checkpoint:
            return
        import signal
        import threading
        if threading.current_thread() is not threading.main_thread():
            return

        def on_term(signum, frame):
            self._preempted = True
        signal.signal(signal.SIGTERM, on_term)

    # ---- loop -------------------------------------------------------------------------------------
    def train(self, resume_from_checkpoint: str | bool | None = None, ignore_keys_for_eval=None):
        a = self.args
        resume = resume_from_checkpoint if resume_from_checkpoint is not None else a.resume_from_checkpoint
        if resume is True:
            ckpts = list_checkpoints(a.output_dir)
            resume = ckpts[-1] if ckpts else None
        self._setup(resume or None)
        self.model.train()
        if a.gradient_checkpointing:
            if hasattr(self.model, "gradient_checkpointing_enable") and not hasattr(self.model, "activation_checkpointing"):
                self.model.gradient_checkpointing_enable(**({"gradient_checkpointing_kwargs": a.gradient_checkpointing_kwargs}
                                                            if a.gradient_checkpointing_kwargs else {}))
            else:
                self.model.activation_checkpointing = True       # framework models: per-block torch.utils.checkpoint
        self._install_preemption_handler()
        self._call("on_train_begin")
        if a.eval_on_start and self.eval_dataset is not None:
            self.evaluate()
        t0 = time.perf_counter()
        tokens_at_start = self.state.num_input_tokens_seen
        window: list[dict[str, float]] = []
        for batch in self.get_train_dataloader():
            if a.activation_offloading:          # saved activations live in pinned host memory between forward and backward
                with torch.autograd.graph.save_on_cpu(pin_memory=torch.cuda.is_available()):
                    metrics = self.training_step(batch)
            else:
                metrics = self.training_step(batch)
            window.append(metrics)
            if self._preempted:                   # SIGTERM: write a just-in-time checkpoint between steps and stop
                if a.output_dir:
                    self._save_checkpoint(self.state.global_step)
                break
            step = self.state.global_step
            self.state.epoch = step * self.sample_rate
            if a.logging_strategy == "steps" and (step % a.logging_steps == 0 or (a.logging_first_step and step == 1)):
                self.log(self._mean(window))
                window = []
            if a.torch_empty_cache_steps and step % a.torch_empty_cache_steps == 0 and torch.cuda.is_available():
                torch.cuda.empty_cache()
            if a.eval_strategy == "steps" and a.eval_steps and step % a.eval_steps == 0 and self.eval_dataset is not None \
                    and self.state.epoch >= a.eval_delay:
                self.evaluate()
            if self.control.should_save or (a.save_strategy == "steps" and a.save_steps and step % a.save_steps == 0 and a.output_dir):
                self._save_checkpoint(step)
                self.control.should_save = False
            if a.privacy_target_epsilon is not None and a.privacy_noise_multiplier is not None and self.accountant.budget_exceeded():
                self.control.should_training_stop = True      # stop-at-epsilon for fixed-noise runs
            if self.control.should_training_stop or step >= self.state.max_steps:
                break
        if window:
            self.log(self._mean(window))
        self.state.epsilon = self.epsilon()
        runtime = time.perf_counter() - t0
        out = {"train_runtime": runtime, "global_step": self.state.global_step, "epsilon": self.state.epsilon,
               "train_samples_per_second": self.perf.state("train").samples_per_second}
        if a.include_tokens_per_second:
            out["train_tokens_per_second"] = (self.state.num_input_tokens_seen - tokens_at_start) / max(runtime, 1e-9)
        if a.include_num_input_tokens_seen:
            out["num_input_tokens_seen"] = self.state.num_input_tokens_seen
        step_losses = [r["loss"] for r in self.state.log_history if "loss" in r and "train_runtime" not in r]
        if step_losses:
            out["train_loss"] = float(np.mean(step_losses))       # mean of the logged (windowed) training losses
        out = TrainOutput(out)
        self.log(out)
        if a.load_best_model_at_end:
            self._load_best_model()
        self._call("on_train_end")
        if a.push_to_hub:
            self.push_to_hub(commit_message="End of training")
        return out

    def _load_best_model(self) -> None:
        """``load_best_model_at_end``: put the weights of the best evaluated checkpoint back into the model."""
        path = self.state.best_model_checkpoint
        if not path or not os.path.isdir(path):
            return
        from safetensors.torch import load_file
        for name in ("adapter_model.safetensors", FILES["weights"]):
            f = os.path.join(path, name)
            if os.path.exists(f):
                with torch.no_grad():
                    self.model.load_state_dict(load_file(f), strict=False)
        if self.engine_kind == "reference":           # later evaluations write the functional copy back into the model
            self._trainable = {n: p.detach().clone() for n, p in self.model.named_parameters() if p.requires_grad}

    @staticmethod
    def _mean(rows: list[dict[str, float]]) -> dict[str, float]:
        keys = rows[0].keys() if rows else []
        return {k: float(np.mean([r[k] for r in rows])) for k in keys}

    def epsilon(self, delta: float | None = None) -> float:
        return float(self.accountant.epsilon_at(self.target_delta if delta is None else delta))

    def log(self, logs: dict[str, float]) -> None:
        logs = {**logs, "step": self.state.global_step, "epoch": round(self.state.epoch, 4)}
        if self.accountant is not None and self.state.global_step and "epsilon" not in logs:
            logs["epsilon"] = self.epsilon()
        self.state.log_history.append(logs)
        self._call("on_log", logs=logs)

    # ---- evaluation ---------------------------------------------------------------------------------
    @torch.no_grad()
    def evaluation_loop(self, dataset: Any, description: str = "Evaluation", prediction_loss_only: bool | None = None,
                        metric_key_prefix: str = "eval") -> EvaluationResult:
        """One pass over ``dataset`` on THIS rank: per-example losses always, predictions / labels / inputs unless
        ``prediction_loss_only``.  Batches stay on the device and move to host memory every ``eval_accumulation_steps``
        batches; ``eval_do_concat_batches=False`` hands ``compute_metrics`` the per-batch list;
        ``include_for_metrics=["inputs", "loss"]`` adds ``inputs`` / ``losses`` to the :class:`EvalPrediction`.  The
        metrics here are this rank's (``{prefix}_loss`` = mean per-example loss); :meth:`evaluate` combines ranks."""
        a = self.args
        loss_only = a.prediction_loss_only if prediction_loss_only is None else prediction_loss_only
        want = set(a.include_for_metrics or [])
        acc_ = PredictionAccumulator(prediction_loss_only=loss_only, eval_accumulation_steps=a.eval_accumulation_steps,
                                     eval_do_concat_batches=a.eval_do_concat_batches, include_inputs="inputs" in want,
                                     include_losses="loss" in want)
        if self.engine_kind == "reference" if hasattr(self, "engine_kind") else False:
            self._write_back()
        was_training = self.model.training
        self.model.eval()
        bs = a.eval_batch_size
        tokens = 0
        for lo in range(0, len(dataset), bs):
            batch = self._to_device(self.data_collator([dataset[i] for i in range(lo, min(len(dataset), lo + bs))]))
            has_labels = "labels" in batch
            losses = self.compute_batch_per_example_loss(batch) if has_labels else None
            logits = None
            if not loss_only and "input_ids" in batch:       # pair batches (DPO) have no single sequence to predict for
                logits = self.model(batch["input_ids"])
                logits = getattr(logits, "logits", logits)
                if self.preprocess_logits_for_metrics is not None:
                    logits = self.preprocess_logits_for_metrics(logits, batch.get("labels"))
            acc_.add(losses, logits, batch.get("labels"), batch.get("input_ids"))
            tokens += int((batch["labels"] != -100).sum()) if has_labels else 0
        self.model.train(was_training)
        losses, preds, labels, inputs = acc_.finalize()
        metrics: dict[str, float] = {}
        if losses is not None and losses.numel():
            metrics[f"{metric_key_prefix}_loss"] = float(losses.mean())
        res = EvaluationResult(preds, labels, metrics, acc_.num_samples)
        res.losses, res.inputs, res.tokens = losses, inputs, tokens           # for evaluate / predict
        res.num_batches, res.offloads = acc_.num_batches, acc_.offloads
        return res

    def _metrics_from(self, res: EvaluationResult, prefix: str, gather: bool) -> dict[str, float]:
        """Run the user's ``compute_metrics`` on the collected predictions (gathered over ranks when the data was sharded)."""
        if self.compute_metrics is None or res.predictions is None or res.label_ids is None:
            return {}
        want = set(self.args.include_for_metrics or [])
        preds, labels, inputs, losses = res.predictions, res.label_ids, res.inputs, res.losses
        if gather and self.args.world_size > 1:
            if not self.args.eval_do_concat_batches:
                raise ValueError("eval_do_concat_batches=False with several ranks: per-batch lists are not gathered; "
                                 "call evaluation_loop on each rank instead")
            preds, labels = self._gather_padded(preds), self._gather_padded(labels)
            inputs = self._gather_padded(inputs) if inputs is not None else None
            losses = gather_tensors(losses.to(self.device)).cpu() if losses is not None else None
        out = self.compute_metrics(EvalPrediction(preds, labels, inputs if "inputs" in want else None,
                                                  losses if "loss" in want else None))
        return with_metric_prefix(to_python(dict(out)), prefix)

    def _gather_padded(self, t: torch.Tensor) -> torch.Tensor:
        """``gather_tensors`` for predictions whose trailing sizes differ between ranks (padded with -100 to the largest)."""
        if not isinstance(t, torch.Tensor):
            raise ValueError("only tensor predictions are gathered over ranks")
        tail = [int(reduce_scalar(int(t.shape[d]), "max")) for d in range(1, t.ndim)]
        if list(t.shape[1:]) != tail:
            wide = t.new_full((t.shape[0], *tail), -100)
            wide[(slice(None),) + tuple(slice(0, n) for n in t.shape[1:])] = t
            t = wide
        return gather_tensors(t.to(self.device)).cpu()

    @torch.no_grad()
    def evaluate(self, eval_dataset: Any = None, ignore_keys=None, metric_key_prefix: str = "eval") -> dict[str, float]:
        data = eval_dataset if eval_dataset is not None else self.eval_dataset
        if data is None:
            raise ValueError("evaluation needs an eval_dataset")
        a = self.args
        start = time.time()
        shard = local_shard(data, rank=a.process_index, world_size=a.world_size)
        # nobody consumes predictions without compute_metrics: keep only the losses then (no logits pass, no host copies)
        res = self.evaluation_loop(shard, "Evaluation", prediction_loss_only=True if self.compute_metrics is None else None,
                                   metric_key_prefix=metric_key_prefix)
        total = float(reduce_scalar(float(res.losses.sum()) if res.losses is not None else 0.0, "sum"))
        count = int(reduce_scalar(int(res.losses.numel()) if res.losses is not None else 0, "sum"))
        tokens = int(reduce_scalar(res.tokens, "sum"))
        metrics = {f"{metric_key_prefix}_loss": total / max(count, 1), f"{metric_key_prefix}_samples": float(count)}
        metrics.update(self._metrics_from(res, metric_key_prefix, gather=True))
        metrics.update(speed_metrics(metric_key_prefix, start, num_samples=count, num_steps=res.num_batches, num_tokens=tokens or None))
        if self.accountant is not None and self.state.global_step:
            metrics["epsilon"] = self.epsilon()
        self.log(metrics)
        self._call("on_evaluate", metrics=metrics)
        return metrics

    @torch.no_grad()
    def predict(self, test_dataset: Any, ignore_keys=None, metric_key_prefix: str = "test") -> PredictionOutput:
        start = time.time()
        res = self.evaluation_loop(test_dataset, "Prediction", metric_key_prefix=metric_key_prefix)
        metrics = dict(res.metrics)
        metrics.update(self._metrics_from(res, metric_key_prefix, gather=False))
        metrics.update(speed_metrics(metric_key_prefix, start, num_samples=res.num_samples, num_steps=res.num_batches))
        for cb in self.callbacks:
            if hasattr(cb, "on_predict"):
                cb.on_predict(self.args, self.state, self.control, metrics=metrics, model=self.model)
        return EvaluationResult(res.predictions, res.label_ids, metrics, res.num_samples)

    # ---- checkpoints ----------------------------------------------------------------------------------
    def save_model(self, output_dir: str | None = None) -> None:
        out = output_dir or self.args.output_dir
        if not out:
            raise ValueError("no output_dir")
        if getattr(self, "engine_kind", None) == "reference":
            self._write_back()
        if self.args.should_save:
            os.makedirs(out, exist_ok=True)
            sd = {k: v.detach().to("cpu").contiguous().clone() for k, v in self.model.state_dict().items()}
            only_adapter = any("lora_" in k for k in sd) and not any(p.requires_grad for n, p in self.model.named_parameters() if "lora_" not in n)
            if only_adapter:
                sd = {k: v for k, v in sd.items() if "lora_" in k}
            name = "adapter_model.safetensors" if only_adapter else FILES["weights"]
            if self.args.save_safetensors:
                from safetensors.torch import save_file
                seen: dict[int, str] = {}
                uniq = {}
                for k, v in sd.items():            # tied weights: keep one copy
                    ptr = self.model.state_dict()[k].data_ptr()
                    if ptr in seen:
                        continue
                    seen[ptr] = k
                    uniq[k] = v
                save_file(uniq, os.path.join(out, name), metadata={"format": "pt"})
            else:
                torch.save(sd, os.path.join(out, name.replace(".safetensors", ".bin")))
            cfg = getattr(self.model, "config", None)
            if cfg is not None and dataclasses.is_dataclass(cfg):
                json.dump(dataclasses.asdict(cfg), open(os.path.join(out, "config.json"), "w"), indent=1)

    def _runtime(self) -> RuntimeCheckpoint:
        a = self.args
        ref = self.engine_kind == "reference"
        ms, mp = self._participation(self.sampler, self.state.max_steps)
        if ref:
            clip_sd, noise_sd = state_dict(self._clip_state), state_dict(_noise_public(self._noise_state))
        else:
            # fused engine: the noise stream is (key, optimizer step), both in dp_optimizer.pt; the adaptive clipping state
            # (bounds, step counter of ITS noise stream, last counts) lives in the engine and is saved here
            ad = self._fused.adaptive
            clip_sd = {"adaptive": state_dict(ad), "clipping_norm": self._fused.clipping_norm} if ad is not None else {}
            noise_sd = {}
        per_epoch = max(1, round(1.0 / self.sample_rate)) if self.sample_rate else 1
        return RuntimeCheckpoint(
            version=DP_STATE_BUNDLE_VERSION, clip_state=clip_sd, noise_state=noise_sd, sampler_state=state_dict(self.sampler),
            sample_rate=self.sample_rate, target_delta=self.target_delta, noise_multiplier=self.noise_multiplier,
            expected_steps_per_epoch=per_epoch, expected_batch_size=self.expected_batch, total_steps=self.state.max_steps,
            mechanism_kind=a.privacy_noise_mechanism, mf_n_steps=self.state.max_steps if self._strategy else None,
            mf_min_sep=ms, mf_max_participations=mp, lr_scheduler=a.lr_scheduler, learning_rate=float(a.learning_rate),
            warmup_steps=float(a.warmup_steps), lr_scheduler_kwargs=dict(a.lr_scheduler_kwargs),
            extras={"mechanism_kwargs": dict(a.privacy_noise_mechanism_kwargs), "sampling_mode": a.sampling_mode,
                    "clipping_norm": a.clipping_norm, "clipping_mode": a.clipping_mode, "engine": self.engine_kind})

    def _save_checkpoint(self, step: int) -> str:
        a = self.args
        final = os.path.join(a.output_dir, f"checkpoint-{step}")
        tmp = final + ".tmp"
        if a.should_save:
            shutil.rmtree(tmp, ignore_errors=True)
            os.makedirs(tmp, exist_ok=True)
        _barrier()
        self.save_model(tmp)
        opt_sd = self._fused.opt.state_dict() if self.engine_kind == "fused" else state_dict(self._opt_state)
        if a.should_save and not a.save_only_model:
            torch.save(opt_sd, os.path.join(tmp, FILES["optimizer"]))
            if self.engine_kind == "reference" and self._strategy is not None:
                torch.save(state_dict(self._noise_state._inner_state), os.path.join(tmp, "dp_noise_buffers.pt"))
            save_runtime_checkpoint(self._runtime(), os.path.join(tmp, FILES["state"]))
            with open(os.path.join(tmp, FILES["accountant"]), "w") as f:
                f.write(self.accountant.to_json())
            with open(os.path.join(tmp, FILES["trainer_state"]), "w") as f:
                f.write(self.state.to_json())
            torch.save(a.to_dict(), os.path.join(tmp, FILES["args"]))
        _barrier()
        rng = {"python": random.getstate(), "numpy": np.random.get_state(), "torch": torch.get_rng_state(),
               "cuda": torch.cuda.get_rng_state_all() if torch.cuda.is_available() else None}
        if os.path.isdir(tmp):
            # Hugging Face naming: one `rng_state.pth` for a single process, `rng_state_{rank}.pth` with several
            torch.save(rng, os.path.join(tmp, "rng_state.pth" if a.world_size == 1 else f"rng_state_{a.process_index}.pth"))
        _barrier()
        if a.should_save:
            shutil.rmtree(final, ignore_errors=True)
            os.replace(tmp, final)
            rotate_checkpoints(a.output_dir, a.save_total_limit, keep=final)
        _barrier()
        self._call("on_save")
        return final

    def _load_checkpoint_meta(self, path: str):
        runtime = load_runtime_checkpoint(os.path.join(path, FILES["state"]))
        a = self.args
        ex = runtime.extras
        drift = {"privacy_noise_mechanism": (runtime.mechanism, a.privacy_noise_mechanism),
                 "max_steps": (runtime.max_steps, self.state.max_steps),
                 "expected_batch_size": (float(runtime.expected_batch_size), float(a.train_batch_size))}
        for key, now in (("sampling_mode", a.sampling_mode), ("clipping_norm", a.clipping_norm), ("clipping_mode", a.clipping_mode)):
            if key in ex:                       # a bundle written by the reference carries no such entry: nothing to compare
                drift[key] = (ex[key], now)
        bad = {k: v for k, v in drift.items() if v[0] != v[1]}
        if bad:
            raise ValueError(f"refusing to resume: DP-relevant arguments changed since the checkpoint was written: {bad}")
        saved = acc.Accountant.from_state_dict(json.load(open(os.path.join(path, FILES["accountant"]))))
        return runtime, saved.process

    def _load_checkpoint_state(self, path: str, runtime: RuntimeCheckpoint) -> None:
        from safetensors.torch import load_file
        for name in ("adapter_model.safetensors", FILES["weights"]):
            f = os.path.join(path, name)
            if os.path.exists(f):
                self.model.load_state_dict(load_file(f), strict=False)
        opt_sd = torch.load(os.path.join(path, FILES["optimizer"]), weights_only=False)
        if self.engine_kind == "fused":
            self._fused.opt.load_state_dict(opt_sd)
            if self._fused.adaptive is not None and runtime.clip_state.get("adaptive") is not None:
                # bounds and the step counter of the adaptive mechanism's own noise stream: without them a resumed run
                # would restart from the initial bound and draw the same Gaussians for new clipped-count releases
                self._fused.adaptive = from_state_dict(self._fused.adaptive, runtime.clip_state["adaptive"])
                self._fused.clipping_norm = runtime.clip_state["clipping_norm"]
        else:
            self._trainable = {n: p.detach().clone() for n, p in self.model.named_parameters() if p.requires_grad}
            self._opt_state = from_state_dict(self._optimizer.init(self._trainable), opt_sd)
            self._clip_state = from_state_dict(self._clip_state, runtime.clip_state)
            pub = from_state_dict(_noise_public(self._noise_state), runtime.noise_state)
            self._noise_state = dataclasses.replace(self._noise_state, _step_counter=pub["step"])
            if self._strategy is not None:
                inner = torch.load(os.path.join(path, "dp_noise_buffers.pt"), weights_only=False)
                self._noise_state = dataclasses.replace(self._noise_state, _inner_state=from_state_dict(self._noise_state._inner_state, inner),
                                                        _first_max_norm=pub.get("first_max_norm"))
        self.sampler = from_state_dict(self.sampler, runtime.sampler_state)
        st = json.load(open(os.path.join(path, FILES["trainer_state"])))
        self.state = DPTrainerState(**{k: v for k, v in st.items() if k in {f.name for f in dataclasses.fields(DPTrainerState)}})
        rng_file = os.path.join(path, f"rng_state_{self.args.process_index}.pth")
        if not os.path.exists(rng_file):
            rng_file = os.path.join(path, "rng_state.pth")
        if os.path.exists(rng_file):
            rng = torch.load(rng_file, weights_only=False)
            random.setstate(rng["python"])
            np.random.set_state(rng["numpy"])
            torch.set_rng_state(rng["torch"])


class _Trimmed:
    def __init__(self, data, n):
        self.data, self.n = data, n

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        if isinstance(i, slice):
            return _Slice(self.data, *i.indices(self.n))
        return self.data[i]


class _Slice:
    def __init__(self, data, lo, hi, step):
        self.data, self.lo, self.hi = data, lo, hi

    def __len__(self):
        return self.hi - self.lo

    def __getitem__(self, i):
        return self.data[self.lo + i]


@dataclasses.dataclass(frozen=True)
class _EpochProcess(acc.core.DpHorizonProcess):
    """Whole-epoch process charged per step: ``n`` steps cost ``ceil(n / steps_per_epoch)`` epochs."""
    epoch: acc.DpProcess
    steps_per_epoch: int

    def pld_at(self, n_steps, config=None):
        return self.epoch.repeated_pld(max(1, math.ceil(n_steps / self.steps_per_epoch)), config)

    def _build_pld(self, config):
        return self.pld_at(1, config)


def _noise_public(state) -> dict[str, Any]:
    return {"step": state._step_counter, "seed": str(state._rng_key.seed), "first_max_norm": getattr(state, "_first_max_norm", None)}


def _barrier() -> None:
    if is_distributed():
        dist.barrier()


__all__ = ["BestModelSaveCallback", "DPTrainer", "DPTrainerState", "DP_STATE_BUNDLE_VERSION", "EvalPrediction", "EvaluationResult", "TrainOutput",
           "PredictionAccumulator", "PredictionOutput",
           "PrinterCallback", "RuntimeCheckpoint", "TrainerCallback", "TrainerControl", "build_lr_schedule",
           "build_optimizer", "build_strategy", "default_per_example_loss", "list_checkpoints", "rotate_checkpoints"]

from ..utils.namespaces import submodule as _sub  # noqa: E402

_sub(__name__, "types", "Return types of the trainers.", {"EvalPrediction": EvalPrediction, "EvaluationResult": EvaluationResult,
                                                           "PredictionOutput": PredictionOutput, "TrainOutput": TrainOutput})

