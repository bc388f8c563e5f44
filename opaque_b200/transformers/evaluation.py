"""Evaluation containers and helpers of the trainers.

* :class:`EvaluationResult` — what ``evaluate`` / ``predict`` / ``evaluation_loop`` return (``predictions``, ``label_ids``,
  ``metrics``, ``num_samples``); ``PredictionOutput`` is the same class under its Hugging Face name.
* :class:`EvalPrediction` — the argument of a user's ``compute_metrics``; unpacks as ``(predictions, label_ids)`` and also
  carries ``inputs`` / ``losses`` when ``include_for_metrics`` asks for them.
* :class:`PredictionAccumulator` — collects per-batch losses, predictions, labels and inputs during an evaluation loop.
  Batches are kept on the device they arrive on and moved to host memory every ``eval_accumulation_steps`` batches as ONE
  concatenated chunk (each value crosses the bus once; chunks already on the host are not touched again), so a long
  evaluation of a large-vocabulary model does not pile its logits up in device memory.  ``finalize`` returns one tensor
  per stream (ragged sequence lengths padded with −100, the value metric functions mask) or, with
  ``eval_do_concat_batches=False``, the list of per-batch tensors.
* :func:`speed_metrics`, :func:`with_metric_prefix` — the ``{prefix}_runtime`` / ``_samples_per_second`` /
  ``_steps_per_second`` entries and the key prefixing that Hugging Face reports use.

Parity: packages/opaque-transformers/src/opaque/api/transformers/trainer/_eval.py (accumulator with hot / cold buffers,
speed metrics, prefixing) and trainer/types.py (``EvaluationResult``).
"""
from __future__ import annotations

import dataclasses
import time
from typing import Any, Iterator

import torch

PAD_VALUE = -100          # what ragged predictions / labels / inputs are padded with: metric code masks this value


@dataclasses.dataclass
class EvaluationResult:
    predictions: Any
    label_ids: Any
    metrics: dict[str, float]
    num_samples: int = 0


PredictionOutput = EvaluationResult


class TrainOutput(dict):
    """What ``train()`` returns: the dict of final metrics (``out["global_step"]``, ``out["epsilon"]``, …) that ALSO has
    the Hugging Face attributes ``global_step``, ``training_loss`` and ``metrics``."""

    @property
    def global_step(self) -> int:
        return int(self.get("global_step", 0))

    @property
    def training_loss(self) -> float:
        return float(self.get("train_loss", float("nan")))

    @property
    def metrics(self) -> dict:
        return dict(self)


class EvalPrediction:
    """Argument of ``compute_metrics``: ``predictions, label_ids = eval_pred`` works, and so do the attributes."""

    def __init__(self, predictions: Any, label_ids: Any, inputs: Any = None, losses: Any = None):
        self.predictions, self.label_ids, self.inputs, self.losses = predictions, label_ids, inputs, losses
        self._fields = (predictions, label_ids) + ((inputs,) if inputs is not None else ()) + ((losses,) if losses is not None else ())

    def __iter__(self) -> Iterator[Any]:
        return iter(self._fields)

    def __getitem__(self, i: int) -> Any:
        return self._fields[i]

    def __len__(self) -> int:
        return len(self._fields)


def _map_nested(fn, value: Any) -> Any:
    if isinstance(value, torch.Tensor):
        return fn(value)
    if isinstance(value, (list, tuple)):
        return type(value)(_map_nested(fn, v) for v in value)
    if isinstance(value, dict):
        return {k: _map_nested(fn, v) for k, v in value.items()}
    return value


def _cat_padded(chunks: list[torch.Tensor]) -> torch.Tensor:
    """Concatenate along dim 0; trailing dimensions that differ (sequence lengths) are padded to the longest with −100."""
    if len(chunks) == 1:
        return chunks[0]
    if any(c.ndim != chunks[0].ndim for c in chunks):
        raise ValueError("evaluation batches of different rank cannot be concatenated: set eval_do_concat_batches=False")
    if all(c.shape[1:] == chunks[0].shape[1:] for c in chunks):
        return torch.cat(chunks)
    tail = [max(c.shape[d] for c in chunks) for d in range(1, chunks[0].ndim)]
    out = chunks[0].new_full((sum(c.shape[0] for c in chunks), *tail), PAD_VALUE)
    row = 0
    for c in chunks:
        out[(slice(row, row + c.shape[0]),) + tuple(slice(0, s) for s in c.shape[1:])] = c
        row += c.shape[0]
    return out


def _cat_nested(chunks: list[Any]) -> Any:
    first = chunks[0]
    if isinstance(first, torch.Tensor):
        return _cat_padded(chunks)
    if isinstance(first, (list, tuple)):
        return type(first)(_cat_nested([c[i] for c in chunks]) for i in range(len(first)))
    if isinstance(first, dict):
        return {k: _cat_nested([c[k] for c in chunks]) for k in first}
    return first


class _Stream:
    """One collected quantity: batches waiting on the device, and chunks already on the host."""

    def __init__(self) -> None:
        self.pending: list[Any] = []
        self.host: list[Any] = []

    def add(self, value: Any) -> None:
        self.pending.append(_map_nested(lambda t: t.detach(), value))

    def offload(self, concat: bool) -> None:
        if not self.pending:
            return
        if concat:
            self.host.append(_map_nested(lambda t: t.cpu(), _cat_nested(self.pending)))
        else:
            self.host.extend(_map_nested(lambda t: t.cpu(), v) for v in self.pending)
        self.pending = []

    def result(self, concat: bool) -> Any:
        self.offload(concat)
        if not self.host:
            return None
        return _cat_nested(self.host) if concat else list(self.host)


class PredictionAccumulator:
    """See the module docstring.  ``add`` once per batch, ``finalize`` once at the end."""

    def __init__(self, *, prediction_loss_only: bool = False, eval_accumulation_steps: int | None = None,
                 eval_do_concat_batches: bool = True, include_inputs: bool = False, include_losses: bool = False):
        if eval_accumulation_steps is not None and eval_accumulation_steps < 1:
            raise ValueError("eval_accumulation_steps must be a positive number of batches (or None: offload at the end)")
        self.prediction_loss_only = prediction_loss_only
        self.every = eval_accumulation_steps
        self.concat = eval_do_concat_batches
        self.include_inputs, self.include_losses = include_inputs, include_losses
        self.losses, self.logits, self.labels, self.inputs = _Stream(), _Stream(), _Stream(), _Stream()
        self.num_batches = 0
        self.num_samples = 0
        self.offloads = 0

    def add(self, losses: torch.Tensor | None, logits: Any = None, labels: Any = None, inputs: Any = None) -> None:
        """``losses``: one value per example of the batch (a scalar is repeated by the batch size, so a mean-reduced loss
        still weighs every example once)."""
        n = None
        for v in (labels, inputs, logits):
            if isinstance(v, torch.Tensor):
                n = int(v.shape[0])
                break
        if losses is not None:
            if losses.ndim == 0:
                losses = losses.repeat(n or 1)
            n = int(losses.shape[0]) if n is None else n
            self.losses.add(losses.float())
        if not self.prediction_loss_only:
            if logits is not None:
                self.logits.add(logits)
            if labels is not None:
                self.labels.add(labels)
            if inputs is not None and self.include_inputs:
                self.inputs.add(inputs)
        self.num_batches += 1
        self.num_samples += n or 0
        if self.every is not None and self.num_batches % self.every == 0:
            self.offload()

    def offload(self) -> None:
        """Move what is waiting on the device to host memory (one concatenated chunk per stream)."""
        for s in (self.losses, self.logits, self.labels, self.inputs):
            s.offload(self.concat)
        self.offloads += 1

    def finalize(self) -> tuple[torch.Tensor | None, Any, Any, Any]:
        """``(per-example losses, predictions, label_ids, inputs)``; the last three are ``None`` when not collected."""
        losses = self.losses.result(True)
        if self.prediction_loss_only:
            return losses, None, None, None
        return losses, self.logits.result(self.concat), self.labels.result(self.concat), self.inputs.result(self.concat)

    def eval_prediction(self) -> EvalPrediction:
        losses, preds, labels, inputs = self.finalize()
        return EvalPrediction(preds, labels, inputs if self.include_inputs else None, losses if self.include_losses else None)


def speed_metrics(prefix: str, start_time: float, num_samples: int | None = None, num_steps: int | None = None,
                  num_tokens: int | None = None) -> dict[str, float]:
    """``{prefix}_runtime`` in seconds (from ``time.time()`` at ``start_time``) and the rates that follow from it."""
    runtime = time.time() - start_time
    out = {f"{prefix}_runtime": round(runtime, 4)}
    if runtime <= 0:
        return out
    if num_samples is not None:
        out[f"{prefix}_samples_per_second"] = round(num_samples / runtime, 3)
    if num_steps is not None:
        out[f"{prefix}_steps_per_second"] = round(num_steps / runtime, 3)
    if num_tokens is not None:
        out[f"{prefix}_tokens_per_second"] = round(num_tokens / runtime, 3)
    return out


def with_metric_prefix(metrics: dict[str, Any], prefix: str) -> dict[str, Any]:
    """Keys that do not start with ``{prefix}_`` get it; ``epsilon`` (a property of the run, not of a split) keeps its name."""
    out = {}
    for k, v in metrics.items():
        out[k if k.startswith(prefix + "_") or k == "epsilon" else f"{prefix}_{k}"] = v
    return out


def to_python(value: Any) -> Any:
    """Tensors and numpy scalars inside a metrics dict become plain Python numbers / lists (JSON-ready)."""
    if isinstance(value, torch.Tensor):
        return value.item() if value.numel() == 1 else value.tolist()
    if hasattr(value, "item") and getattr(value, "size", 2) == 1:
        return value.item()
    if isinstance(value, dict):
        return {k: to_python(v) for k, v in value.items()}
    if isinstance(value, (list, tuple)):
        return type(value)(to_python(v) for v in value)
    return value


__all__ = ["EvalPrediction", "EvaluationResult", "PAD_VALUE", "PredictionAccumulator", "PredictionOutput", "TrainOutput", "speed_metrics",
           "to_python", "with_metric_prefix"]
