"""Trainers: ``DPTrainer``, ``TrainingArguments`` and the TRL-shaped ``trl.SFTTrainer`` / ``trl.DPOTrainer``.

Parity: packages/opaque-transformers/src/opaque/transformers/__init__.py.
"""
from . import evaluation, trl
from .evaluation import EvalPrediction, EvaluationResult
from .trainer import DPTrainer, DPTrainerState, TrainerCallback
from .. import __version__  # noqa: F401
from .training_args import TrainingArguments

__all__ = ["DPTrainer", "DPTrainerState", "EvalPrediction", "EvaluationResult", "TrainerCallback", "TrainingArguments", "evaluation", "trl"]
