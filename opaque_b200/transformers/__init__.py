"""Trainers: ``DPTrainer``, ``TrainingArguments`` and the TRL-shaped ``trl.SFTTrainer`` / ``trl.DPOTrainer``.

Parity: packages/opaque-transformers/src/opaque/transformers/__init__.py.
"""
from . import trl
from .trainer import DPTrainer, DPTrainerState, TrainerCallback
from .training_args import TrainingArguments

__all__ = ["DPTrainer", "DPTrainerState", "TrainerCallback", "TrainingArguments", "trl"]
