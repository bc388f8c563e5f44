"""Alignment task library: SFT / DPO losses, log-probabilities, collators, metrics.

Parity: packages/opaque-alignment/src/opaque/alignment/__init__.py (namespaces ``data, dpo, metric, sft``).
"""
from . import data, dpo, sft
from . import sft as metric

__all__ = ["data", "dpo", "metric", "sft"]
