"""Alignment task library: SFT / DPO losses, log-probabilities, collators, metrics.

Parity: packages/opaque-alignment/src/opaque/alignment/__init__.py (namespaces ``data, dpo, metric, sft``).
"""
from . import chat_template, data, dpo, sft
from . import sft as metric

__all__ = ["chat_template", "data", "dpo", "metric", "sft"]
