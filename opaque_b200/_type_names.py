"""Type names that the reference exposes through its ``types`` modules and that have no class of their own here: typed
dictionaries for collator inputs / outputs, protocols for the ``(fn, state)`` factories, and aliases where one class of
this package plays several of the reference's roles.

Parity: packages/opaque-alignment/src/opaque/api/alignment/{sft,dpo}/collator/types.py,
packages/opaque-engine/src/opaque/api/engine/clipping/_types.py, packages/opaque-dpsgd/src/opaque/api/dpsgd/noise/_types.py.
"""
from __future__ import annotations

from typing import Any, Protocol, TypedDict

import torch

from .engine.clipping import ClippedFunAux, ClippedGradAux
from .types import ClippedPytree, ClipState, NoisedPytree, NoiseState, SecondMomentClippingOutput, SecondMomentNoiseOutput


class LMExample(TypedDict, total=False):
    """One language-modelling row before collation."""
    input_ids: list[int]
    completion_mask: list[int]
    assistant_masks: list[int]


class LMBatch(TypedDict, total=False):
    """What ``language_modeling_collator`` returns: right-padded ids, aligned labels (−100 = not scored), attention mask."""
    input_ids: torch.Tensor
    labels: torch.Tensor
    attention_mask: torch.Tensor


class PreferenceExample(TypedDict, total=False):
    """One preference pair before collation (token ids)."""
    prompt_input_ids: list[int]
    chosen_input_ids: list[int]
    rejected_input_ids: list[int]
    ref_chosen_logps: float
    ref_rejected_logps: float


class PreferenceBatch(TypedDict, total=False):
    """What ``preference_collator`` returns: prompt + response sequences of both sides, labels scored on the response only."""
    chosen_input_ids: torch.Tensor
    chosen_labels: torch.Tensor
    chosen_attention_mask: torch.Tensor
    rejected_input_ids: torch.Tensor
    rejected_labels: torch.Tensor
    rejected_attention_mask: torch.Tensor
    ref_chosen_logps: torch.Tensor
    ref_rejected_logps: torch.Tensor


# one aux class serves the fixed, automatic and adaptive clipping modes (the mode-specific values live in the clip state)
AutoClippedFunAux = ClippedFunAux
AutoClippedGradAux = ClippedGradAux
AdaptiveClippedGradAux = ClippedGradAux
ClippedGradResult = tuple        # (ClippedPytree | (ClippedPytree, aux), ClipState)


class ClippedGradFn(Protocol):
    """``grad_fn(*args, state=clip_state) -> (ClippedPytree | (ClippedPytree, aux), ClipState)``: what ``clipped_grad`` returns."""

    def __call__(self, *args: Any, state: ClipState, **kwargs: Any) -> tuple[Any, ClipState]: ...


GaussianNoiseInput = ClippedPytree | SecondMomentClippingOutput
GaussianNoiseOutput = NoisedPytree | SecondMomentNoiseOutput


class GaussianNoiseFn(Protocol):
    """``noise_fn(clipped, state) -> (noised, state)``: what ``gaussian_noise`` returns."""

    def __call__(self, clipped: Any, state: NoiseState) -> tuple[Any, NoiseState]: ...


__all__ = ["AdaptiveClippedGradAux", "AutoClippedFunAux", "AutoClippedGradAux", "ClippedGradFn", "ClippedGradResult", "GaussianNoiseFn",
           "GaussianNoiseInput", "GaussianNoiseOutput", "LMBatch", "LMExample", "PreferenceBatch", "PreferenceExample"]
