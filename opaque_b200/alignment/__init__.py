"""Alignment task library: SFT / DPO losses, log-probabilities, collators, metrics.

Parity: packages/opaque-alignment/src/opaque/alignment/__init__.py (namespaces ``data, dpo, metric, sft``).
"""
from . import chat_template, data, dpo, metric, reference, sft, unshifted
from .. import __version__
from ..utils.namespaces import submodule as _sub

# the reference's deeper import paths (opaque.alignment.dpo.loss, ...): same objects under the same dotted names
_LOSS = ("sigmoid_loss hinge_loss robust_loss ipo_loss discopop_loss chosen_nll_loss apo_zero_loss apo_down_loss exo_loss nca_loss "
         "bco_loss sppo_loss simpo_loss odds_ratio_loss f_divergence_remap f_divergence_logits mpo_combine wpo_weights ld_dpo_split "
         "orpo_loss dpo_loss wpo_weight ld_dpo_logp").split()
_sub(dpo.__name__, "loss", "Preference loss heads and their building blocks.",
     {**{n: getattr(dpo, n) for n in _LOSS}, "sequence_logp": dpo.completion_logp, "fused_sequence_logp": dpo.fused_completion_logp})
_sub(dpo.__name__, "collator", "Preference-pair collation (factory form, the reference's batch layout).",
     {"preference_collator": unshifted.preference_collator})
_sub(dpo.__name__, "data", "Preference dataset helpers.", {"extract_prompt": dpo.extract_prompt})
_sub(dpo.__name__, "metric", "Reward telemetry.", {"reward_metrics": dpo.reward_metrics, "reward_margins": dpo.reward_margins})
_sub(dpo.__name__, "reference", "Reference-policy helpers.", {n: getattr(reference, n) for n in reference.__all__})
_sub(sft.__name__, "collator", "Language-modelling collation (factory form, unshifted labels).",
     {"language_modeling_collator": unshifted.language_modeling_collator})
_sub(sft.__name__, "loss", "SFT losses with the causal shift inside (labels as the factory collator emits them).",
     {n: getattr(unshifted, n) for n in ("dft_loss", "fused_dft_loss", "fused_nll_loss", "nll_loss")})
from .. import _type_names as _T  # noqa: E402
_sub(dpo.__name__ + ".collator", "types", "Row and batch types of the preference collator.",
     {"PreferenceBatch": _T.PreferenceBatch, "PreferenceExample": _T.PreferenceExample}, bind=False)  # alignment.dpo.collator.types
_sub(sft.__name__ + ".collator", "types", "Row and batch types of the language-modelling collator.",
     {"LMBatch": _T.LMBatch, "LMExample": _T.LMExample}, bind=False)
metric.token_accuracy = sft.token_accuracy          # the name this namespace had before it became a module of its own

__all__ = ["chat_template", "data", "dpo", "metric", "reference", "sft", "unshifted", "__version__"]
