"""Model adaptation entry points (API of ``opaque.patches``).

The reference monkey-patches Hugging Face modeling code so it survives ``vmap(grad)`` and swaps module forwards
for Triton kernels.  This framework owns its model families (``opaque_b200.models``), so "patching" means
*converting*: ``apply_model_patches(model)`` takes a Hugging Face model (or config) of a supported family and
returns the equivalent framework model with weights copied, which already runs on the sm_100a kernels and needs no
vmap work-arounds (the fused engine is explicit-batch).  A model that is already a framework model is returned
unchanged.  ``apply_runtime_patches`` is kept for API compatibility and reports what is (not) needed.

Parity: packages/opaque-patches/src/opaque/api/patches/__init__.py:20-160, transformers/_factory.py, _registry.py,
_router.py, peft/_router.py.
"""
from __future__ import annotations

from collections.abc import Callable
from typing import Any

import torch

from . import kernels
from ..models import GPT2Config, GPT2LMHeadModel, LlamaConfig, LlamaForCausalLM, MoEConfig, MoEForCausalLM

_FAMILIES: dict[str, Callable[[Any, dict], torch.nn.Module]] = {}
_RUNTIME = {"patched": False}

# model_type -> family builder; llama-shaped families share one implementation
LLAMA_LIKE = ("llama", "mistral", "ministral", "qwen2", "qwen3", "mellum", "smollm3", "granite", "olmo2", "olmo3",
              "exaone4", "phi3", "glm4", "cohere", "cohere2", "gemma", "gemma2", "gemma3")
MOE_LIKE = ("mixtral", "qwen2_moe", "qwen3_moe", "qwen3_5_moe", "qwen3_next", "gpt_oss", "hunyuan_v1_moe", "deepseek_v4")


def register_family(model_type: str, builder: Callable[[Any, dict], torch.nn.Module]) -> None:
    """Register ``builder(hf_config, options) -> nn.Module`` for a Hugging Face ``model_type``."""
    _FAMILIES[model_type] = builder


def _cfg_get(cfg: Any, name: str, default=None):
    return cfg.get(name, default) if isinstance(cfg, dict) else getattr(cfg, name, default)


def _build_llama(cfg: Any, opt: dict) -> torch.nn.Module:
    c = LlamaConfig(vocab_size=_cfg_get(cfg, "vocab_size"), hidden_size=_cfg_get(cfg, "hidden_size"),
                    intermediate_size=_cfg_get(cfg, "intermediate_size"), num_hidden_layers=_cfg_get(cfg, "num_hidden_layers"),
                    num_attention_heads=_cfg_get(cfg, "num_attention_heads"),
                    num_key_value_heads=_cfg_get(cfg, "num_key_value_heads") or _cfg_get(cfg, "num_attention_heads"),
                    rms_norm_eps=_cfg_get(cfg, "rms_norm_eps", 1e-6), rope_theta=_cfg_get(cfg, "rope_theta", 10000.0),
                    max_position_embeddings=_cfg_get(cfg, "max_position_embeddings", 8192),
                    tie_word_embeddings=bool(_cfg_get(cfg, "tie_word_embeddings", False)), head_dim=_cfg_get(cfg, "head_dim"))
    return LlamaForCausalLM(c, dtype=opt.get("dtype", torch.bfloat16), device=opt.get("device"))


def _build_gpt2(cfg: Any, opt: dict) -> torch.nn.Module:
    c = GPT2Config(vocab_size=_cfg_get(cfg, "vocab_size"), n_positions=_cfg_get(cfg, "n_positions", 1024),
                   n_embd=_cfg_get(cfg, "n_embd"), n_layer=_cfg_get(cfg, "n_layer"), n_head=_cfg_get(cfg, "n_head"),
                   layer_norm_epsilon=_cfg_get(cfg, "layer_norm_epsilon", 1e-5))
    return GPT2LMHeadModel(c, dtype=opt.get("dtype", torch.bfloat16), device=opt.get("device"))


def _build_moe(cfg: Any, opt: dict) -> torch.nn.Module:
    c = MoEConfig(vocab_size=_cfg_get(cfg, "vocab_size"), hidden_size=_cfg_get(cfg, "hidden_size"),
                  num_hidden_layers=_cfg_get(cfg, "num_hidden_layers"), num_attention_heads=_cfg_get(cfg, "num_attention_heads"),
                  num_key_value_heads=_cfg_get(cfg, "num_key_value_heads") or _cfg_get(cfg, "num_attention_heads"),
                  num_experts=_cfg_get(cfg, "num_experts") or _cfg_get(cfg, "num_local_experts"),
                  moe_intermediate_size=_cfg_get(cfg, "moe_intermediate_size") or _cfg_get(cfg, "intermediate_size"),
                  num_shared_experts=int(_cfg_get(cfg, "num_shared_experts", 0) or (1 if _cfg_get(cfg, "shared_expert_intermediate_size") else 0)),
                  num_experts_per_tok=_cfg_get(cfg, "num_experts_per_tok", 2), norm_topk_prob=bool(_cfg_get(cfg, "norm_topk_prob", False)),
                  rms_norm_eps=_cfg_get(cfg, "rms_norm_eps", 1e-6), rope_theta=_cfg_get(cfg, "rope_theta", 1e6),
                  max_position_embeddings=_cfg_get(cfg, "max_position_embeddings", 4096))
    return MoEForCausalLM(c, dtype=opt.get("dtype", torch.bfloat16), device=opt.get("device"))


for _t in LLAMA_LIKE:
    register_family(_t, _build_llama)
for _t in MOE_LIKE:
    register_family(_t, _build_moe)
register_family("gpt2", _build_gpt2)


def supported_families() -> list[str]:
    return sorted(_FAMILIES)


def _is_framework_model(model: Any) -> bool:
    return isinstance(model, (LlamaForCausalLM, GPT2LMHeadModel, MoEForCausalLM))


def apply_transformers_model_patches(model: Any, *, performance: bool = True, compat: bool = True, **kw: Any):
    """Convert a Hugging Face model (or bare config) of a registered family into the framework's model."""
    if _is_framework_model(model):
        return model
    cfg = getattr(model, "config", model)
    mtype = _cfg_get(cfg, "model_type")
    if mtype not in _FAMILIES:
        raise ValueError(f"model_type {mtype!r} has no registered family; known: {supported_families()}")
    out = _FAMILIES[mtype](cfg, kw)
    if isinstance(model, torch.nn.Module):
        sd = model.state_dict()
        if mtype == "gpt2":
            from ..models.gpt2 import from_hf_state_dict
            sd = from_hf_state_dict(sd)
            pad = out.wte.weight.shape[0] - sd["wte.weight"].shape[0]
            if pad > 0:
                sd["wte.weight"] = torch.cat([sd["wte.weight"], sd["wte.weight"].new_zeros(pad, sd["wte.weight"].shape[1])])
        missing, unexpected = out.load_state_dict(sd, strict=False)
        real_missing = [k for k in missing if "rope_" not in k]
        if real_missing and kw.get("strict", True):
            raise ValueError(f"weights missing for {real_missing[:5]} ... while converting {mtype}")
    return out


def apply_peft_model_patches(model: Any, *, r: int | None = None, lora_alpha: float | None = None,
                             target_modules=("q_proj", "k_proj", "v_proj", "o_proj"), **kw: Any):
    """Attach LoRA adapters (PEFT naming) to a framework model, or read ``r / alpha / targets`` from a PEFT config."""
    cfg = kw.get("peft_config")
    if cfg is not None:
        r = r or _cfg_get(cfg, "r")
        lora_alpha = lora_alpha or _cfg_get(cfg, "lora_alpha")
        target_modules = _cfg_get(cfg, "target_modules", target_modules)
    if r is None:
        return model
    model.add_lora(int(r), float(lora_alpha or 2 * r), tuple(target_modules))
    return model


def apply_model_patches(model: Any, *, performance: bool = True, compat: bool = True, peft: bool = True,
                        fused_linear_cross_entropy: bool = False, **kwargs: Any):
    """One call for both steps; ``fused_linear_cross_entropy`` is always on (``per_example_loss`` uses it)."""
    peft_kw = {k: kwargs.pop(k) for k in ("r", "lora_alpha", "target_modules", "peft_config") if k in kwargs}
    out = apply_transformers_model_patches(model, performance=performance, compat=compat, **kwargs)
    if peft and peft_kw:
        out = apply_peft_model_patches(out, **peft_kw)
    return out


def apply_runtime_patches(*, performance: bool = True, compat: bool = True, **kwargs: Any) -> dict[str, str]:
    """Nothing in the runtime needs patching: report why, and mark the call as done."""
    _RUNTIME["patched"] = True
    return {"vmap_masking": "not needed: the fused engine is explicit-batch, the reference engine uses framework models",
            "empty_batches": "handled by alignment.data collators and the engines' empty-batch short-circuit",
            "vmap_checkpointing": "not needed: torch.utils.checkpoint works in the explicit-batch engine",
            "vmap_grouped_mm": "not needed: grouped GEMMs are called outside vmap"}


def is_runtime_patched() -> bool:
    return _RUNTIME["patched"]


__all__ = ["apply_model_patches", "apply_peft_model_patches", "apply_runtime_patches", "apply_transformers_model_patches",
           "is_runtime_patched", "kernels", "register_family", "supported_families"]
