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

import math
from collections.abc import Callable
from typing import Any

import torch

from . import inplace, kernels
from ..models import GPT2Config, GPT2LMHeadModel, LlamaConfig, LlamaForCausalLM, MoEConfig, MoEForCausalLM

_FAMILIES: dict[str, Callable[[Any, dict], torch.nn.Module]] = {}
_RUNTIME = {"patched": False}

# model_type -> family builder.  Only families whose block structure these modules reproduce exactly are registered;
# the others are listed with the reason, so a conversion can never silently drop a feature of the architecture.
LLAMA_LIKE = ("llama", "mistral", "ministral", "mellum", "qwen2", "qwen3", "gemma", "gemma2", "gemma3_text", "phi3", "granite",
              "smollm3", "olmo2", "olmo3", "exaone4", "glm4", "cohere", "cohere2")
MOE_LIKE = ("mixtral", "qwen2_moe", "qwen3_moe", "hunyuan_v1_moe", "gpt_oss")
ROPE_INTERLEAVED = frozenset({"glm4", "cohere", "cohere2"})      # families that rotate the pairs (2i, 2i+1); q / k rows are permuted on conversion
UNSUPPORTED = {
    "gemma3": "the multimodal wrapper; convert its text model (model_type gemma3_text)",
}
# deepseek_v4 (latent attention), qwen3_next and qwen3_5_moe (gated delta-net layers) are not converted either: they stay
# Hugging Face models and get kernel forwards in place (patches/inplace.py), as the reference does for them.


def register_family(model_type: str, builder: Callable[..., Any]) -> None:
    """Register a family for a Hugging Face ``model_type``: either ``builder(hf_config, options) -> nn.Module`` (the model
    is CONVERTED into this package's modules) or a function built by ``inplace.make_apply_model_patches`` (the model stays
    a Hugging Face model and gets kernel forwards in place)."""
    if getattr(builder, "is_model_patch_fn", False):
        inplace.register_inplace_family(model_type, builder)
    else:
        _FAMILIES[model_type] = builder


def _cfg_get(cfg: Any, name: str, default=None):
    v = cfg.get(name, default) if isinstance(cfg, dict) else getattr(cfg, name, default)
    return default if v is None else v


def _rope_theta(cfg: Any, default: float) -> float:
    rp = _cfg_get(cfg, "rope_parameters") or {}
    if isinstance(rp, dict) and rp.get("rope_theta"):
        return float(rp["rope_theta"])
    return float(_cfg_get(cfg, "rope_theta", default))


def rope_row_permutation(head_dim: int, rotary_dim: int, interleaved: bool) -> torch.Tensor:
    """Order of one head's rows that turns a source rotary layout into this package's.

    The kernels here rotate the pairs ``(i, i + head_dim/2)`` and leave a pair alone where the tables hold
    ``cos = 1, sin = 0``.  A source model rotates, inside its first ``rotary_dim`` dimensions, either the pairs
    ``(2i, 2i+1)`` (``interleaved``) or ``(i, i + rotary_dim/2)``, and passes the other dimensions through.  Taking q and
    k rows in the returned order puts the two members of rotating pair ``i`` at ``i`` and ``head_dim/2 + i`` and fills the
    remaining positions with the pass-through dimensions; q·k is unchanged because both are permuted alike.
    """
    half, rh = head_dim // 2, rotary_dim // 2
    if interleaved:
        first, second = [2 * i for i in range(rh)], [2 * i + 1 for i in range(rh)]
    else:
        first, second = list(range(rh)), [rh + i for i in range(rh)]
    rest = list(range(rotary_dim, head_dim))
    keep = half - rh
    return torch.tensor(first + rest[:keep] + second + rest[keep:], dtype=torch.long)


def _layer_windows(cfg: Any) -> tuple | None:
    """Per-layer attention window from ``layer_types`` (``sliding_attention`` layers get ``sliding_window``)."""
    types, window = _cfg_get(cfg, "layer_types"), _cfg_get(cfg, "sliding_window")
    if not types or window is None:
        return None
    bad = sorted(set(types) - {"sliding_attention", "full_attention"})
    if bad:
        raise NotImplementedError(f"layer types {bad} are not implemented")
    return tuple(int(window) if t == "sliding_attention" else None for t in types)


def _rope_scaling(cfg: Any) -> dict | None:
    """The rope scaling dictionary of a Hugging Face config (``rope_parameters`` in new configs, ``rope_scaling`` in old
    ones), or ``None`` for plain RoPE; unknown kinds are refused when the tables are built."""
    for name in ("rope_parameters", "rope_scaling"):
        rp = _cfg_get(cfg, name)
        if isinstance(rp, dict):
            kind = rp.get("rope_type", rp.get("type", "default")) or "default"
            if kind != "default":
                out = {k: v for k, v in rp.items() if k != "rope_theta"}
                out["rope_type"] = kind
                out.setdefault("original_max_position_embeddings", _cfg_get(cfg, "max_position_embeddings"))
                return out
    return None


def _build_llama(cfg: Any, opt: dict) -> torch.nn.Module:
    mtype = _cfg_get(cfg, "model_type")
    extra: dict[str, Any] = {}
    if mtype == "qwen2":
        extra.update(attention_bias=True)
    elif mtype == "qwen3":
        extra.update(qk_norm=True, attention_bias=bool(_cfg_get(cfg, "attention_bias", False)))
    elif mtype == "granite":
        extra.update(attention_bias=bool(_cfg_get(cfg, "attention_bias", False)), attention_out_bias=bool(_cfg_get(cfg, "attention_bias", False)),
                     mlp_bias=bool(_cfg_get(cfg, "mlp_bias", False)), embedding_scale=float(_cfg_get(cfg, "embedding_multiplier", 1.0)),
                     attention_multiplier=float(_cfg_get(cfg, "attention_multiplier", 1.0)),
                     residual_multiplier=float(_cfg_get(cfg, "residual_multiplier", 1.0)), logits_scaling=float(_cfg_get(cfg, "logits_scaling", 1.0)))
    elif mtype == "olmo2":
        extra.update(attention_bias=bool(_cfg_get(cfg, "attention_bias", False)), attention_out_bias=bool(_cfg_get(cfg, "attention_bias", False)),
                     post_norm=True, qk_norm_full=True)
    elif mtype == "smollm3":
        extra.update(attention_bias=bool(_cfg_get(cfg, "attention_bias", False)), attention_out_bias=bool(_cfg_get(cfg, "attention_bias", False)),
                     mlp_bias=bool(_cfg_get(cfg, "mlp_bias", False)), no_rope_layers=tuple(int(x) for x in _cfg_get(cfg, "no_rope_layers")))
    elif mtype in ("gemma2", "gemma3_text"):
        extra.update(hidden_act=_cfg_get(cfg, "hidden_activation") or _cfg_get(cfg, "hidden_act", "gelu_pytorch_tanh"), norm_offset=1.0,
                     norm_casting="gemma", embedding_scale=float(_cfg_get(cfg, "hidden_size")) ** 0.5, sandwich_norm=True,
                     attention_multiplier=float(_cfg_get(cfg, "query_pre_attn_scalar", 256)) ** -0.5,
                     attention_bias=bool(_cfg_get(cfg, "attention_bias", False)), attention_out_bias=bool(_cfg_get(cfg, "attention_bias", False)),
                     attn_logit_softcap=_cfg_get(cfg, "attn_logit_softcapping"), final_logit_softcap=_cfg_get(cfg, "final_logit_softcapping"),
                     layer_windows=_layer_windows(cfg))
        if _cfg_get(cfg, "use_bidirectional_attention"):
            raise NotImplementedError("bidirectional attention is not implemented")
        if mtype == "gemma3_text":
            rp = _cfg_get(cfg, "rope_parameters") or {}
            local, full = rp.get("sliding_attention") or {}, rp.get("full_attention") or {}
            if (local.get("rope_type") or "default") != "default":
                raise NotImplementedError("rope scaling on the windowed layers is not implemented")
            extra.update(qk_norm=True, local_rope_theta=float(local.get("rope_theta") or _cfg_get(cfg, "rope_local_base_freq", 10000.0)))
            opt = {**opt, "_rope": (float(full.get("rope_theta") or 1e6),
                                    None if (full.get("rope_type") or "default") == "default" else {k: v for k, v in full.items() if k != "rope_theta"})}
    elif mtype == "olmo3":
        extra.update(attention_bias=bool(_cfg_get(cfg, "attention_bias", False)), attention_out_bias=bool(_cfg_get(cfg, "attention_bias", False)),
                     post_norm=True, qk_norm_full=True, layer_windows=_layer_windows(cfg))
        if _rope_scaling(cfg) is not None:
            raise NotImplementedError("OLMo-3 applies rope scaling to its full-attention layers only; that split is not implemented")
    elif mtype == "glm4":
        extra.update(attention_bias=bool(_cfg_get(cfg, "attention_bias", True)), sandwich_norm=True,
                     partial_rotary_factor=float(_cfg_get(cfg, "partial_rotary_factor", 0.5)))
    elif mtype in ("cohere", "cohere2"):
        if _cfg_get(cfg, "use_qk_norm", False):
            raise NotImplementedError("Cohere q/k LayerNorm with per-head weights is not implemented")
        extra.update(attention_bias=bool(_cfg_get(cfg, "attention_bias", False)), attention_out_bias=bool(_cfg_get(cfg, "attention_bias", False)),
                     norm_type="layernorm", parallel_block=True, logits_scaling=1.0 / float(_cfg_get(cfg, "logit_scale", 1.0)))
        if mtype == "cohere2":
            windows = _layer_windows(cfg)
            extra.update(layer_windows=windows)
            if windows is not None:                    # full-attention layers carry no rotary embedding
                extra.update(no_rope_layers=tuple(1 if w is not None else 0 for w in windows))
        opt = {**opt, "_eps": float(_cfg_get(cfg, "layer_norm_eps", 1e-5))}
    elif mtype == "exaone4":
        windows = _layer_windows(cfg)
        extra.update(post_norm=True, qk_norm=True, layer_windows=windows)
        if _cfg_get(cfg, "sliding_window") is not None and windows is not None:      # hybrid: global layers carry no rotary embedding
            extra.update(no_rope_layers=tuple(1 if w is not None else 0 for w in windows))
    elif mtype == "gemma":
        extra.update(hidden_act=_cfg_get(cfg, "hidden_activation") or _cfg_get(cfg, "hidden_act", "gelu_pytorch_tanh"), norm_offset=1.0,
                     norm_casting="gemma", embedding_scale=float(_cfg_get(cfg, "hidden_size")) ** 0.5)
    else:
        extra.update(attention_bias=bool(_cfg_get(cfg, "attention_bias", False)), attention_out_bias=bool(_cfg_get(cfg, "attention_bias", False)),
                     mlp_bias=bool(_cfg_get(cfg, "mlp_bias", False)))
    if "hidden_act" not in extra:
        extra["hidden_act"] = _cfg_get(cfg, "hidden_act", "silu")
    if "partial_rotary_factor" not in extra:          # e.g. Phi-4-mini: 0.75 with the (i, i + rotary_dim/2) layout
        rp = _cfg_get(cfg, "rope_parameters") or {}
        pf = _cfg_get(cfg, "partial_rotary_factor") or (rp.get("partial_rotary_factor") if isinstance(rp, dict) else None)
        if pf and float(pf) < 1.0:
            extra["partial_rotary_factor"] = float(pf)
    window = _cfg_get(cfg, "sliding_window") if _cfg_get(cfg, "use_sliding_window", mtype in ("mistral", "ministral")) else None
    theta, scaling = opt.get("_rope") or (_rope_theta(cfg, 10000.0), _rope_scaling(cfg))
    c = LlamaConfig(vocab_size=_cfg_get(cfg, "vocab_size"), hidden_size=_cfg_get(cfg, "hidden_size"),
                    intermediate_size=_cfg_get(cfg, "intermediate_size"), num_hidden_layers=_cfg_get(cfg, "num_hidden_layers"),
                    num_attention_heads=_cfg_get(cfg, "num_attention_heads"),
                    num_key_value_heads=_cfg_get(cfg, "num_key_value_heads") or _cfg_get(cfg, "num_attention_heads"),
                    rms_norm_eps=opt.get("_eps") or _cfg_get(cfg, "rms_norm_eps", 1e-6), rope_theta=theta, rope_scaling=scaling,
                    max_position_embeddings=_cfg_get(cfg, "max_position_embeddings", 8192),
                    tie_word_embeddings=bool(_cfg_get(cfg, "tie_word_embeddings", False)), head_dim=_cfg_get(cfg, "head_dim"),
                    sliding_window=window, **extra)
    return LlamaForCausalLM(c, dtype=opt.get("dtype", torch.bfloat16), device=opt.get("device"))


def _build_gpt2(cfg: Any, opt: dict) -> torch.nn.Module:
    c = GPT2Config(vocab_size=_cfg_get(cfg, "vocab_size"), n_positions=_cfg_get(cfg, "n_positions", 1024),
                   n_embd=_cfg_get(cfg, "n_embd"), n_layer=_cfg_get(cfg, "n_layer"), n_head=_cfg_get(cfg, "n_head"),
                   layer_norm_epsilon=_cfg_get(cfg, "layer_norm_epsilon", 1e-5))
    return GPT2LMHeadModel(c, dtype=opt.get("dtype", torch.bfloat16), device=opt.get("device"))


def _build_moe(cfg: Any, opt: dict) -> torch.nn.Module:
    mtype = _cfg_get(cfg, "model_type")
    shared = _cfg_get(cfg, "shared_expert_intermediate_size", 0) if mtype == "qwen2_moe" else 0
    dense: tuple = ()
    if mtype in ("qwen2_moe", "qwen3_moe"):        # a layer is sparse when it is not listed as MLP-only and falls on the sparse step
        only, step = set(_cfg_get(cfg, "mlp_only_layers") or ()), int(_cfg_get(cfg, "decoder_sparse_step", 1) or 1)
        dense = tuple(i for i in range(_cfg_get(cfg, "num_hidden_layers")) if i in only or (i + 1) % step != 0)
    if mtype == "gpt_oss":
        hd = _cfg_get(cfg, "head_dim") or _cfg_get(cfg, "hidden_size") // _cfg_get(cfg, "num_attention_heads")
        c = MoEConfig(vocab_size=_cfg_get(cfg, "vocab_size"), hidden_size=_cfg_get(cfg, "hidden_size"),
                      num_hidden_layers=_cfg_get(cfg, "num_hidden_layers"), num_attention_heads=_cfg_get(cfg, "num_attention_heads"),
                      num_key_value_heads=_cfg_get(cfg, "num_key_value_heads") or _cfg_get(cfg, "num_attention_heads"),
                      num_experts=_cfg_get(cfg, "num_local_experts"), moe_intermediate_size=_cfg_get(cfg, "intermediate_size"),
                      num_shared_experts=0, attention_bias=bool(_cfg_get(cfg, "attention_bias", True)),
                      attention_out_bias=bool(_cfg_get(cfg, "attention_bias", True)), head_dim=hd,
                      num_experts_per_tok=_cfg_get(cfg, "num_experts_per_tok", 4), norm_topk_prob=True,       # softmax over the top-k logits
                      rms_norm_eps=_cfg_get(cfg, "rms_norm_eps", 1e-5), rope_theta=_rope_theta(cfg, 150000.0),
                      rope_scaling=_rope_scaling(cfg), router_bias=True, expert_bias=True, expert_act="gpt_oss",
                      attention_sinks=True, layer_windows=_layer_windows(cfg),
                      max_position_embeddings=_cfg_get(cfg, "max_position_embeddings", 4096))
        return MoEForCausalLM(c, dtype=opt.get("dtype", torch.bfloat16), device=opt.get("device"))
    if mtype == "hunyuan_v1_moe":
        for name in ("num_experts", "moe_topk"):
            if not isinstance(_cfg_get(cfg, name), int):
                raise NotImplementedError(f"per-layer {name} lists are not implemented")
        rp = _cfg_get(cfg, "rope_parameters") or {}
        theta = float(rp.get("rope_theta") or _cfg_get(cfg, "rope_theta", 10000.0))
        hd = _cfg_get(cfg, "head_dim") or _cfg_get(cfg, "hidden_size") // _cfg_get(cfg, "num_attention_heads")
        scaling = _rope_scaling(cfg)
        if rp.get("rope_type") == "dynamic" and rp.get("alpha"):       # NTK-alpha: a larger base, no position scaling
            theta, scaling = theta * float(rp["alpha"]) ** (hd / (hd - 2)), None
        inter = _cfg_get(cfg, "intermediate_size")
        c = MoEConfig(vocab_size=_cfg_get(cfg, "vocab_size"), hidden_size=_cfg_get(cfg, "hidden_size"),
                      num_hidden_layers=_cfg_get(cfg, "num_hidden_layers"), num_attention_heads=_cfg_get(cfg, "num_attention_heads"),
                      num_key_value_heads=_cfg_get(cfg, "num_key_value_heads") or _cfg_get(cfg, "num_attention_heads"),
                      num_experts=_cfg_get(cfg, "num_experts"), moe_intermediate_size=inter, num_shared_experts=1,
                      shared_intermediate_size=inter, shared_expert_gate=False, attention_bias=bool(_cfg_get(cfg, "attention_bias", False)),
                      head_dim=hd, qk_norm=True, qk_norm_after_rope=True, num_experts_per_tok=_cfg_get(cfg, "moe_topk"),
                      norm_topk_prob=True, rms_norm_eps=_cfg_get(cfg, "rms_norm_eps", 1e-5), rope_theta=theta, rope_scaling=scaling,
                      max_position_embeddings=_cfg_get(cfg, "max_position_embeddings", 4096))
        return MoEForCausalLM(c, dtype=opt.get("dtype", torch.bfloat16), device=opt.get("device"))
    c = MoEConfig(vocab_size=_cfg_get(cfg, "vocab_size"), hidden_size=_cfg_get(cfg, "hidden_size"),
                  num_hidden_layers=_cfg_get(cfg, "num_hidden_layers"), num_attention_heads=_cfg_get(cfg, "num_attention_heads"),
                  num_key_value_heads=_cfg_get(cfg, "num_key_value_heads") or _cfg_get(cfg, "num_attention_heads"),
                  num_experts=_cfg_get(cfg, "num_experts") or _cfg_get(cfg, "num_local_experts"),
                  moe_intermediate_size=_cfg_get(cfg, "moe_intermediate_size") if mtype != "mixtral" else _cfg_get(cfg, "intermediate_size"),
                  num_shared_experts=1 if shared else 0, shared_intermediate_size=shared or None, shared_expert_gate=bool(shared),
                  attention_bias=mtype == "qwen2_moe", head_dim=_cfg_get(cfg, "head_dim"), qk_norm=mtype == "qwen3_moe",
                  num_experts_per_tok=_cfg_get(cfg, "num_experts_per_tok", 2),
                  norm_topk_prob=bool(_cfg_get(cfg, "norm_topk_prob", mtype == "mixtral")) or mtype == "mixtral",
                  rms_norm_eps=_cfg_get(cfg, "rms_norm_eps", 1e-6), rope_theta=_rope_theta(cfg, 1e6),
                  rope_scaling=_rope_scaling(cfg), dense_layers=dense,
                  dense_intermediate_size=_cfg_get(cfg, "intermediate_size") if dense else None,
                  max_position_embeddings=_cfg_get(cfg, "max_position_embeddings", 4096))
    return MoEForCausalLM(c, dtype=opt.get("dtype", torch.bfloat16), device=opt.get("device"))


for _t in LLAMA_LIKE:
    register_family(_t, _build_llama)
for _t in MOE_LIKE:
    register_family(_t, _build_moe)
register_family("gpt2", _build_gpt2)


def _convert_state_dict(mtype: str, sd: dict, out: torch.nn.Module) -> dict:
    """Rename / split / pad a Hugging Face state dict so that it loads into the framework model with ``strict=True``."""
    if mtype == "gpt2":
        from ..models.gpt2 import from_hf_state_dict
        sd = from_hf_state_dict(sd)
        pad = out.wte.weight.shape[0] - sd["wte.weight"].shape[0]
        if pad > 0:
            sd["wte.weight"] = torch.cat([sd["wte.weight"], sd["wte.weight"].new_zeros(pad, sd["wte.weight"].shape[1])])
        return {k: v for k, v in sd.items() if not k.endswith(".attn.bias") and not k.endswith(".attn.masked_bias")}
    res: dict[str, torch.Tensor] = {}
    moe = mtype in MOE_LIKE
    for k, v in sd.items():
        if "rotary_emb" in k:
            continue
        if moe:
            k = k.removeprefix("model.")
        if mtype == "gpt_oss":
            k = k.replace(".mlp.router.", ".mlp.gate.")
            if k.endswith("experts.gate_up_proj"):                 # [E, H, 2I] with gate / up interleaved -> [E, 2I, H], gate rows first
                v = torch.cat([v[:, :, 0::2], v[:, :, 1::2]], dim=2).transpose(1, 2).contiguous()
            elif k.endswith("experts.gate_up_proj_bias"):
                k, v = k[: -len("gate_up_proj_bias")] + "gate_up_bias", torch.cat([v[:, 0::2], v[:, 1::2]], dim=1)
            elif k.endswith("experts.down_proj"):                  # [E, I, H] -> [E, H, I]
                v = v.transpose(1, 2).contiguous()
            elif k.endswith("experts.down_proj_bias"):
                k = k[: -len("down_proj_bias")] + "down_bias"
            elif k.endswith("mlp.gate.bias"):
                rows = out.config.padded_experts
                v = torch.cat([v, v.new_zeros(rows - v.shape[0])]) if v.shape[0] < rows else v
        if mtype == "hunyuan_v1_moe":
            k = (k.replace(".query_layernorm.", ".q_norm.").replace(".key_layernorm.", ".k_norm.")
                 .replace(".mlp.gate.wg.", ".mlp.gate.").replace(".mlp.shared_mlp.", ".mlp.shared_expert."))
        if mtype == "phi3" and k.endswith("self_attn.qkv_proj.weight"):
            cfg = out.config
            nq, nkv = cfg.num_attention_heads * cfg.hd, cfg.num_key_value_heads * cfg.hd
            base = k[: -len("qkv_proj.weight")]
            res[base + "q_proj.weight"], res[base + "k_proj.weight"], res[base + "v_proj.weight"] = v[:nq], v[nq:nq + nkv], v[nq + nkv:]
            continue
        if mtype == "phi3" and k.endswith("mlp.gate_up_proj.weight"):
            half = v.shape[0] // 2
            base = k[: -len("gate_up_proj.weight")]
            res[base + "gate_proj.weight"], res[base + "up_proj.weight"] = v[:half], v[half:]
            continue
        if mtype == "glm4":
            if k.endswith("mlp.gate_up_proj.weight"):
                half = v.shape[0] // 2
                base = k[: -len("gate_up_proj.weight")]
                res[base + "gate_proj.weight"], res[base + "up_proj.weight"] = v[:half], v[half:]
                continue
            # four norms per layer: (input, post_self_attn) around attention, (post_attention, post_mlp) around the MLP
            for src, dst in ((".post_attention_layernorm.", ".pre_feedforward_layernorm."),
                             (".post_self_attn_layernorm.", ".post_attention_layernorm."),
                             (".post_mlp_layernorm.", ".post_feedforward_layernorm.")):
                if src in k:
                    k = k.replace(src, dst)
                    break
        if moe and (k.endswith("mlp.gate.weight") or k.endswith("mlp.shared_expert_gate.weight")):
            rows = out.config.padded_experts if k.endswith("mlp.gate.weight") else 8
            v = torch.cat([v, v.new_zeros(rows - v.shape[0], v.shape[1])]) if v.shape[0] < rows else v
        res[k] = v
    cfg = out.config
    factor = float(getattr(cfg, "partial_rotary_factor", 1.0))
    if not moe and (mtype in ROPE_INTERLEAVED or factor < 1.0):
        hd = cfg.hd
        perm = rope_row_permutation(hd, int(hd * factor), mtype in ROPE_INTERLEAVED)
        for k in list(res):
            if k.endswith(("self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.q_proj.bias", "self_attn.k_proj.bias",
                           "self_attn.q_proj.lora_B", "self_attn.k_proj.lora_B")):       # LoRA B rows are output rows too
                v = res[k]
                heads = v.shape[0] // hd
                res[k] = v.reshape(heads, hd, *v.shape[1:])[:, perm].reshape(v.shape).contiguous()
    tied = getattr(out.config, "tie_word_embeddings", False)
    if "lm_head.weight" not in res:
        emb = "embed_tokens.weight" if moe else "model.embed_tokens.weight"
        if tied or emb in res:
            res["lm_head.weight"] = res[emb]
    return res


def supported_families() -> list[str]:
    """Sorted Hugging Face ``model_type`` names that ``apply_model_patches`` accepts: converted into this package's models,
    or (``inplace.inplace_families()``) kept as Hugging Face models with kernel forwards patched in."""
    return sorted(set(_FAMILIES) | set(inplace.INPLACE_FAMILIES))


def _is_framework_model(model: Any) -> bool:
    return isinstance(model, (LlamaForCausalLM, GPT2LMHeadModel, MoEForCausalLM))


def apply_transformers_model_patches(model: Any, *, performance: bool = True, compat: bool = True, **kw: Any):
    """Convert a Hugging Face model (or bare config) of a registered family into the framework's model.

    The converted state dict must load with ``strict=True`` (every weight of the source has a place, every parameter of
    the target gets a value); families whose blocks differ from the modules here raise ``NotImplementedError`` with the
    reason instead of converting approximately.
    """
    if _is_framework_model(model):
        return model
    cfg = getattr(model, "config", model)
    mtype = _cfg_get(cfg, "model_type")
    if mtype in UNSUPPORTED:
        raise NotImplementedError(f"model_type {mtype!r} is not converted: {UNSUPPORTED[mtype]}")
    custom = inplace.registered_inplace_family(mtype)
    if custom is not None:                       # a family registered through the factory API: patched in place
        if not isinstance(model, torch.nn.Module):
            raise ValueError(f"model_type {mtype!r} is patched in place: pass the instantiated model, not a config")
        custom(model, performance=performance, compat=compat)
        return model
    if mtype in inplace.INPLACE_FAMILIES:
        if not isinstance(model, torch.nn.Module):
            raise ValueError(f"model_type {mtype!r} is patched in place: pass the instantiated Hugging Face model, not a config")
        if performance:
            inplace.apply_inplace_patches(model, mtype)
        return model
    if mtype not in _FAMILIES:
        raise ValueError(f"model_type {mtype!r} has no registered family; known: {supported_families()}")
    out = _FAMILIES[mtype](cfg, kw)
    out.source_model_type = mtype               # which Hugging Face naming / rotary layout adapters are exported in
    if isinstance(model, torch.nn.Module):
        sd = _convert_state_dict(mtype, dict(model.state_dict()), out)
        missing, unexpected = out.load_state_dict(sd, strict=False)
        missing = [k for k in missing if "rope_" not in k]
        if (missing or unexpected) and kw.get("strict", True):
            raise ValueError(f"converting {mtype}: missing {missing[:5]}, unexpected {list(unexpected)[:5]}")
    return out


def _is_peft_wrapped(model: Any) -> bool:
    """A model wrapped by the PEFT library: ``peft_config`` (adapter name -> config) and ``base_model.model`` (the
    Hugging Face model with adapter layers injected).  Recognised by structure, so the library need not be importable."""
    base = getattr(model, "base_model", None)
    return isinstance(getattr(model, "peft_config", None), dict) and isinstance(getattr(base, "model", None), torch.nn.Module)


_PEFT_REFUSED = {"use_dora": "DoRA (weight-decomposed adapters)", "modules_to_save": "modules_to_save (fully trained copies)",
                 "fan_in_fan_out": "fan_in_fan_out (transposed base weights)", "layer_replication": "layer replication",
                 "rank_pattern": "per-module ranks (rank_pattern)", "alpha_pattern": "per-module alpha (alpha_pattern)"}


def convert_peft_model(model: Any, *, adapter_name: str | None = None, **kw: Any):
    """Turn a PEFT-wrapped Hugging Face model (``peft.get_peft_model(hf, LoraConfig(...))``) into this package's model with
    the same base weights AND the same LoRA factors, so that training continues from the adapter as it is.

    Read from the wrapper by structure: ``peft_config[adapter]`` (``r``, ``lora_alpha``, ``target_modules``,
    ``use_rslora``), and from the injected layers ``<module>.base_layer.weight``, ``<module>.lora_A.<adapter>.weight``
    ``[r, in]``, ``<module>.lora_B.<adapter>.weight`` ``[out, r]``.  Options this package has no module for (DoRA,
    ``modules_to_save``, transposed base weights, per-module ranks, adapter bias) are refused by name; LoRA dropout is
    refused unless it is zero (a per-call random mask would have to be shared with the per-example gradient kernels).

    Parity: packages/opaque-patches/src/opaque/api/patches/peft/_router.py (PEFT layers routed onto fused LoRA kernels).
    """
    if not _is_peft_wrapped(model):
        raise ValueError("not a PEFT-wrapped model: expected .peft_config (dict) and .base_model.model")
    name = adapter_name or getattr(model, "active_adapter", None) or next(iter(model.peft_config))
    if isinstance(name, (list, tuple)):
        if len(name) != 1:
            raise NotImplementedError(f"several active adapters {list(name)}: pick one with adapter_name=")
        name = name[0]
    if name not in model.peft_config:
        raise ValueError(f"adapter {name!r} not in {sorted(model.peft_config)}")
    cfg = model.peft_config[name]
    ptype = str(_cfg_get(cfg, "peft_type", "LORA")).upper().split(".")[-1]
    if ptype != "LORA":
        raise NotImplementedError(f"PEFT method {ptype!r}: only LoRA adapters are converted")
    for field, what in _PEFT_REFUSED.items():
        if _cfg_get(cfg, field, None):
            raise NotImplementedError(f"PEFT option {what} is not supported")
    if str(_cfg_get(cfg, "bias", "none")) != "none":
        raise NotImplementedError("PEFT option bias != 'none' (trainable biases beside the adapter) is not supported")
    if float(_cfg_get(cfg, "lora_dropout", 0.0) or 0.0) != 0.0:
        raise NotImplementedError("lora_dropout > 0 is not supported: set it to 0 for differentially private training")
    r = int(_cfg_get(cfg, "r"))
    alpha = float(_cfg_get(cfg, "lora_alpha", r))
    if _cfg_get(cfg, "use_rslora", False):
        alpha = alpha * math.sqrt(r)             # rank-stabilised scaling alpha / sqrt(r), expressed as alpha' / r
    hf = model.base_model.model
    sd, targets = {}, set()
    a_tag, b_tag = f".lora_A.{name}.weight", f".lora_B.{name}.weight"
    for k, v in hf.state_dict().items():
        if ".base_layer." in k:
            sd[k.replace(".base_layer.", ".")] = v
        elif k.endswith(a_tag):
            sd[k[: -len(a_tag)] + ".lora_A"] = v
            targets.add(k[: -len(a_tag)].split(".")[-1])
        elif k.endswith(b_tag):
            sd[k[: -len(b_tag)] + ".lora_B"] = v
        elif ".lora_A." in k or ".lora_B." in k or ".lora_embedding_" in k or ".lora_magnitude_vector" in k:
            if f".{name}." in k or k.endswith(f".{name}"):
                raise NotImplementedError(f"adapter tensor {k!r} has no counterpart here")
            continue                                 # another (inactive) adapter
        else:
            sd[k] = v
    if not targets:
        raise ValueError(f"adapter {name!r} has no LoRA layers in the wrapped model")
    hcfg = hf.config
    mtype = _cfg_get(hcfg, "model_type")
    if mtype not in _FAMILIES:
        raise NotImplementedError(f"model_type {mtype!r} under PEFT: only converted families ({sorted(_FAMILIES)}) take adapters")
    out = _FAMILIES[mtype](hcfg, kw)
    if not hasattr(out, "add_lora"):
        raise NotImplementedError(f"model_type {mtype!r} has no LoRA support in this package")
    out.source_model_type = mtype
    out.add_lora(r, alpha, tuple(sorted(targets)))
    conv = _convert_state_dict(mtype, sd, out)
    missing, unexpected = out.load_state_dict(conv, strict=False)
    missing = [k for k in missing if "rope_" not in k]
    if missing or unexpected:
        raise ValueError(f"converting PEFT-wrapped {mtype}: missing {missing[:5]}, unexpected {list(unexpected)[:5]}")
    return out


def _qk_row_permutation(model: Any, mtype: str) -> torch.Tensor | None:
    """The q / k output-row permutation that conversion applied for this family (``None``: rows kept as they are)."""
    cfg = model.config
    factor = float(getattr(cfg, "partial_rotary_factor", 1.0))
    if mtype in MOE_LIKE or not (mtype in ROPE_INTERLEAVED or factor < 1.0):
        return None
    return rope_row_permutation(cfg.hd, int(cfg.hd * factor), mtype in ROPE_INTERLEAVED)


def peft_adapter_state_dict(model: Any, *, model_type: str | None = None) -> dict[str, torch.Tensor]:
    """The model's LoRA factors under the names and row order the PEFT library saves them in:
    ``base_model.model.<hugging face module path>.lora_A.weight`` / ``.lora_B.weight`` (no adapter name in the key)."""
    mtype = model_type or getattr(model, "source_model_type", "llama")
    perm = _qk_row_permutation(model, mtype)
    prefix = "base_model.model." + ("model." if mtype in MOE_LIKE else "")
    out: dict[str, torch.Tensor] = {}
    for name, p in model.named_parameters():
        if not name.endswith((".lora_A", ".lora_B")):
            continue
        v = p.detach().to("cpu").clone()
        if perm is not None and name.endswith(("self_attn.q_proj.lora_B", "self_attn.k_proj.lora_B")):
            inv = torch.empty_like(perm)
            inv[perm] = torch.arange(perm.numel())
            hd = perm.numel()
            v = v.reshape(v.shape[0] // hd, hd, v.shape[1])[:, inv].reshape(v.shape).contiguous()
        out[prefix + name + ".weight"] = v
    if not out:
        raise ValueError("the model has no LoRA factors")
    return out


def export_peft_adapter(model: Any, output_dir: str, *, base_model_name_or_path: str | None = None,
                        model_type: str | None = None) -> str:
    """Write the LoRA adapter as the two files the PEFT library loads: ``adapter_model.safetensors`` and
    ``adapter_config.json`` (``PeftModel.from_pretrained(base, output_dir)`` on the Hugging Face side)."""
    import json
    import os
    from safetensors.torch import save_file
    sd = peft_adapter_state_dict(model, model_type=model_type)
    mods = [m for m in model.modules() if getattr(m, "lora_A", None) is not None]
    r = int(mods[0].lora_A.shape[0])
    targets = sorted({k.split(".")[-3] for k in sd})
    os.makedirs(output_dir, exist_ok=True)
    save_file(sd, os.path.join(output_dir, "adapter_model.safetensors"), metadata={"format": "pt"})
    cfg = {"peft_type": "LORA", "task_type": "CAUSAL_LM", "r": r, "lora_alpha": float(mods[0].scaling) * r, "lora_dropout": 0.0,
           "bias": "none", "target_modules": targets, "fan_in_fan_out": False, "use_rslora": False, "use_dora": False,
           "modules_to_save": None, "inference_mode": True, "base_model_name_or_path": base_model_name_or_path}
    with open(os.path.join(output_dir, "adapter_config.json"), "w") as f:
        json.dump(cfg, f, indent=1)
    return output_dir


def load_peft_adapter(model: Any, path_or_state: Any, *, model_type: str | None = None) -> Any:
    """Load an adapter saved by the PEFT library (a directory with ``adapter_model.safetensors`` + ``adapter_config.json``,
    or the state dict itself) into a framework model; LoRA factors are attached first if the model has none."""
    import json
    import os
    mtype = model_type or getattr(model, "source_model_type", "llama")
    if isinstance(path_or_state, (str, os.PathLike)):
        from safetensors.torch import load_file
        sd = load_file(os.path.join(path_or_state, "adapter_model.safetensors"))
        with open(os.path.join(path_or_state, "adapter_config.json")) as f:
            cfg = json.load(f)
        if not any(getattr(m, "lora_A", None) is not None for m in model.modules()):
            tmp = type("Cfg", (), cfg)()
            for field, what in _PEFT_REFUSED.items():
                if cfg.get(field):
                    raise NotImplementedError(f"PEFT option {what} is not supported")
            alpha = float(cfg.get("lora_alpha", cfg["r"])) * (math.sqrt(cfg["r"]) if cfg.get("use_rslora") else 1.0)
            model.add_lora(int(tmp.r), alpha, tuple(cfg["target_modules"]))
    else:
        sd = dict(path_or_state)
    perm = _qk_row_permutation(model, mtype)
    prefix = "base_model.model." + ("model." if mtype in MOE_LIKE else "")
    params = dict(model.named_parameters())
    loaded = 0
    with torch.no_grad():
        for k, v in sd.items():
            name = k.removeprefix(prefix)
            for tag in (".lora_A.weight", ".lora_B.weight", ".lora_A.default.weight", ".lora_B.default.weight"):
                if name.endswith(tag):
                    name = name[: -len(tag)] + tag[:7]
                    break
            else:
                raise ValueError(f"unexpected adapter tensor {k!r}")
            if name not in params:
                raise ValueError(f"adapter tensor {k!r} has no LoRA factor {name!r} in the model")
            if perm is not None and name.endswith(("self_attn.q_proj.lora_B", "self_attn.k_proj.lora_B")):
                hd = perm.numel()
                v = v.reshape(v.shape[0] // hd, hd, v.shape[1])[:, perm].reshape(v.shape)
            params[name].copy_(v)
            loaded += 1
    want = sum(1 for n in params if n.endswith((".lora_A", ".lora_B")))
    if loaded != want:
        raise ValueError(f"the adapter holds {loaded} tensors, the model has {want} LoRA factors")
    return model


def apply_peft_model_patches(model: Any, *, r: int | None = None, lora_alpha: float | None = None,
                             target_modules=("q_proj", "k_proj", "v_proj", "o_proj"), **kw: Any):
    """Attach LoRA adapters (PEFT naming) to a framework model, or read ``r / alpha / targets`` from a PEFT config.
    A model already wrapped by the PEFT library is converted together with its adapter (:func:`convert_peft_model`)."""
    if _is_peft_wrapped(model):
        return convert_peft_model(model, **{k: v for k, v in kw.items() if k != "peft_config"})
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
    if _is_peft_wrapped(model):                 # a PEFT-wrapped Hugging Face model: base weights and adapter together
        for k in ("r", "lora_alpha", "target_modules", "peft_config"):
            kwargs.pop(k, None)
        return convert_peft_model(model, **kwargs)
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
    """True once ``apply_runtime_patches`` ran in this process."""
    return _RUNTIME["patched"]


def apply_checkpoint_patch(vmap_checkpointing: bool = True) -> bool:
    """Activation checkpointing under per-example gradients needs no patch of ``torch.utils.checkpoint`` here: the fused
    engine is explicit-batch (the stock checkpoint works), and under ``vmap(grad)`` this package's models use
    ``functional.functional_checkpoint``.  Kept so that set-up code written for the reference runs; marks the call."""
    _RUNTIME["checkpoint"] = True
    return True


def is_checkpoint_patched() -> bool:
    """True once :func:`apply_checkpoint_patch` ran in this process."""
    return bool(_RUNTIME.get("checkpoint"))


def apply_masking_patches(vmap_masking: bool = True) -> str:
    """Attention-mask construction under ``vmap``: not needed (framework models build masks from shapes only)."""
    return apply_runtime_patches()["vmap_masking"]


def apply_collator_patches(empty_batches: bool = True) -> str:
    """Empty Poisson batches in collators: handled by ``alignment.data`` collators themselves."""
    return apply_runtime_patches()["empty_batches"]


def apply_grouped_mm_patches(vmap_grouped_mm: bool = True) -> str:
    """Grouped expert GEMMs under ``vmap``: not needed (they are called outside ``vmap``)."""
    return apply_runtime_patches()["vmap_grouped_mm"]


def supported_inplace_families() -> list[str]:
    return sorted(set(inplace.INPLACE_FAMILIES) | set(inplace._FAMILY_APPLY))


__all__ = ["apply_checkpoint_patch", "apply_collator_patches", "apply_grouped_mm_patches", "apply_masking_patches", "is_checkpoint_patched",
           "apply_model_patches", "apply_peft_model_patches", "convert_peft_model", "export_peft_adapter", "load_peft_adapter", "peft_adapter_state_dict", "apply_runtime_patches", "apply_transformers_model_patches",
           "inplace", "is_runtime_patched", "kernels", "register_family", "supported_families"]


from .. import __version__  # noqa: E402,F401
from ..utils.namespaces import submodule as _sub  # noqa: E402

# import paths of the reference.  ``torch`` and ``transformers`` are not bound as attributes of this package: the names
# belong to the libraries (``import opaque_b200.patches.torch`` and ``from opaque_b200.patches.transformers import ...`` work).
_sub(__name__, "peft", "LoRA / PEFT entry points.", {"apply_peft_model_patches": apply_peft_model_patches, "convert_peft_model": convert_peft_model,
                                                    "export_peft_adapter": export_peft_adapter, "load_peft_adapter": load_peft_adapter})
_sub(__name__, "torch", "Runtime patches of PyTorch itself (none are needed here).",
     {"apply_checkpoint_patch": apply_checkpoint_patch, "is_checkpoint_patched": is_checkpoint_patched}, bind=False)
_sub(__name__, "transformers", "Hugging Face model adaptation: conversion, in-place patches and the factory API for new families.",
     {**{n: getattr(inplace, n) for n in ("FamilyPatchFn", "ForwardFactory", "ForwardFn", "ModelPatchFn", "ModulePatcher", "family_name",
                                         "make_apply_family_patches", "make_apply_model_patches", "register_activation_kind",
                                         "register_fused_add_rms_kind", "register_moe_kind", "register_rms_norm_kind")},
      "apply_transformers_model_patches": apply_transformers_model_patches, "register_family": register_family,
      "supported_families": supported_families}, bind=False)
_sub(__name__ + ".transformers", "runtime", "Process-wide runtime patches (reported as not needed).",
     {"apply_collator_patches": apply_collator_patches, "apply_grouped_mm_patches": apply_grouped_mm_patches,
      "apply_masking_patches": apply_masking_patches})
_sub(__name__ + ".transformers", "types", "Callable types of the factory API.",
     {n: getattr(inplace, n) for n in ("FamilyPatchFn", "ForwardFactory", "ForwardFn", "ModelPatchFn", "ModulePatcher")}, bind=False)

