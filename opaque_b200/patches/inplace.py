"""In-place kernel patches for Hugging Face families that are not converted into this package's own models.

Hybrid linear-attention models (``qwen3_next``, ``qwen3_5_moe``: gated delta-net layers between full-attention layers)
and latent-attention models (``deepseek_v4``) keep their Hugging Face modules; what this package replaces is the forward
of the pieces it has kernels for, instance by instance:

* the plain RMSNorm (``x·rsqrt(mean x² + eps)·(1 + w)`` computed in fp32 for the Qwen families, ``·w`` Llama style for
  DeepSeek) → :func:`opaque_b200.ops.rms_norm`; the gated norm variants stay as they are;
* the gated MLP ``down(act(gate(x))·up(x))`` → fused SwiGLU kernel between the projections;
* the routed experts (``gate_up_proj [E, 2I, d]``, ``down_proj [E, d, I]``) → tokens sorted by expert and two launches
  of the grouped tcgen05 GEMM instead of a Python loop over experts.

A patched forward takes the kernel path only for CUDA bf16 tensors outside ``torch.func`` transforms (the kernels are
explicit-batch autograd functions without batching rules) and calls the original forward otherwise, so a patched model
still runs under the ``vmap(grad)`` reference engine and on the CPU.  RoPE, attention, the delta-net recurrence and the
router are left to Hugging Face.

Parity: packages/opaque-patches/src/opaque/api/patches/transformers/models/{qwen3_next,qwen3_5_moe,deepseek_v4}.py
(which modules of each family are patched) and transformers/_factory.py (instance-level replacement).
"""
from __future__ import annotations

import types
from typing import Any

import torch

from .. import ops

# model_type -> class NAMES inside the family's modeling file and the norm convention
INPLACE_FAMILIES: dict[str, dict[str, Any]] = {
    "qwen3_next": {"rms_norm": "Qwen3NextRMSNorm", "norm_kind": "gemma", "mlp": "Qwen3NextMLP", "experts": "Qwen3NextExperts"},
    "qwen3_5_moe": {"rms_norm": "Qwen3_5MoeRMSNorm", "norm_kind": "gemma", "mlp": "Qwen3_5MoeMLP", "experts": "Qwen3_5MoeExperts"},
    "qwen3_5_moe_text": {"rms_norm": "Qwen3_5MoeRMSNorm", "norm_kind": "gemma", "mlp": "Qwen3_5MoeMLP", "experts": "Qwen3_5MoeExperts"},
    # scaled experts and interleaved partial RoPE are left alone, as in the reference: only the norm is replaced
    "deepseek_v4": {"rms_norm": "DeepseekV4RMSNorm", "norm_kind": "llama", "mlp": None, "experts": None},
}

_ORIGINAL = "_opaque_b200_original_forward"


def _in_transform() -> bool:
    try:
        return torch._C._functorch.peek_interpreter_stack() is not None
    except Exception:      # noqa: BLE001 — private API; without it assume no transform is active
        return False


def _kernel_ok(*tensors: torch.Tensor) -> bool:
    return (ops.functional.kernels_enabled() and not _in_transform()
            and all(t is not None and t.is_cuda and t.dtype == torch.bfloat16 for t in tensors))


def _rms_forward(kind: str):
    def forward(self, x):
        w = self.weight
        eps = float(getattr(self, "eps", getattr(self, "variance_epsilon", 1e-6)))
        if _kernel_ok(x, w) and x.shape[-1] % 8 == 0:
            if kind == "gemma":
                return ops.rms_norm(x, w, eps, 1.0, "gemma")
            return ops.rms_norm(x, w, eps, 0.0, "llama")
        return getattr(self, _ORIGINAL)(x)
    return forward


def _act_name(module) -> str | None:
    cfg = getattr(module, "config", None)
    name = getattr(cfg, "hidden_act", None) if cfg is not None else None
    return name if isinstance(name, str) else None


def _mlp_forward(self, x):
    gp, up, dp = self.gate_proj, self.up_proj, self.down_proj
    if (_act_name(self) == "silu" and gp.bias is None and up.bias is None and _kernel_ok(x, gp.weight, up.weight, dp.weight)
            and gp.weight.shape[0] % 8 == 0):
        return dp(ops.swiglu(gp(x), up(x)))
    return getattr(self, _ORIGINAL)(x)


def _experts_forward(self, hidden_states, top_k_index, top_k_weights):
    w1, w2 = self.gate_up_proj, self.down_proj
    if (hidden_states.ndim == 2 and _act_name(self) in (None, "silu") and _kernel_ok(hidden_states, w1, w2)
            and top_k_index.numel() > 0 and w1.shape[0] <= 256 and w1.shape[2] % 64 == 0 and w2.shape[2] % 64 == 0):
        from ..models.moe import _Experts
        return _Experts.apply(hidden_states, top_k_index, top_k_weights, w1, w2, 1, hidden_states.shape[0])
    return getattr(self, _ORIGINAL)(hidden_states, top_k_index, top_k_weights)


def inplace_families() -> list[str]:
    """Hugging Face ``model_type`` names that are patched in place (not converted)."""
    return sorted(INPLACE_FAMILIES)


def apply_inplace_patches(model: torch.nn.Module, model_type: str | None = None) -> dict[str, int]:
    """Replace the forwards listed above on every matching module INSTANCE of ``model``; returns how many of each kind.

    Idempotent; :func:`remove_inplace_patches` restores the original forwards.
    """
    mtype = model_type or getattr(getattr(model, "config", None), "model_type", None)
    if mtype not in INPLACE_FAMILIES:
        raise ValueError(f"model_type {mtype!r} is not an in-place family; known: {inplace_families()}")
    spec = INPLACE_FAMILIES[mtype]
    table = {spec["rms_norm"]: ("rms_norm", _rms_forward(spec["norm_kind"]))}
    if spec["mlp"]:
        table[spec["mlp"]] = ("mlp", _mlp_forward)
    if spec["experts"]:
        table[spec["experts"]] = ("experts", _experts_forward)
    counts = {"rms_norm": 0, "mlp": 0, "experts": 0}
    for mod in model.modules():
        hit = table.get(type(mod).__name__)
        if hit is None:
            continue
        kind, fn = hit
        if kind == "experts" and not (hasattr(mod, "gate_up_proj") and hasattr(mod, "down_proj")):
            continue
        if not hasattr(mod, _ORIGINAL):
            object.__setattr__(mod, _ORIGINAL, mod.forward)
            mod.forward = types.MethodType(fn, mod)
        counts[kind] += 1
    if not any(counts.values()):
        raise ValueError(f"no module of {mtype!r} matched {sorted(table)}: is this the Hugging Face implementation of the family?")
    return counts


def remove_inplace_patches(model: torch.nn.Module) -> int:
    """Undo :func:`apply_inplace_patches`; returns the number of modules restored."""
    n = 0
    for mod in model.modules():
        if _ORIGINAL in mod.__dict__:
            orig = mod.__dict__.pop(_ORIGINAL)
            mod.__dict__.pop("forward", None)                      # the class's forward is visible again
            if getattr(orig, "__func__", None) is not type(mod).forward:
                mod.forward = orig                                 # the original was itself an instance-level override
            n += 1
    return n


__all__ = ["INPLACE_FAMILIES", "apply_inplace_patches", "inplace_families", "remove_inplace_patches"]
