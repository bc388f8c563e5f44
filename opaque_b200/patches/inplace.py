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


# ------------------------------------------------------------------------------------------------------------------
# Factory API: build in-place patch functions for further families out of registered forward factories.
#
# A *forward factory* takes a module's original bound ``forward`` and returns the replacement (a plain function of the
# same arguments, ``self`` not included).  Kinds are looked up by name, so a family description is data: which class
# plays which role, and which kind of norm / gated activation / experts forward it needs.
#
# Parity: packages/opaque-patches/src/opaque/api/patches/transformers/_factory.py (register_*_kind,
# make_apply_model_patches), _family.py (family_name, make_apply_family_patches), types.py (the callable protocols).

ForwardFn = Any            # a model or component ``forward`` implementation
ForwardFactory = Any       # Callable[[ForwardFn], ForwardFn]
ModulePatcher = Any        # Callable[[module], bool]: applies process-wide patches to an imported modeling module
FamilyPatchFn = Any        # what make_apply_family_patches returns: f(*, performance=True, compat=True, kernels=None, **kw)
ModelPatchFn = Any         # what make_apply_model_patches returns: f(model=None, *, performance=True, compat=True, kernels=None, **kw)


def _bound(fn):
    """Forward factory from one of this module's ``forward(self, ...)`` functions: the original forward stays reachable
    through the instance attribute that :func:`apply_inplace_patches` also uses."""
    def factory(original):
        owner = original.__self__
        if _ORIGINAL not in owner.__dict__:
            object.__setattr__(owner, _ORIGINAL, original)          # where the kernel forwards find their fallback

        def forward(*args, **kwargs):
            return fn(owner, *args, **kwargs)
        return forward
    return factory


_RMS_NORM_KINDS: dict[str, Any] = {"llama": _bound(_rms_forward("llama")), "gemma": _bound(_rms_forward("gemma"))}
_ACTIVATION_KINDS: dict[str, Any] = {"swiglu": _bound(_mlp_forward)}
_FUSED_ADD_RMS_KINDS: dict[str, Any] = {}
_MOE_KINDS: dict[str, Any] = {"swiglu": _bound(_experts_forward)}
_ROLE_KINDS = {"rms_norm": ("rms_norm_kind", _RMS_NORM_KINDS), "mlp": ("activation_kind", _ACTIVATION_KINDS),
               "decoder_layer": ("fused_add_rms_kind", _FUSED_ADD_RMS_KINDS), "experts": ("moe_kind", _MOE_KINDS)}
_PATCHED_FAMILIES: set[str] = set()
_FAMILY_APPLY: dict[str, Any] = {}
_FACTORY_ORIGINAL = "_opaque_b200_factory_original_forward"


def register_rms_norm_kind(name: str, factory) -> None:
    """Register an RMSNorm forward factory under ``name`` (``make_apply_model_patches(rms_norm_kind=name)``)."""
    _RMS_NORM_KINDS[name] = factory


def register_activation_kind(name: str, factory) -> None:
    """Register a gated-MLP forward factory under ``name`` (``make_apply_model_patches(activation_kind=name)``)."""
    _ACTIVATION_KINDS[name] = factory


def register_fused_add_rms_kind(name: str, factory) -> None:
    """Register a decoder-layer forward factory (residual add fused with the norm) under ``name``."""
    _FUSED_ADD_RMS_KINDS[name] = factory


def register_moe_kind(name: str, factory) -> None:
    """Register a routed-experts forward factory under ``name`` (``make_apply_model_patches(moe_kind=name)``)."""
    _MOE_KINDS[name] = factory


def family_name(model: Any) -> str | None:
    """The Hugging Face ``model_type`` of a model (or config), ``None`` when it has none."""
    cfg = getattr(model, "config", model)
    name = cfg.get("model_type") if isinstance(cfg, dict) else getattr(cfg, "model_type", None)
    return name if isinstance(name, str) else None


def make_apply_family_patches(family: str, *patchers, module_path: str | None = None):
    """``apply(*, performance=True, compat=True, kernels=None)`` that runs the process-wide ``patchers`` of a family ONCE
    (each is called with the imported modeling module when ``module_path`` is given, else without arguments)."""
    def apply(*, performance: bool = True, compat: bool = True, kernels: bool | None = None, **kwargs: Any) -> None:
        if family in _PATCHED_FAMILIES or not (performance or compat):
            return
        module = None
        if module_path:
            import importlib
            module = importlib.import_module(module_path)
        for patcher in patchers:
            patcher(module) if module is not None else patcher()
        _PATCHED_FAMILIES.add(family)
    apply.family = family
    return apply


def make_apply_model_patches(*, family: str, family_apply=None, module_path: str | None = None, classes: dict[str, str],
                             activation_kind=None, rms_norm_kind=None, fused_add_rms_kind=None, moe_kind=None):
    """Build ``apply(model=None, *, performance=True, compat=True, kernels=None, **toggles)`` for a family.

    ``classes`` maps a role (``"rms_norm"``, ``"mlp"``, ``"decoder_layer"``, ``"experts"``) to the class NAME that plays it
    in the family's modeling file; each ``*_kind`` is a registered name, a forward factory, or ``None`` (role left alone).
    Applying replaces ``forward`` on every matching module INSTANCE of ``model`` (idempotent); a toggle named after the
    role (``rms_norm=False``, ``mlp=False``, …) skips it.  Returns how many modules of each role were patched.
    """
    chosen = {"rms_norm": rms_norm_kind, "mlp": activation_kind, "decoder_layer": fused_add_rms_kind, "experts": moe_kind}
    resolved: dict[str, Any] = {}
    for role, kind in chosen.items():
        if kind is None or role not in classes:
            continue
        arg, table = _ROLE_KINDS[role]
        if isinstance(kind, str):
            if kind not in table:
                raise ValueError(f"{arg}={kind!r} is not registered; known: {sorted(table)}")
            kind = table[kind]
        resolved[role] = kind

    def apply(model: Any = None, *, performance: bool = True, compat: bool = True, kernels: bool | None = None, **toggles: Any):
        if family_apply is not None:
            family_apply(performance=performance, compat=compat, kernels=kernels)
        counts = {role: 0 for role in resolved}
        if model is None or not performance:
            return counts
        by_class = {classes[role]: role for role in resolved if toggles.get(role, True)}
        for mod in model.modules():
            role = by_class.get(type(mod).__name__)
            if role is None:
                continue
            if _FACTORY_ORIGINAL not in mod.__dict__:
                original = mod.forward
                object.__setattr__(mod, _FACTORY_ORIGINAL, original)
                mod.forward = resolved[role](original)
            counts[role] += 1
        return counts
    apply.family, apply.is_model_patch_fn = family, True
    return apply


def register_inplace_family(name: str, apply_fn) -> None:
    """Make ``apply_model_patches`` route models of ``model_type == name`` to ``apply_fn`` (a function built by
    :func:`make_apply_model_patches`); the model stays a Hugging Face model."""
    _FAMILY_APPLY[name] = apply_fn


def registered_inplace_family(name: str | None):
    return _FAMILY_APPLY.get(name) if name else None


def remove_factory_patches(model: torch.nn.Module) -> int:
    """Undo what functions built by :func:`make_apply_model_patches` did to ``model``; returns the number restored."""
    n = 0
    for mod in model.modules():
        if _FACTORY_ORIGINAL in mod.__dict__:
            mod.__dict__.pop(_FACTORY_ORIGINAL)
            mod.__dict__.pop(_ORIGINAL, None)
            mod.__dict__.pop("forward", None)
            n += 1
    return n


__all__ += ["FamilyPatchFn", "ForwardFactory", "ForwardFn", "ModelPatchFn", "ModulePatcher", "family_name", "make_apply_family_patches",
            "make_apply_model_patches", "register_activation_kind", "register_fused_add_rms_kind", "register_inplace_family",
            "register_moe_kind", "register_rms_norm_kind", "registered_inplace_family", "remove_factory_patches"]
