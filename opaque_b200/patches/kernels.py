"""Kernel namespace with the reference's public names (``opaque_rms_norm`` …), backed by ``opaque_b200.ops``.

Parity: packages/opaque-patches/src/opaque/api/patches/kernels/__init__.py and the signatures listed in
rms_norm.py:630, fused_add_rms_norm.py:524, cross_entropy.py:585-681, linear_cross_entropy.py:1071,
rope_embedding.py:754-770, lora.py:1269-1312, moe.py:179.
"""
from __future__ import annotations

import torch

from .. import ops
from ..engine import fused
from ..models.layers import linear_cross_entropy, per_example_token_weights
from ..models.moe import _Experts
from ..ops.functional import (ACTIVATION_GEGLU_APPROX, ACTIVATION_GEGLU_EXACT, ACTIVATION_SWIGLU, selective_log_softmax)


def opaque_rms_norm(x, weight, eps=1e-6, offset=0.0, casting_mode="llama", *, in_place_backward=False, row_mode=None):
    return ops.rms_norm(x, weight, eps, offset, casting_mode)


def opaque_fused_add_rms_norm(x, residual, weight, eps=1e-6, offset=0.0, casting_mode="llama", *, in_place_backward=False):
    return ops.fused_add_rms_norm(x, residual, weight, eps, offset, casting_mode)


def opaque_swiglu(gate, up):
    return ops.swiglu(gate, up)


def opaque_geglu_exact(gate, up):
    return ops.geglu(gate, up, approximate=False)


def opaque_geglu_approx(gate, up):
    return ops.geglu(gate, up, approximate=True)


def opaque_rope(Q, cos, sin):
    """Rotate one tensor ``[B, T, H, D]`` (cos / sin ``[T, D/2]`` fp32 tables)."""
    q, _ = ops.rope_qk(Q, Q[..., :1, :].contiguous(), cos, sin)
    return q


def opaque_rope_qk(Q, K, cos, sin, rope_indices=None):
    return ops.rope_qk(Q, K, cos, sin, rope_indices)


def opaque_slow_rope(Q, cos, sin, rope_indices=None):
    return ops.rope_qk_ref(Q, Q[..., :1, :], cos, sin, rope_indices)[0]


def opaque_cross_entropy_loss(logits, labels, logit_softcapping=0, logit_scaling=0, label_smoothing=0.0):
    """Mean NLL over non-ignored tokens."""
    nll = ops.cross_entropy(logits.reshape(-1, logits.shape[-1]), labels.reshape(-1), logit_softcapping=float(logit_softcapping),
                            logit_scaling=float(logit_scaling), label_smoothing=label_smoothing)
    n = (labels.reshape(-1) != -100).sum().clamp_min(1)
    return nll.sum() / n


def opaque_selective_log_softmax(logits, indices):
    return selective_log_softmax(logits.reshape(-1, logits.shape[-1]), indices.reshape(-1)).view(indices.shape)


def opaque_linear_cross_entropy_loss(hidden_states, weight, labels, ignore_index=-100, logit_softcapping=0,
                                     label_smoothing=0.0, use_token_scaling=False):
    """Mean NLL of ``hidden_states @ weightᵀ`` without materialising logits for ignored rows."""
    if logit_softcapping or label_smoothing or use_token_scaling:
        logits = hidden_states.reshape(-1, hidden_states.shape[-1]) @ weight.t()
        nll = ops.cross_entropy(logits, labels.reshape(-1), ignore_index=ignore_index, logit_softcapping=float(logit_softcapping),
                                label_smoothing=label_smoothing)
        if use_token_scaling:
            nll = nll * torch.exp(-nll).detach()
        return nll.sum() / (labels.reshape(-1) != ignore_index).sum().clamp_min(1)
    lab = labels.reshape(-1)
    w = (lab != ignore_index).float()
    w = w / w.sum().clamp_min(1)
    return linear_cross_entropy(hidden_states.reshape(-1, hidden_states.shape[-1]), weight, lab, w, ignore_index=ignore_index).sum()


def opaque_lora_w(X, W, A, B, scaling):
    """``X Wᵀ + scaling·(X Aᵀ) Bᵀ`` with ``A [r, in]``, ``B [out, r]``."""
    return fused.lora_linear(X, W, None, A, B, scaling)


def opaque_lora_qkv(X, Wq, Aq, Bq, Sq, Wk, Ak, Bk, Sk, Wv, Av, Bv, Sv):
    return (fused.lora_linear(X, Wq, None, Aq, Bq, Sq), fused.lora_linear(X, Wk, None, Ak, Bk, Sk),
            fused.lora_linear(X, Wv, None, Av, Bv, Sv))


def opaque_lora_mlp(X, Wg, Ag, Bg, Sg, Wu, Au, Bu, Su, Wd, Ad, Bd, Sd, activation="swiglu"):
    gate, up = fused.lora_linear(X, Wg, None, Ag, Bg, Sg), fused.lora_linear(X, Wu, None, Au, Bu, Su)
    h = ops.swiglu(gate, up) if activation == "swiglu" else ops.geglu(gate, up, approximate=activation == "geglu_approx")
    return fused.lora_linear(h, Wd, None, Ad, Bd, Sd)


def opaque_moe(x, gate_up_proj, down_proj, top_k_index, top_k_weights, *, grouped=True):
    """Sparse MoE experts: ``x [T, H]``, stacked ``gate_up_proj [E, 2I, H]``, ``down_proj [E, H, I]``."""
    T = x.shape[0]
    return _Experts.apply(x, top_k_index, top_k_weights.to(x.dtype), gate_up_proj, down_proj, 1, T)


opaque_fused_moe = opaque_moe

__all__ = ["ACTIVATION_GEGLU_APPROX", "ACTIVATION_GEGLU_EXACT", "ACTIVATION_SWIGLU", "opaque_cross_entropy_loss",
           "opaque_fused_add_rms_norm", "opaque_fused_moe", "opaque_geglu_approx", "opaque_geglu_exact",
           "opaque_linear_cross_entropy_loss", "opaque_lora_mlp", "opaque_lora_qkv", "opaque_lora_w", "opaque_moe",
           "opaque_rms_norm", "opaque_rope", "opaque_rope_qk", "opaque_selective_log_softmax", "opaque_slow_rope",
           "opaque_swiglu"]
