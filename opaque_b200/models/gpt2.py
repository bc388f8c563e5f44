"""GPT-2 decoder (LayerNorm, learned positions, GELU MLP, tied input/output embedding).

Parameter names follow Hugging Face ``GPT2LMHeadModel``.  HF stores the projections as ``Conv1D``
(``[in, out]``); here they are ``[out, in]`` linears and :func:`from_hf_state_dict` transposes on load.
The vocabulary is padded to a multiple of 64 rows so that logits rows stay 16-byte aligned for TMA.

Reference counterpart: packages/opaque-patches/src/opaque/api/patches/transformers/models/gpt2.py
(the reference only batchifies and disables the KV cache for this family).
"""
from __future__ import annotations

import dataclasses

import torch
from torch import nn

from .. import ops
from ..functional import functional_checkpoint
from .layers import Embedding, LayerNorm, Linear, linear_cross_entropy, per_example_token_weights


@dataclasses.dataclass
class GPT2Config:
    vocab_size: int = 50257
    n_positions: int = 1024
    n_embd: int = 768
    n_layer: int = 12
    n_head: int = 12
    layer_norm_epsilon: float = 1e-5

    @property
    def padded_vocab(self) -> int:
        return (self.vocab_size + 63) // 64 * 64

    @staticmethod
    def small() -> "GPT2Config":
        return GPT2Config()

    @staticmethod
    def tiny() -> "GPT2Config":
        return GPT2Config(vocab_size=500, n_positions=256, n_embd=128, n_layer=2, n_head=4)


class _SplitHeads(torch.autograd.Function):
    """``[B, T, 3·d]`` → three ``[B, heads, T, d/heads]`` views; the backward writes the three gradients into ONE
    buffer (one gather kernel) instead of three zero-filled full-size tensors that are then added."""

    @staticmethod
    def forward(ctx, qkv, heads):
        B, T, d3 = qkv.shape
        v5 = qkv.view(B, T, 3, heads, d3 // (3 * heads))
        ctx.shape = (B, T, 3, heads, d3 // (3 * heads))
        return tuple(v5[:, :, i].transpose(1, 2) for i in range(3))

    @staticmethod
    def backward(ctx, gq, gk, gv):
        return ops.merge_heads3(gq, gk, gv), None


class GPT2Block(nn.Module):
    def __init__(self, cfg: GPT2Config, dtype, device):
        super().__init__()
        d = cfg.n_embd
        self.nh = cfg.n_head
        self.ln_1 = LayerNorm(d, cfg.layer_norm_epsilon, dtype=dtype, device=device)
        self.attn_c_attn = Linear(d, 3 * d, bias=True, dtype=dtype, device=device)
        self.attn_c_proj = Linear(d, d, bias=True, dtype=dtype, device=device)
        self.ln_2 = LayerNorm(d, cfg.layer_norm_epsilon, dtype=dtype, device=device)
        self.mlp_c_fc = Linear(d, 4 * d, bias=True, dtype=dtype, device=device)
        self.mlp_c_proj = Linear(4 * d, d, bias=True, dtype=dtype, device=device)

    def forward(self, h):
        B, T, d = h.shape
        qkv = self.attn_c_attn(self.ln_1(h))
        if qkv.is_cuda and ops.functional.kernels_enabled():
            q, k, v = _SplitHeads.apply(qkv, self.nh)
        else:                                    # plain views (also what runs under vmap in the reference engine)
            v5 = qkv.view(B, T, 3, self.nh, d // self.nh)
            q, k, v = (v5[:, :, i].transpose(1, 2) for i in range(3))
        o = nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
        h = h + self.attn_c_proj(o.transpose(1, 2).reshape(B, T, d))
        return h + self.mlp_c_proj(ops.activation(self.mlp_c_fc(self.ln_2(h)), "gelu_tanh"))


class GPT2LMHeadModel(nn.Module):
    def __init__(self, cfg: GPT2Config, *, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.config = cfg
        self.wte = Embedding(cfg.padded_vocab, cfg.n_embd, dtype=dtype, device=device)
        self.wpe = Embedding(cfg.n_positions, cfg.n_embd, dtype=dtype, device=device)
        self.h = nn.ModuleList(GPT2Block(cfg, dtype, device) for _ in range(cfg.n_layer))
        self.ln_f = LayerNorm(cfg.n_embd, cfg.layer_norm_epsilon, dtype=dtype, device=device)
        self.activation_checkpointing = False      # set by the trainer's gradient_checkpointing

    def hidden_states(self, input_ids):
        B, T = input_ids.shape
        pos = torch.arange(T, device=input_ids.device).expand(B, T)
        h = self.wte(input_ids) + self.wpe(pos)
        for blk in self.h:
            if getattr(self, "activation_checkpointing", False) and torch.is_grad_enabled():
                h = (torch.utils.checkpoint.checkpoint(blk, h, use_reentrant=False) if ops.functional.kernels_enabled()
                     else functional_checkpoint(blk, h))          # torch.func transforms need the functional form
            else:
                h = blk(h)
        return self.ln_f(h)

    def forward(self, input_ids):
        return self.hidden_states(input_ids) @ self.wte.weight.t()

    def token_nll(self, input_ids, labels):
        """Per-token negative log-likelihood ``[N, T]`` (0 where ignored)."""
        from .llama import _token_nll
        return _token_nll(self, self.wte.weight, input_ids, labels)

    def per_example_loss(self, input_ids, labels):
        B, T = input_ids.shape
        h = self.hidden_states(input_ids).reshape(B * T, -1)
        w = per_example_token_weights(labels).reshape(-1)
        rows = linear_cross_entropy(h, self.wte.weight, labels.reshape(-1), w)
        return rows.view(B, T).sum(1)


def from_hf_state_dict(sd: dict) -> dict:
    """Map a Hugging Face GPT-2 state dict onto this module's names (transposing ``Conv1D`` weights)."""
    out = {}
    for k, v in sd.items():
        k = k.removeprefix("transformer.")
        if k == "lm_head.weight":
            continue
        k = k.replace("attn.c_attn", "attn_c_attn").replace("attn.c_proj", "attn_c_proj")
        k = k.replace("mlp.c_fc", "mlp_c_fc").replace("mlp.c_proj", "mlp_c_proj")
        if k.endswith(".weight") and any(t in k for t in ("attn_c_attn", "attn_c_proj", "mlp_c_fc", "mlp_c_proj")):
            v = v.t().contiguous()
        out[k] = v
    return out
