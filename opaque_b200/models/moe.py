"""Mixture-of-experts decoder (Mixtral / Qwen-MoE style): top-k softmax router, stacked SwiGLU experts, shared experts.

Expert weights are stacked as in Hugging Face (``gate_up_proj [E, 2I, H]``, ``down_proj [E, H, I]``) and replicated
across data-parallel ranks.  Tokens are sorted by (expert, example), so that

  * forward / input gradients are ONE launch each of the grouped tcgen05 GEMM over contiguous expert blocks,
  * every (expert, example) pair is a contiguous row segment: the ragged tcgen05 ghost-norm kernel adds
    ``‖A_{e,i}ᵀ G_{e,i}‖²`` to example i's squared norm, and
  * the clip-weighted grouped tcgen05 weight-gradient GEMM (one segment per expert, per-row factor
    ``c_{example(row)}``) reduces ``Σ_i c_i · A_{e,i}ᵀ G_{e,i}`` into the sharded gradient — per-example expert
    gradients are never materialised (the reference materialises ``(B, E, 2I, H)`` through "virtual experts").

Reference counterparts: packages/opaque-patches/src/opaque/api/patches/kernels/{fused_moe.py:48-462, moe.py:49-221,
_grouped_moe.py}, transformers/models/mixtral.py, components/moe.py.
"""
from __future__ import annotations

import dataclasses

import torch
from torch import nn
from torch.autograd import Function

from .. import ops
from ..functional import functional_checkpoint
from ..engine import fused
from .layers import Embedding, Linear, RMSNorm, linear_cross_entropy, per_example_token_weights
from .llama import LlamaAttention, LlamaConfig, LlamaMLP


@dataclasses.dataclass
class MoEConfig:
    vocab_size: int = 151936
    hidden_size: int = 2048
    num_hidden_layers: int = 24
    num_attention_heads: int = 16
    num_key_value_heads: int = 16
    num_experts: int = 60
    moe_intermediate_size: int = 1408
    num_shared_experts: int = 4
    num_experts_per_tok: int = 4
    norm_topk_prob: bool = False
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1000000.0
    rope_scaling: dict | None = None
    dense_layers: tuple = ()                   # indices of layers whose MLP is a plain gated MLP instead of experts
    dense_intermediate_size: int | None = None
    # GPT-OSS: router and expert biases, clamped gate * sigmoid(1.702 gate) * (up + 1) activation, attention sinks,
    # output-projection bias and alternating sliding windows
    router_bias: bool = False
    expert_bias: bool = False
    expert_act: str = "swiglu"                 # swiglu | gpt_oss
    attention_sinks: bool = False
    attention_out_bias: bool = False
    layer_windows: tuple | None = None
    max_position_embeddings: int = 4096
    # family variants: Qwen-MoE has q/k/v biases, a sigmoid gate on the shared expert and its own shared width
    attention_bias: bool = False
    shared_expert_gate: bool = False
    shared_intermediate_size: int | None = None
    head_dim: int | None = None
    qk_norm: bool = False
    qk_norm_after_rope: bool = False

    @property
    def padded_experts(self) -> int:
        return (self.num_experts + 7) // 8 * 8          # router rows padded so gradient rows stay 16-byte aligned

    def attn_config(self) -> LlamaConfig:
        return LlamaConfig(vocab_size=self.vocab_size, hidden_size=self.hidden_size, num_attention_heads=self.num_attention_heads,
                           num_key_value_heads=self.num_key_value_heads, rms_norm_eps=self.rms_norm_eps,
                           rope_theta=self.rope_theta, max_position_embeddings=self.max_position_embeddings,
                           attention_bias=self.attention_bias, head_dim=self.head_dim, qk_norm=self.qk_norm,
                           qk_norm_after_rope=self.qk_norm_after_rope, rope_scaling=self.rope_scaling,
                           attention_sinks=self.attention_sinks, attention_out_bias=self.attention_out_bias,
                           layer_windows=self.layer_windows, num_hidden_layers=self.num_hidden_layers,
                           intermediate_size=self.shared_intermediate_size or self.moe_intermediate_size * max(self.num_shared_experts, 1))

    @staticmethod
    def tiny() -> "MoEConfig":
        return MoEConfig(vocab_size=512, hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=4,
                         num_experts=6, moe_intermediate_size=64, num_shared_experts=1, num_experts_per_tok=2,
                         max_position_embeddings=256)


def grouped_linear(a: torch.Tensor, w: torch.Tensor, offs: torch.Tensor, *, transposed: bool = False) -> torch.Tensor:
    """Rows of group e (``offs[e-1] .. offs[e]``, cumulative ends ``offs [E]``) times expert e's weight.

    ``transposed=False``: ``w [E, N, K]`` and ``out = a @ w[e]ᵀ`` (forward);  ``True``: ``w [E, K, N]`` and
    ``out = a @ w[e]`` (data gradient against the weight as stored).  On the GPU this is one launch of the grouped
    tcgen05 GEMM; elsewhere a loop over experts.
    """
    K = a.shape[1]
    if ops.functional.kernels_enabled() and a.is_cuda and a.dtype == torch.bfloat16 and w.is_contiguous() and a.shape[0] > 0 and K % 8 == 0 \
            and (not transposed or K % 64 == 0) and w.shape[0] <= 256:
        goffs = torch.zeros(offs.numel() + 1, dtype=torch.int32, device=offs.device)
        goffs[1:] = offs
        return ops.gemm(a if a.is_contiguous() else a.contiguous(), w, b_layout="kn" if transposed else "nk", group_offs=goffs)
    out = a.new_zeros(a.shape[0], w.shape[2] if transposed else w.shape[1])
    lo = 0
    for e, hi in enumerate(offs.tolist()):
        if hi > lo:
            out[lo:hi] = a[lo:hi] @ (w[e] if transposed else w[e].t())
        lo = hi
    return out


def route_sort(topk_idx: torch.Tensor, num_experts: int, batch: int, tokens: int):
    """Sort the ``T·k`` (token, expert) assignments by (expert, example).

    Returns ``token_sorted`` (token id of each sorted row), ``slot_sorted`` (position in ``[T·k]``), cumulative
    per-expert row offsets ``offs [E]`` (int32) and the (expert, example) segment table ``seg [E·B + 1]`` (int32).
    """
    T, k = topk_idx.shape
    flat_e = topk_idx.reshape(-1)
    token_of = torch.arange(T, device=topk_idx.device).repeat_interleave(k)
    key = flat_e * batch + token_of // tokens
    order = torch.argsort(key, stable=True)
    # scatter-add instead of bincount: bincount reads the maximum back to the host, which a graph capture cannot do
    counts = torch.zeros(num_experts * batch, dtype=torch.int64, device=key.device).scatter_add_(0, key, torch.ones_like(key))
    seg = torch.zeros(num_experts * batch + 1, dtype=torch.int32, device=topk_idx.device)
    seg[1:] = counts.cumsum(0)
    offs = seg[batch::batch].contiguous()
    return token_of[order], order, offs, seg


class _Experts(Function):
    @staticmethod
    def forward(ctx, x, topk_idx, topk_w, w1, w2, batch, tokens):
        T, H = x.shape
        E, two_i, _ = w1.shape
        I = two_i // 2
        token_sorted, slot_sorted, offs, seg = route_sort(topk_idx, E, batch, tokens)
        xs = x.index_select(0, token_sorted)
        h = grouped_linear(xs, w1, offs)
        act = ops.swiglu(h[:, :I], h[:, I:])
        y = grouped_linear(act, w2, offs)
        wrow = topk_w.reshape(-1).index_select(0, slot_sorted).to(y.dtype)
        out = torch.zeros_like(x).index_add_(0, token_sorted, y * wrow[:, None])
        ctx.save_for_backward(xs, h, act, y, wrow, token_sorted, slot_sorted, offs, seg, w1, w2)
        ctx.meta = (batch, tokens, topk_w.shape)
        return out

    @staticmethod
    def backward(ctx, dout):
        xs, h, act, y, wrow, token_sorted, slot_sorted, offs, seg, w1, w2 = ctx.saved_tensors
        batch, tokens, wshape = ctx.meta
        I = w2.shape[2]
        g = dout.index_select(0, token_sorted)
        dw_rows = (g.float() * y.float()).sum(-1)
        dtopk = torch.zeros(wshape, dtype=torch.float32, device=dout.device).reshape(-1).index_copy_(0, slot_sorted, dw_rows).view(wshape)
        dy = (g * wrow[:, None]).contiguous()
        dact = grouped_linear(dy, w2, offs, transposed=True)
        gate, up = h[:, :I].float(), h[:, I:].float()
        sig = torch.sigmoid(gate)
        silu = gate * sig
        dh = torch.cat([dact.float() * up * sig * (1 + gate * (1 - sig)), dact.float() * silu], dim=1).to(h.dtype)
        dxs = grouped_linear(dh, w1, offs, transposed=True)
        dx = torch.zeros_like(dout).index_add_(0, token_sorted, dxs)
        cap = fused.current_capture()
        if cap is not None:
            ex_row = (token_sorted // tokens).to(torch.int32)
            cap.add_grouped_linear(w1, xs, dh, offs, seg, ex_row, tokens)
            cap.add_grouped_linear(w2, act.contiguous(), dy, offs, seg, ex_row, tokens)
            return dx, None, dtopk.to(wrow.dtype), None, None, None, None
        E = w1.shape[0]
        gw1, gw2 = torch.zeros_like(w1, dtype=torch.float32), torch.zeros_like(w2, dtype=torch.float32)
        lo = 0
        for e, hi in enumerate(offs.tolist()):
            if hi > lo:
                gw1[e] = dh[lo:hi].float().t() @ xs[lo:hi].float()
                gw2[e] = dy[lo:hi].float().t() @ act[lo:hi].float()
            lo = hi
        return dx, None, dtopk.to(wrow.dtype), gw1.to(w1.dtype), gw2.to(w2.dtype), None, None


class _GroupedFrozenLinear(Function):
    """``rows of group e @ w[e]ᵀ`` for frozen expert weights ``w [E, N, K]``: two grouped-GEMM launches, forward and data
    gradient (against the weight as stored); no weight gradient."""

    @staticmethod
    def forward(ctx, a, w, offs):
        ctx.save_for_backward(w, offs)
        return grouped_linear(a, w, offs)

    @staticmethod
    def backward(ctx, dy):
        w, offs = ctx.saved_tensors
        return grouped_linear(dy.contiguous(), w, offs, transposed=True), None, None


class MoEExperts(nn.Module):
    def __init__(self, cfg: MoEConfig, dtype, device):
        super().__init__()
        E, I, H = cfg.num_experts, cfg.moe_intermediate_size, cfg.hidden_size
        self.gate_up_proj = nn.Parameter(torch.empty(E, 2 * I, H, dtype=dtype, device=device).normal_(std=0.02))
        self.down_proj = nn.Parameter(torch.empty(E, H, I, dtype=dtype, device=device).normal_(std=0.02))
        self.act = cfg.expert_act
        if cfg.expert_bias:
            self.gate_up_bias = nn.Parameter(torch.zeros(E, 2 * I, dtype=dtype, device=device))
            self.down_bias = nn.Parameter(torch.zeros(E, H, dtype=dtype, device=device))
        else:
            self.gate_up_bias = self.down_bias = None
        if self.act not in ("swiglu", "gpt_oss"):
            raise ValueError(f"unknown expert_act {self.act!r}")

    def forward(self, x2d, topk_idx, topk_w, batch, tokens):
        if ops.functional.kernels_enabled() and self.gate_up_bias is None and self.act == "swiglu":
            return _Experts.apply(x2d, topk_idx, topk_w, self.gate_up_proj, self.down_proj, batch, tokens)
        # biased / clamped experts (GPT-OSS): while they are FROZEN (LoRA on attention) tokens are sorted by expert and the
        # two projections are launches of the grouped GEMM, with the bias rows and the clamped activation as element-wise
        # steps in between; to TRAIN them only the dense form exists (every expert for every token), which the fused
        # engine refuses (they bypass its layers) and the reference engine maps over examples
        if ops.functional.kernels_enabled() and x2d.is_cuda and x2d.dtype == torch.bfloat16 and self._frozen() \
                and self.gate_up_proj.shape[2] % 64 == 0 and self.down_proj.shape[2] % 64 == 0 and self.gate_up_proj.shape[0] <= 256:
            return self._sorted_frozen(x2d, topk_idx, topk_w, batch, tokens)
        return self._dense(x2d, topk_idx, topk_w)

    def _frozen(self) -> bool:
        ps = (self.gate_up_proj, self.down_proj, self.gate_up_bias, self.down_bias)
        return not any(p is not None and p.requires_grad for p in ps)

    def _sorted_frozen(self, x2d, topk_idx, topk_w, batch, tokens):
        """Frozen experts with bias rows and / or the GPT-OSS activation on the grouped GEMM (``k / E`` of the dense form's
        arithmetic).  Gradients flow to the tokens and the routing weights; the expert parameters get none."""
        E, two_i, _ = self.gate_up_proj.shape
        I = two_i // 2
        token_sorted, slot_sorted, offs, _ = route_sort(topk_idx, E, batch, tokens)
        rows = token_sorted.shape[0]
        expert_of_row = torch.searchsorted(offs.to(torch.int64), torch.arange(rows, device=x2d.device), right=True).clamp_(max=E - 1)
        xs = x2d.index_select(0, token_sorted)
        h = _GroupedFrozenLinear.apply(xs, self.gate_up_proj, offs)
        if self.gate_up_bias is not None:
            h = h + self.gate_up_bias.index_select(0, expert_of_row)
        if self.act == "gpt_oss":
            gate, up = h[:, :I].float().clamp(max=7.0), h[:, I:].float().clamp(min=-7.0, max=7.0)
            act = ((up + 1.0) * gate * torch.sigmoid(1.702 * gate)).to(h.dtype)
        else:
            act = ops.swiglu(h[:, :I], h[:, I:])
        y = _GroupedFrozenLinear.apply(act.contiguous(), self.down_proj, offs)
        if self.down_bias is not None:
            y = y + self.down_bias.index_select(0, expert_of_row)
        wrow = topk_w.reshape(-1).index_select(0, slot_sorted).to(y.dtype)
        return torch.zeros_like(x2d).index_add(0, token_sorted, y * wrow[:, None])

    def _dense(self, x2d, topk_idx, topk_w):
        """Plain-PyTorch form for ``plain_torch_ops()`` (the reference engine maps it over examples with ``vmap``, which
        cannot pass through a custom autograd node or data-dependent gathers): every expert is evaluated for every token
        and the routing weights, zero outside the top-k, select the result.  ``E / k`` times the arithmetic of the sorted
        path — a reference, not a fast path."""
        E, two_i, _ = self.gate_up_proj.shape
        I = two_i // 2
        hit = topk_idx.unsqueeze(-1) == torch.arange(E, device=topk_idx.device)                    # [T, k, E]; vmap-safe one-hot
        route = (hit.to(topk_w.dtype) * topk_w.unsqueeze(-1)).sum(-2)                               # [T, E]
        h = torch.einsum("th,efh->tef", x2d, self.gate_up_proj)
        if self.gate_up_bias is not None:
            h = h + self.gate_up_bias
        if self.act == "gpt_oss":
            gate, up = h[..., :I].clamp(max=7.0), h[..., I:].clamp(min=-7.0, max=7.0)
            act = (up + 1.0) * gate * torch.sigmoid(1.702 * gate)
        else:
            act = torch.nn.functional.silu(h[..., :I]) * h[..., I:]
        y = torch.einsum("tei,ehi->teh", act, self.down_proj)
        if self.down_bias is not None:
            y = y + self.down_bias
        return (y * route.unsqueeze(-1).to(y.dtype)).sum(1)


class SparseMoeBlock(nn.Module):
    def __init__(self, cfg: MoEConfig, dtype, device):
        super().__init__()
        self.cfg = cfg
        self.gate = Linear(cfg.hidden_size, cfg.padded_experts, bias=cfg.router_bias, dtype=dtype, device=device)
        self.experts = MoEExperts(cfg, dtype, device)
        self.shared_expert = LlamaMLP(cfg.attn_config(), dtype, device) if cfg.num_shared_experts > 0 else None
        self.shared_expert_gate = Linear(cfg.hidden_size, 8, dtype=dtype, device=device) \
            if cfg.shared_expert_gate and self.shared_expert is not None else None      # row 0 is the gate, rows 1-7 padding

    def forward(self, x):
        B, T, H = x.shape
        cfg = self.cfg
        logits = self.gate(x).float()[..., :cfg.num_experts]
        probs = torch.softmax(logits, dim=-1)
        w, idx = torch.topk(probs, cfg.num_experts_per_tok, dim=-1)
        if cfg.norm_topk_prob:
            w = w / w.sum(-1, keepdim=True)
        y = self.experts(x.reshape(B * T, H), idx.reshape(B * T, -1), w.reshape(B * T, -1).to(x.dtype), B, T).view(B, T, H)
        if self.shared_expert is not None:
            sh = self.shared_expert(x)
            if self.shared_expert_gate is not None:
                sh = sh * torch.sigmoid(self.shared_expert_gate(x)[..., :1].float()).to(sh.dtype)
            y = y + sh
        return y


class MoEDecoderLayer(nn.Module):
    def __init__(self, cfg: MoEConfig, dtype, device, layer_idx: int = 0):
        super().__init__()
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype=dtype, device=device)
        self.self_attn = LlamaAttention(cfg.attn_config(), dtype, device, layer_idx)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype=dtype, device=device)
        if layer_idx in tuple(cfg.dense_layers):
            if not cfg.dense_intermediate_size:
                raise ValueError("dense_layers needs dense_intermediate_size")
            self.mlp = LlamaMLP(dataclasses.replace(cfg.attn_config(), intermediate_size=cfg.dense_intermediate_size), dtype, device)
        else:
            self.mlp = SparseMoeBlock(cfg, dtype, device)

    def forward(self, h, cos, sin, pos):
        h = h + self.self_attn(self.input_layernorm(h), cos, sin, pos)
        return h + self.mlp(self.post_attention_layernorm(h))


class MoEForCausalLM(nn.Module):
    def __init__(self, cfg: MoEConfig, *, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.config = cfg
        self.embed_tokens = Embedding(cfg.vocab_size, cfg.hidden_size, dtype=dtype, device=device)
        self.layers = nn.ModuleList(MoEDecoderLayer(cfg, dtype, device, i) for i in range(cfg.num_hidden_layers))
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype=dtype, device=device)
        self.lm_head = Linear(cfg.hidden_size, cfg.vocab_size, dtype=dtype, device=device)
        cos, sin = ops.rope_tables(cfg.head_dim or cfg.hidden_size // cfg.num_attention_heads, cfg.max_position_embeddings, cfg.rope_theta,
                                   device=device, scaling=cfg.rope_scaling)
        self.register_buffer("rope_cos", cos, persistent=False)
        self.activation_checkpointing = False      # set by the trainer's gradient_checkpointing
        self.register_buffer("rope_sin", sin, persistent=False)

    def hidden_states(self, input_ids, position_ids=None):
        h = self.embed_tokens(input_ids)
        for layer in self.layers:
            if getattr(self, "activation_checkpointing", False) and torch.is_grad_enabled():
                if ops.functional.kernels_enabled():
                    h = torch.utils.checkpoint.checkpoint(layer, h, self.rope_cos, self.rope_sin, position_ids, use_reentrant=False)
                else:
                    h = functional_checkpoint(layer, h, self.rope_cos, self.rope_sin, position_ids)
            else:
                h = layer(h, self.rope_cos, self.rope_sin, position_ids)
        return self.norm(h)

    def forward(self, input_ids, position_ids=None):
        return self.lm_head(self.hidden_states(input_ids, position_ids))

    def token_nll(self, input_ids, labels, position_ids=None):
        """Per-token negative log-likelihood ``[N, T]`` (0 where ignored)."""
        from .llama import _token_nll
        return _token_nll(self, self.lm_head.weight, input_ids, labels, position_ids=position_ids)

    def per_example_loss(self, input_ids, labels, position_ids=None):
        B, T = input_ids.shape
        h = self.hidden_states(input_ids, position_ids).reshape(B * T, -1)
        w = per_example_token_weights(labels).reshape(-1)
        rows = linear_cross_entropy(h, self.lm_head.weight, labels.reshape(-1), w)
        return rows.view(B, T).sum(1)
