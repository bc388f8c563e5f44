"""Llama-family decoder (RMSNorm, RoPE, GQA attention, SwiGLU) with per-example losses.

Parameter names follow Hugging Face ``LlamaForCausalLM`` (``model.layers.N.self_attn.q_proj.weight``
…, LoRA factors as ``…q_proj.lora_A`` / ``lora_B``) so safetensors checkpoints and PEFT adapters map
one to one.  Attention runs through PyTorch SDPA (flash kernels) in an explicit-batch layout — the
fused engine needs no vmap, which is what forces eager attention in the reference
(docs/user-guide/huggingface/model-patches.md:128-146).

Reference counterparts: packages/opaque-patches/src/opaque/api/patches/transformers/models/llama.py,
components/{attention,rms_norm,rope,swiglu,cross_entropy}.py, peft/components/{linear,qkv}.py.
"""
from __future__ import annotations

import dataclasses

import torch
from torch import nn

from .. import ops
from ..engine import fused
from ..functional import functional_checkpoint
from .layers import Embedding, LayerNorm, Linear, RMSNorm, linear_cross_entropy, per_example_token_weights


@dataclasses.dataclass
class LlamaConfig:
    vocab_size: int = 128256
    hidden_size: int = 4096
    intermediate_size: int = 14336
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    rms_norm_eps: float = 1e-5
    rope_theta: float = 500000.0
    rope_scaling: dict | None = None      # Hugging Face rope_scaling dictionary (linear / dynamic / llama3 / yarn)
    max_position_embeddings: int = 8192
    tie_word_embeddings: bool = False
    head_dim: int | None = None
    # family variants (Qwen2: q/k/v bias; Qwen3: per-head RMSNorm on q and k; Gemma: GeGLU, (1 + w) norms computed in
    # fp32, embeddings scaled by sqrt(d))
    attention_bias: bool = False
    attention_out_bias: bool = False
    mlp_bias: bool = False
    hidden_act: str = "silu"                 # silu | gelu_pytorch_tanh | gelu
    norm_offset: float = 0.0
    norm_casting: str = "llama"              # llama | gemma
    embedding_scale: float = 1.0
    qk_norm: bool = False
    sliding_window: int | None = None        # accepted when sequences are not longer than the window
    # Granite multipliers and SmolLM3 layers without rotary embedding
    attention_multiplier: float | None = None      # softmax scale (default 1/sqrt(head_dim))
    residual_multiplier: float = 1.0
    logits_scaling: float = 1.0                     # logits are divided by this
    no_rope_layers: tuple[int, ...] | None = None   # per layer: 1 = rotary embedding applied, 0 = not
    # OLMo-2: norms AFTER the sub-layers (h + norm(f(h))) and q/k norms over the whole projection
    post_norm: bool = False
    qk_norm_full: bool = False
    qk_norm_after_rope: bool = False         # HunYuan: the per-head q / k norms follow the rotary embedding
    # Gemma-2/3, OLMo-3, EXAONE-4: per-layer attention windows (None = full attention), norms on both sides of each
    # sub-layer, tanh capping of attention scores and of the final logits, a second rotary base for windowed layers
    layer_windows: tuple | None = None
    sandwich_norm: bool = False
    attn_logit_softcap: float | None = None
    final_logit_softcap: float | None = None
    local_rope_theta: float | None = None
    # GLM-4 / Phi-4-mini: only the first head_dim * factor dimensions rotate.  The kernels rotate pairs (i, i + head_dim/2),
    # so a converted checkpoint has its q / k rows permuted accordingly (patches.rope_row_permutation)
    partial_rotary_factor: float = 1.0
    attention_sinks: bool = False            # GPT-OSS: one learned logit per head joins every softmax and is then dropped
    # Cohere: LayerNorm without bias instead of RMSNorm, and attention and MLP both reading ONE normed input
    # (h + attn(n(h)) + mlp(n(h)))
    norm_type: str = "rms"                   # rms | layernorm
    parallel_block: bool = False

    @property
    def hd(self) -> int:
        return self.head_dim or self.hidden_size // self.num_attention_heads

    @staticmethod
    def llama3_8b() -> "LlamaConfig":
        return LlamaConfig()

    @staticmethod
    def llama32_1b() -> "LlamaConfig":
        return LlamaConfig(hidden_size=2048, intermediate_size=8192, num_hidden_layers=16, num_attention_heads=32,
                           num_key_value_heads=8, tie_word_embeddings=True, head_dim=64)

    @staticmethod
    def tiny(vocab: int = 256) -> "LlamaConfig":
        return LlamaConfig(vocab_size=vocab, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                           num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=256)


_FLASH = {"fn": False}


def _flash_attn():
    """``flash_attn.flash_attn_func`` if the library is installed (it handles score capping and sliding windows inside its
    tiles), else ``None``; outside ``torch.func`` transforms only (it is an autograd function without batching rules)."""
    if _FLASH["fn"] is False:
        try:
            from flash_attn import flash_attn_func
            _FLASH["fn"] = flash_attn_func
        except Exception:      # noqa: BLE001 — optional dependency
            _FLASH["fn"] = None
    if _FLASH["fn"] is None:
        return None
    try:
        if torch._C._functorch.peek_interpreter_stack() is not None:
            return None
    except Exception:      # noqa: BLE001
        pass
    return _FLASH["fn"]


class LlamaAttention(nn.Module):
    def __init__(self, cfg: LlamaConfig, dtype, device, layer_idx: int = 0):
        super().__init__()
        self.scale = cfg.attention_multiplier
        self.use_rope = cfg.no_rope_layers is None or bool(cfg.no_rope_layers[layer_idx])
        d, hd = cfg.hidden_size, cfg.hd
        self.nh, self.nkv, self.hd = cfg.num_attention_heads, cfg.num_key_value_heads, hd
        self.q_proj = Linear(d, self.nh * hd, bias=cfg.attention_bias, dtype=dtype, device=device)
        self.k_proj = Linear(d, self.nkv * hd, bias=cfg.attention_bias, dtype=dtype, device=device)
        self.v_proj = Linear(d, self.nkv * hd, bias=cfg.attention_bias, dtype=dtype, device=device)
        self.o_proj = Linear(self.nh * hd, d, bias=cfg.attention_out_bias, dtype=dtype, device=device)
        self.window = cfg.layer_windows[layer_idx] if cfg.layer_windows is not None else cfg.sliding_window
        self.softcap = cfg.attn_logit_softcap
        self.sinks = nn.Parameter(torch.zeros(self.nh, dtype=dtype, device=device)) if cfg.attention_sinks else None
        self.local_rope = cfg.local_rope_theta is not None and self.window is not None
        self.qk_full = cfg.qk_norm_full
        self.qk_after = cfg.qk_norm_after_rope
        if cfg.qk_norm_full:
            self.q_norm = RMSNorm(self.nh * hd, cfg.rms_norm_eps, dtype=dtype, device=device)
            self.k_norm = RMSNorm(self.nkv * hd, cfg.rms_norm_eps, dtype=dtype, device=device)
        elif cfg.qk_norm:
            self.q_norm = RMSNorm(hd, cfg.rms_norm_eps, offset=cfg.norm_offset, casting_mode=cfg.norm_casting, dtype=dtype, device=device)
            self.k_norm = RMSNorm(hd, cfg.rms_norm_eps, offset=cfg.norm_offset, casting_mode=cfg.norm_casting, dtype=dtype, device=device)
        else:
            self.q_norm = self.k_norm = None

    def forward(self, x, cos, sin, pos):
        B, T, _ = x.shape
        qkv = fused.lora_qkv(x, self.q_proj, self.k_proj, self.v_proj)      # grouped launches when all three carry LoRA
        if qkv is not None:
            q, k, v = qkv
        else:
            q, k, v = self.q_proj(x), self.k_proj(x), self.v_proj(x)
        if self.qk_full:
            q, k = self.q_norm(q), self.k_norm(k)
        q, k = q.view(B, T, self.nh, self.hd), k.view(B, T, self.nkv, self.hd)
        v = v.view(B, T, self.nkv, self.hd)
        if self.q_norm is not None and not self.qk_full and not self.qk_after:
            q, k = self.q_norm(q), self.k_norm(k)
        if self.use_rope:
            if self.local_rope:                       # windowed layers rotate with their own base (tables 2 and 3)
                q, k = ops.rope_qk(q, k, cos[1], sin[1], pos)
            elif isinstance(cos, (tuple, list)):
                q, k = ops.rope_qk(q, k, cos[0], sin[0], pos)
            else:
                q, k = ops.rope_qk(q, k, cos, sin, pos)
        if self.q_norm is not None and self.qk_after:
            q, k = self.q_norm(q), self.k_norm(k)
        flash = _flash_attn() if (self.sinks is None and (self.softcap or (self.window is not None and T > self.window))) else None
        if flash is not None and q.is_cuda and q.dtype == torch.bfloat16 and ops.functional.kernels_enabled() and self.hd % 8 == 0 \
                and self.hd <= 256:
            # capped scores and / or a sliding window longer sequences do not fit: the flash-attention library applies
            # tanh capping and the band mask inside its tiles ([B, T, H, D] in and out: no transposes, no [T, T] scores)
            o = flash(q, k, v, softmax_scale=self.scale if self.scale is not None else self.hd ** -0.5, causal=True,
                      window_size=(self.window - 1, 0) if (self.window is not None and T > self.window) else (-1, -1),
                      softcap=float(self.softcap or 0.0))
            return self.o_proj(o.reshape(B, T, self.nh * self.hd))
        if self.softcap or self.sinks is not None:
            # capped attention scores / attention sinks: no library attention kernel applies tanh between QK^T and the
            # softmax or appends a sink logit, so the scores are formed explicitly ([B, heads, T, T] in fp32) — correct for
            # every length, meant for short ones
            scale = self.scale if self.scale is not None else self.hd ** -0.5
            qh, kh, vh = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
            if self.nkv != self.nh:
                kh = kh.repeat_interleave(self.nh // self.nkv, dim=1)
                vh = vh.repeat_interleave(self.nh // self.nkv, dim=1)
            sc = torch.matmul(qh, kh.transpose(-1, -2)).float() * scale
            if self.softcap:
                sc = self.softcap * torch.tanh(sc / self.softcap)
            idx = torch.arange(T, device=x.device)
            keep = idx[:, None] >= idx[None, :]
            if self.window is not None:
                keep = keep & (idx[:, None] - idx[None, :] < self.window)
            sc = sc.masked_fill(~keep, float("-inf"))
            if self.sinks is not None:
                sink = self.sinks.float().view(1, self.nh, 1, 1).expand(B, self.nh, T, 1)
                probs = torch.softmax(torch.cat([sc, sink], dim=-1), dim=-1)[..., :-1]      # the sink takes mass, adds nothing
            else:
                probs = torch.softmax(sc, dim=-1)
            o = torch.matmul(probs.to(vh.dtype), vh)
        elif self.window is not None and T > self.window:
            # sequences longer than the window: a banded causal mask (key j visible from query i when 0 <= i - j < window).
            # This takes the masked attention path of the library, not the causal flash path; shorter sequences never
            # come here
            idx = torch.arange(T, device=x.device)
            band = (idx[:, None] >= idx[None, :]) & (idx[:, None] - idx[None, :] < self.window)
            o = nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                                           attn_mask=band, enable_gqa=self.nkv != self.nh, scale=self.scale)
        else:
            o = nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                                           is_causal=True, enable_gqa=self.nkv != self.nh, scale=self.scale)
        return self.o_proj(o.transpose(1, 2).reshape(B, T, self.nh * self.hd))


class LlamaMLP(nn.Module):
    def __init__(self, cfg: LlamaConfig, dtype, device):
        super().__init__()
        bias = getattr(cfg, "mlp_bias", False)
        self.gate_proj = Linear(cfg.hidden_size, cfg.intermediate_size, bias=bias, dtype=dtype, device=device)
        self.up_proj = Linear(cfg.hidden_size, cfg.intermediate_size, bias=bias, dtype=dtype, device=device)
        self.down_proj = Linear(cfg.intermediate_size, cfg.hidden_size, bias=bias, dtype=dtype, device=device)
        self.act = getattr(cfg, "hidden_act", "silu")
        if self.act not in ("silu", "gelu_pytorch_tanh", "gelu"):
            raise ValueError(f"unsupported hidden_act {self.act!r}")

    def forward(self, x):
        gp, up_ = self.gate_proj, self.up_proj
        if gp.lora_A is None and up_.lora_A is None and gp.bias is None and up_.bias is None:
            dp = self.down_proj
            if dp.lora_A is None and dp.bias is None:
                # frozen MLP: forward and backward as one function (the GLU backward rides in the down projection's
                # data-gradient epilogue)
                y = fused.glu_mlp(x, gp.weight, up_.weight, dp.weight, self.act)
                if y is not None:
                    return y
            # one GEMM launch for both projections with the gated activation in its epilogue
            h = fused.glu_up(x, gp.weight, up_.weight, self.act)
            if h is not None:
                return self.down_proj(h)
        g, u = self.gate_proj(x), self.up_proj(x)
        if self.act == "silu":
            return self.down_proj(ops.swiglu(g, u))
        return self.down_proj(ops.geglu(g, u, approximate=self.act == "gelu_pytorch_tanh"))


def _make_norm(cfg: LlamaConfig, dtype, device):
    if cfg.norm_type == "layernorm":
        return LayerNorm(cfg.hidden_size, cfg.rms_norm_eps, bias=False, dtype=dtype, device=device)
    if cfg.norm_type != "rms":
        raise ValueError(f"unknown norm_type {cfg.norm_type!r}")
    return RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, offset=cfg.norm_offset, casting_mode=cfg.norm_casting, dtype=dtype, device=device)


class LlamaDecoderLayer(nn.Module):
    def __init__(self, cfg: LlamaConfig, dtype, device, layer_idx: int = 0):
        super().__init__()
        self.res = cfg.residual_multiplier
        nk = dict(offset=cfg.norm_offset, casting_mode=cfg.norm_casting, dtype=dtype, device=device)
        self.post_norm = cfg.post_norm
        self.sandwich = cfg.sandwich_norm
        self.parallel = cfg.parallel_block
        if cfg.parallel_block:
            self.input_layernorm = _make_norm(cfg, dtype, device)
            self.self_attn = LlamaAttention(cfg, dtype, device, layer_idx)
            self.mlp = LlamaMLP(cfg, dtype, device)
            return
        if cfg.sandwich_norm:
            self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, **nk)
            self.pre_feedforward_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, **nk)
            self.post_feedforward_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, **nk)
        elif cfg.post_norm:
            self.post_feedforward_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, **nk)
        else:
            self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, **nk)
        self.self_attn = LlamaAttention(cfg, dtype, device, layer_idx)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, **nk)
        self.mlp = LlamaMLP(cfg, dtype, device)

    @property
    def standard(self) -> bool:
        """Plain pre-norm block (``h += attn(norm(h)); h += mlp(norm(h))`` with RMSNorm and no residual multiplier)."""
        return not (self.parallel or self.sandwich or self.post_norm) and self.res == 1.0

    def forward_carried(self, x, residual, cos, sin, pos):
        """The standard block on a split stream: the hidden state is ``x + residual`` and the sum is only ever formed
        inside the next norm kernel (forward), its two gradient branches only inside that kernel's backward.  Saves the
        four element-wise add launches per block that the plain form costs (two forward, two backward).
        Returns ``(mlp output, residual)``; the caller folds the last pair into the final norm."""
        if residual is None:
            residual = x
            n = self.input_layernorm(x)
        else:
            n, residual = self.input_layernorm(x, residual)
        a = self.self_attn(n, cos, sin, pos)
        n2, residual = self.post_attention_layernorm(a, residual)
        return self.mlp(n2), residual

    def forward(self, h, cos, sin, pos):
        if self.parallel:
            n = self.input_layernorm(h)
            return h + self.self_attn(n, cos, sin, pos) + self.mlp(n)
        if self.sandwich:
            h = h + self.post_attention_layernorm(self.self_attn(self.input_layernorm(h), cos, sin, pos))
            return h + self.post_feedforward_layernorm(self.mlp(self.pre_feedforward_layernorm(h)))
        if self.post_norm:
            h = h + self.post_attention_layernorm(self.self_attn(h, cos, sin, pos))
            return h + self.post_feedforward_layernorm(self.mlp(h))
        if self.res != 1.0:
            h = h + self.res * self.self_attn(self.input_layernorm(h), cos, sin, pos)
            return h + self.res * self.mlp(self.post_attention_layernorm(h))
        h = h + self.self_attn(self.input_layernorm(h), cos, sin, pos)
        return h + self.mlp(self.post_attention_layernorm(h))


class LlamaModel(nn.Module):
    def __init__(self, cfg: LlamaConfig, dtype, device):
        super().__init__()
        self.embed_tokens = Embedding(cfg.vocab_size, cfg.hidden_size, dtype=dtype, device=device)
        self.layers = nn.ModuleList(LlamaDecoderLayer(cfg, dtype, device, i) for i in range(cfg.num_hidden_layers))
        self.norm = _make_norm(cfg, dtype, device)


class LlamaForCausalLM(nn.Module):
    """Causal LM returning one mean next-token loss per example."""

    def __init__(self, cfg: LlamaConfig, *, dtype=torch.bfloat16, device=None, activation_checkpointing: bool = False):
        super().__init__()
        self.config = cfg
        self.model = LlamaModel(cfg, dtype, device)
        self.lm_head = Linear(cfg.hidden_size, cfg.vocab_size, dtype=dtype, device=device)
        if cfg.tie_word_embeddings:
            self.lm_head.weight = self.model.embed_tokens.weight
        cos, sin = ops.rope_tables(cfg.hd, cfg.max_position_embeddings, cfg.rope_theta, device=device, scaling=cfg.rope_scaling,
                                   rotary_dim=int(cfg.hd * cfg.partial_rotary_factor))
        self.register_buffer("rope_cos", cos, persistent=False)
        self.register_buffer("rope_sin", sin, persistent=False)
        if cfg.local_rope_theta is not None:
            lcos, lsin = ops.rope_tables(cfg.hd, cfg.max_position_embeddings, cfg.local_rope_theta, device=device,
                                         rotary_dim=int(cfg.hd * cfg.partial_rotary_factor))
            self.register_buffer("rope_cos_local", lcos, persistent=False)
            self.register_buffer("rope_sin_local", lsin, persistent=False)
        self.activation_checkpointing = activation_checkpointing
        self.ce_chunk = 8192
        # the multiplier is rounded to the parameter dtype once (as Gemma / Granite do), and stays a host scalar
        self._emb_scale = float(torch.tensor(cfg.embedding_scale, dtype=dtype or torch.float32)) if cfg.embedding_scale != 1.0 else 1.0

    # ---- adapters ---------------------------------------------------------------------------
    def add_lora(self, r: int = 16, alpha: float = 32.0, targets=("q_proj", "k_proj", "v_proj", "o_proj")) -> None:
        """Freeze the base model and attach LoRA factors to the named projections."""
        for p in self.parameters():
            p.requires_grad_(False)
        for name, mod in self.named_modules():
            if isinstance(mod, Linear) and name.split(".")[-1] in targets:
                mod.add_lora(r, alpha)
        if {"q_proj", "k_proj", "v_proj"} <= set(targets):
            # frozen q / k / v weights of a block go back to back into one allocation: the three projections (and their data
            # gradients) then run as ONE GEMM launch each
            for layer in self.model.layers:
                att = layer.self_attn
                if att.q_proj.weight.device.type == "cuda":
                    fused.fuse_storage([att.q_proj.weight, att.k_proj.weight, att.v_proj.weight])

    # ---- forward ------------------------------------------------------------------------------
    def hidden_states(self, input_ids: torch.Tensor, position_ids: torch.Tensor | None = None) -> torch.Tensor:
        h = self.model.embed_tokens(input_ids)
        if self._emb_scale != 1.0:
            h = h * self._emb_scale
        cos, sin = self.rope_cos, self.rope_sin
        if self.config.local_rope_theta is not None:           # (global, local) table pairs; windowed layers take the second
            cos, sin = (self.rope_cos, self.rope_cos_local), (self.rope_sin, self.rope_sin_local)
        if (h.is_cuda and ops.functional.kernels_enabled() and isinstance(self.model.norm, RMSNorm)
                and not (self.activation_checkpointing and torch.is_grad_enabled())
                and all(layer.standard for layer in self.model.layers)):
            x, res = h, None
            for layer in self.model.layers:
                x, res = layer.forward_carried(x, res, cos, sin, position_ids)
            h = self.model.norm(x, res)[0] if res is not None else self.model.norm(x)
            return h if self.config.logits_scaling == 1.0 else h / self.config.logits_scaling
        for layer in self.model.layers:
            if self.activation_checkpointing and torch.is_grad_enabled():
                if ops.functional.kernels_enabled():
                    h = torch.utils.checkpoint.checkpoint(layer, h, cos, sin, position_ids, use_reentrant=False)
                else:                                     # torch.func transforms need the functional form
                    h = functional_checkpoint(layer, h, cos, sin, position_ids)
            else:
                h = layer(h, cos, sin, position_ids)
        h = self.model.norm(h)
        return h if self.config.logits_scaling == 1.0 else h / self.config.logits_scaling     # logits = (h / s) Wᵀ

    def forward(self, input_ids, position_ids=None):
        logits = self.lm_head(self.hidden_states(input_ids, position_ids))
        cap = self.config.final_logit_softcap
        return logits if not cap else cap * torch.tanh(logits / cap)

    def token_nll(self, input_ids: torch.Tensor, labels: torch.Tensor, position_ids=None) -> torch.Tensor:
        """Per-token negative log-likelihood ``[N, T]`` (0 where ignored): the building block of sequence log-probabilities
        (preference losses) on the fused engine."""
        return _token_nll(self, self.lm_head.weight, input_ids, labels, float(self.config.final_logit_softcap or 0.0),
                          position_ids=position_ids)

    def per_example_loss(self, input_ids: torch.Tensor, labels: torch.Tensor, position_ids=None, *,
                         scored_suffix: int | None = None) -> torch.Tensor:
        """Mean NLL over each example's scored tokens; ``labels`` are already aligned (−100 = not scored).

        ``scored_suffix = s`` is a promise that only the last ``s`` positions of every sequence carry a label (completion-
        only fine-tuning with a known prompt length, "loss on the last half"): the head and the cross-entropy then run on
        those ``B·s`` rows alone, with static shapes and without reading the number of scored rows back to the host.
        """
        B, T = input_ids.shape
        hs = self.hidden_states(input_ids, position_ids)
        w = per_example_token_weights(labels)
        softcap = float(self.config.final_logit_softcap or 0.0)
        if scored_suffix is not None and 0 < scored_suffix <= T:
            s = int(scored_suffix)
            h = hs[:, T - s:, :].reshape(B * s, -1)
            rows = linear_cross_entropy(h, self.lm_head.weight, labels[:, T - s:].reshape(-1), w[:, T - s:].reshape(-1),
                                        chunk=self.ce_chunk, softcap=softcap, compact=False)
            return rows.view(B, s).sum(1)
        rows = linear_cross_entropy(hs.reshape(B * T, -1), self.lm_head.weight, labels.reshape(-1), w.reshape(-1),
                                    chunk=self.ce_chunk, softcap=softcap)
        return rows.view(B, T).sum(1)


def _token_nll(model, head_weight, input_ids, labels, softcap=0.0, **kw):
    """Per-token NLL ``[N, T]`` (0 where the label is ignored) through the fused head + cross-entropy path."""
    N, T = input_ids.shape
    h = model.hidden_states(input_ids, **kw).reshape(N * T, -1)
    valid = (labels != -100).float().reshape(-1)
    rows = linear_cross_entropy(h, head_weight, labels.reshape(-1), valid, softcap=softcap)
    return rows.view(N, T)


def shift_labels(input_ids: torch.Tensor, loss_fraction: float = 1.0, ignore_index: int = -100) -> torch.Tensor:
    """Next-token labels; only the last ``loss_fraction`` of positions are scored."""
    labels = torch.full_like(input_ids, ignore_index)
    labels[:, :-1] = input_ids[:, 1:]
    if loss_fraction < 1.0:
        T = input_ids.shape[1]
        labels[:, : int(T * (1.0 - loss_fraction))] = ignore_index
    return labels
