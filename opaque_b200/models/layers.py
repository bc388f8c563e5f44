"""DP-aware building blocks shared by the model families.

Each module computes an ordinary batched forward.  When a fused-engine capture is active the
trainable parameters' gradients are produced per example (direct parameters) or deferred to the
clip-weighted GEMM (ghost parameters); otherwise the modules behave like their ``torch.nn``
counterparts, so the same model also runs under the vmap reference engine, plain autograd and on
CPU.

Parity: the reference adapts Hugging Face modules with patches
(packages/opaque-patches/src/opaque/api/patches/transformers/components/*.py, peft/components/*.py);
here the modules are owned by the framework and keep HF parameter names so checkpoints interchange.
"""
from __future__ import annotations

import contextlib
import math

import torch
from torch import nn
from torch.autograd import Function

from .. import ops
from ..engine import fused
from ..ops.functional import cross_entropy_fused_, cross_entropy_ref


_ADAPTERS_OFF = 0


@contextlib.contextmanager
def adapters_disabled():
    """Run the enclosed forward passes WITHOUT the LoRA factors: the frozen base model of an adapter-tuned policy, which
    is the reference model of preference optimisation — no second copy of the weights
    (reference: packages/opaque-alignment/src/opaque/api/alignment/dpo/reference/_adapter.py)."""
    global _ADAPTERS_OFF
    _ADAPTERS_OFF += 1
    try:
        yield
    finally:
        _ADAPTERS_OFF -= 1


class Linear(nn.Module):
    """Linear layer with an optional LoRA adapter (PEFT naming: ``lora_A`` ``[r, in]``, ``lora_B`` ``[out, r]``)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, *, dtype=None, device=None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype, device=device)) if bias else None
        self.lora_A: nn.Parameter | None = None
        self.lora_B: nn.Parameter | None = None
        self.scaling = 0.0
        self.reset_parameters()

    def reset_parameters(self, std: float = 0.02) -> None:
        nn.init.normal_(self.weight, mean=0.0, std=std)

    def add_lora(self, r: int, alpha: float, *, freeze_base: bool = True) -> None:
        w = self.weight
        self.lora_A = nn.Parameter(torch.empty(r, self.in_features, dtype=w.dtype, device=w.device))
        self.lora_B = nn.Parameter(torch.zeros(self.out_features, r, dtype=w.dtype, device=w.device))
        nn.init.kaiming_uniform_(self.lora_A, a=math.sqrt(5))
        self.scaling = alpha / r
        if freeze_base:
            self.weight.requires_grad_(False)
            if self.bias is not None:
                self.bias.requires_grad_(False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.lora_A is not None and not _ADAPTERS_OFF:
            return fused.lora_linear(x, self.weight, self.bias, self.lora_A, self.lora_B, self.scaling)
        return fused.dp_linear(x, self.weight, self.bias)


class Embedding(nn.Module):
    def __init__(self, num_embeddings: int, embedding_dim: int, *, dtype=None, device=None):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(num_embeddings, embedding_dim, dtype=dtype, device=device))
        nn.init.normal_(self.weight, std=0.02)

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        return fused.dp_embedding(ids, self.weight)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6, *, offset: float = 0.0, casting_mode: str = "llama",
                 dtype=None, device=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device))
        self.eps, self.offset, self.casting_mode = eps, offset, casting_mode

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None):
        if residual is not None:
            return ops.fused_add_rms_norm(x, residual, self.weight, self.eps, self.offset, self.casting_mode, layer=self)
        return ops.rms_norm(x, self.weight, self.eps, self.offset, self.casting_mode, layer=self)


class _LayerNormDP(Function):
    """LayerNorm whose weight / bias gradients are produced per example for the capture."""

    @staticmethod
    def forward(ctx, x, weight, bias, eps, layer):
        xf = x.float()
        mu = xf.mean(-1, keepdim=True)
        rstd = torch.rsqrt(xf.var(-1, unbiased=False, keepdim=True) + eps)
        xhat = (xf - mu) * rstd
        ctx.save_for_backward(xhat.to(x.dtype), rstd, weight)
        ctx.layer = layer
        ctx.has_bias = bias is not None
        y = xhat * weight.float()
        return (y + bias.float() if bias is not None else y).to(x.dtype)

    @staticmethod
    def backward(ctx, gy):
        xhat, rstd, weight = ctx.saved_tensors
        g = gy.float()
        xh = xhat.float()
        gw = g * weight.float()
        dx = rstd * (gw - gw.mean(-1, keepdim=True) - xh * (gw * xh).mean(-1, keepdim=True))
        cap = fused.current_capture()
        if cap is not None:
            B = cap.batch_size
            cap.add_per_example_grad(ctx.layer, "weight", (g * xh).reshape(B, -1, g.shape[-1]).sum(1))
            if ctx.has_bias:
                cap.add_per_example_grad(ctx.layer, "bias", g.reshape(B, -1, g.shape[-1]).sum(1))
            return dx.to(gy.dtype), None, None, None, None
        flat = g.reshape(-1, g.shape[-1])
        return (dx.to(gy.dtype), (flat * xh.reshape(flat.shape)).sum(0).to(weight.dtype),
                flat.sum(0).to(weight.dtype) if ctx.has_bias else None, None, None)


class LayerNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5, *, bias: bool = True, dtype=None, device=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device))
        if bias:
            self.bias = nn.Parameter(torch.zeros(dim, dtype=dtype, device=device))
        else:
            self.register_parameter("bias", None)          # Cohere: scale only
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and self.weight.dtype == torch.bfloat16 \
                and ops.functional.kernels_enabled():
            return ops.layer_norm(x, self.weight, self.bias, self.eps, layer=self)      # fused kernels, per-example dW/db
        if self.weight.requires_grad and fused.current_capture() is not None:
            return _LayerNormDP.apply(x, self.weight, self.bias, self.eps, self)
        return nn.functional.layer_norm(x, (x.shape[-1],), self.weight, self.bias, self.eps)


class _LinearCrossEntropy(Function):
    """Output head and token cross-entropy in one node; returns ``row_weight · nll`` per row.

    Rows with zero weight or an ignored label are skipped entirely (no logits are formed for them).
    With a frozen head the rows are processed in chunks so at most ``chunk × V`` logits exist; with a
    trainable head the whole microbatch's ``dlogits`` is kept for the ghost norm and the clip GEMM.
    """

    @staticmethod
    def forward(ctx, hidden, weight, labels, row_weight, chunk, ignore_index, softcap=0.0, compact=True):
        R, d = hidden.shape
        V = weight.shape[0]
        out = torch.zeros(R, dtype=torch.float32, device=hidden.device)
        dh = torch.zeros_like(hidden)
        cap = fused.current_capture()
        trainable = weight.requires_grad and cap is not None
        use_kernel = hidden.is_cuda and hidden.dtype == torch.bfloat16
        own = fused._own_gemm_ok(hidden, weight) and hidden.stride(1) == 1 and hidden.stride(0) % 8 == 0

        def head(h):            # logits = h Wᵀ
            return ops.gemm(h, weight) if own else h @ weight.t()

        def head_t(dz):         # dh = dlogits W
            return ops.gemm(dz, weight, b_layout="kn") if own else dz @ weight
        # fused path: the head GEMM's epilogue produces the cross-entropy statistics straight from tensor memory and
        # stores the bf16 logits once; a one-pass kernel turns them into gradients in place
        fused_ce = own and use_kernel
        need_dh = ctx.needs_input_grad[0]

        def head_ce(h, lab, rw):
            """(nll, w·dlogits | None) for the rows ``h``."""
            if fused_ce:
                nll, lse, z = ops.linear_ce_forward(h, weight, lab, ignore_index=ignore_index, softcap=softcap,
                                                    store_logits=need_dh or trainable)
                if z is not None:
                    ops.linear_ce_dlogits_(z, lab, lse, rw, ignore_index=ignore_index, softcap=softcap)
                return nll, z
            z = head(h)
            if use_kernel:
                return cross_entropy_fused_(z, lab, rw, ignore_index=ignore_index, logit_softcapping=softcap), z
            return _ce_grad_ref(z, lab, rw, ignore_index, softcap)
        if trainable:
            nll, logits = head_ce(hidden, labels, row_weight)
            out = nll * row_weight
            dh = head_t(logits)
            ctx.capture_args = (weight, hidden, logits)
        else:
            if not compact or (hidden.is_cuda and torch.cuda.is_current_stream_capturing()):
                # no host-visible row count (graph capture), or the caller knows that nearly every row is scored: run
                # every row (ignored rows give zero loss and gradient) and skip the device-to-host round trip
                idx = None
            else:
                valid = (row_weight != 0) & (labels != ignore_index)
                idx = valid.nonzero(as_tuple=True)[0]
            for lo in range(0, R if idx is None else idx.numel(), chunk):
                if idx is None:                       # contiguous row range: plain slices, no gather / scatter
                    sl = slice(lo, min(lo + chunk, R))
                    h, lab, rw = hidden[sl], labels[sl], row_weight[sl]
                else:
                    rows = idx[lo:lo + chunk]
                    h, lab, rw = hidden.index_select(0, rows), labels.index_select(0, rows), row_weight.index_select(0, rows)
                nll, logits = head_ce(h, lab, rw)
                if idx is None:
                    out[sl] = nll * rw
                    if logits is not None:
                        dh[sl] = head_t(logits).to(dh.dtype)
                else:
                    out.index_copy_(0, rows, nll * rw)
                    if logits is not None:
                        dh.index_copy_(0, rows, head_t(logits).to(dh.dtype))
            ctx.capture_args = None
        ctx.save_for_backward(dh)
        return out

    @staticmethod
    def backward(ctx, g):
        (dh,) = ctx.saved_tensors
        if ctx.capture_args is not None:
            weight, hidden, dlogits = ctx.capture_args
            cap = fused.current_capture()
            # The stored dlogits carry row_weight only; a loss built on top of the per-row NLL (a weighted or pairwise
            # objective) reaches the head's weight gradient through the upstream factor g of every row.  The gradient
            # is sum_r g_r dlogits_r^T h_r, so the factor goes onto the (narrow) hidden rows, not the vocabulary-wide ones.
            hidden = hidden * g.to(hidden.dtype)[:, None]
            cap.add_linear(weight, hidden if hidden.is_contiguous() else hidden.contiguous(), dlogits)
            ctx.capture_args = None
        return dh * g.to(dh.dtype)[:, None], None, None, None, None, None, None, None


def _ce_grad_ref(logits, labels, row_weight, ignore_index, softcap=0.0):
    z = logits.float().detach().requires_grad_(True)
    with torch.enable_grad():
        nll = cross_entropy_ref(z, labels, ignore_index=ignore_index, logit_softcapping=softcap)
        (nll * row_weight).sum().backward()
    return nll.detach(), z.grad.to(logits.dtype)


def linear_cross_entropy(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, row_weight: torch.Tensor,
                         *, chunk: int = 8192, ignore_index: int = -100, softcap: float = 0.0, compact: bool = True) -> torch.Tensor:
    """``row_weight[r] · nll(hidden[r] Wᵀ, labels[r])`` for every row, never keeping full logits when ``W`` is frozen;
    ``softcap`` > 0 applies ``softcap · tanh(logits / softcap)`` before the softmax (Gemma-2 final logit capping).

    ``compact=True`` (frozen head) gathers the scored rows first, which costs one device-to-host read of their count;
    ``compact=False`` runs every row in place — right when the caller already passes (almost) only scored rows."""
    if weight.requires_grad and fused.current_capture() is None and torch.is_grad_enabled():
        # plain autograd (reference engine, non-private training): the head's gradient flows normally
        return ops.cross_entropy(hidden @ weight.t(), labels, ignore_index=ignore_index, logit_softcapping=softcap) * row_weight
    return _LinearCrossEntropy.apply(hidden, weight, labels, row_weight, chunk, ignore_index, softcap, compact)


def per_example_token_weights(labels: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    """``1/count_i`` on the scored tokens of example i (0 elsewhere): per-example mean NLL as a weighted sum."""
    valid = labels != ignore_index
    counts = valid.sum(dim=1, keepdim=True).clamp_min(1)
    return valid.float() / counts
