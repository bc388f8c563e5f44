"""Fused explicit-batch DP engine (book-keeping ghost clipping) for B200.

One forward / backward per microbatch over an ordinary batched model.  Layers with trainable
parameters are DP-aware autograd functions: their backward computes the input gradient as usual
and, instead of a weight gradient, hands the layer input ``A`` and the output gradient ``G`` to
the active :class:`Capture`:

  * **ghost parameters** (large matrices, embeddings): the tcgen05 ghost-norm kernel adds
    ``‖A_iᵀG_i‖²`` of every example to the microbatch's norm accumulator and ``(A, G)`` are kept
    until the end of the backward pass;
  * **direct parameters** (LoRA factors, biases, norm weights): the per-example gradient is small,
    so it is materialised into one ``[mb, P_direct]`` fp32 buffer (LoRA through the grouped
    tcgen05 weight-gradient kernel, one segment per example).

When backward finishes every example's total squared norm is known: ``c_i = min(1, C/‖g_i‖)``
(guarded), one kernel reduces ``Σ_i c_i·g_i`` of the direct buffer into the gradient and one
clip-weighted tcgen05 GEMM per ghost layer reduces ``Aᵀ·diag(c)·G`` there too (the factor multiplies
each example's partial product in the epilogue).  With several ranks the destination is either the
owners' shards through peer pointers (the launches ARE the reduce-scatter) or a local fp32 buffer that is reduced
once per step — pushed into the owners' shards by one kernel, or pulled out of every rank's buffer in rank order by the
shard step itself; see ``FlatSpace(accumulate=...)``.  After the last
microbatch :class:`~opaque_b200.parallel.ShardedDPOptimizer` adds noise once per coordinate and
applies AdamW-BC on each owner's shard.

Sensitivity.  ``c_i`` is shrunk by ``2⁻⁸ + 2⁻¹²`` relative before use: the ragged GEMM variant applies it
after a round-toward-zero to bf16 and rounds the scaled operand to nearest bf16 (≤ 2⁻⁹ relative), and
the ghost norm carries fp32 accumulation error; the stored contribution of one record therefore
stays within ``C``.  A weight tied between the input embedding and the output head gets its exact
norm (the cross term ``2⟨g_emb, g_head⟩`` is computed from the captured tensors); any other parameter
used more than once in a pass is bounded by ``(Σ‖g_piece‖)²``, an upper bound on its true squared norm,
so clipping stays valid (slightly conservative).

The reference has no counterpart: it materialises per-example gradients with
``vmap(grad)`` (packages/opaque-engine/src/opaque/api/engine/clipping/_clipped_fun.py:207-350) and
all-reduces the sum per leaf (distributed/gradients.py:183-193).
"""
from __future__ import annotations

import contextlib
import dataclasses
import math
from collections.abc import Callable, Mapping
from typing import Any

import torch
from torch.autograd import Function

from .. import ops
from ..parallel.peer import PeerGroup
from ..parallel.sharded import DPStepConfig, FlatSpace, ShardedDPOptimizer
from ..profiling import trace_range
from ..random import RngKey

_ACTIVE: "Capture | None" = None
CLIP_GUARD = 1.0 - 2.0 ** -8 - 2.0 ** -12
LORA_PAD = 64


def current_capture() -> "Capture | None":
    """The active ``Capture`` or ``None``."""
    return _ACTIVE


@contextlib.contextmanager
def activate(cap: "Capture"):
    """Context manager that makes ``capture`` the active one for the DP-aware layers."""
    global _ACTIVE
    prev, _ACTIVE = _ACTIVE, cap
    try:
        yield cap
    finally:
        _ACTIVE = prev


class Capture:
    """Per-microbatch collector of norms and deferred weight-gradient work."""

    MAX_GHOST = 1024

    def __init__(self, engine: "FusedDPEngine", batch_size: int, tokens_per_example: int):
        self.engine = engine
        self.batch_size = batch_size
        self.tokens = tokens_per_example
        dev = engine.device
        sp = engine.space
        self.pe = engine.pe_buffer(batch_size)
        # the norm rows and the segment table are kept per (microbatch, tokens) shape and reused by later microbatches of
        # that shape (one memset instead of an allocation, a fill and an arange); inside a CUDA-graph capture the buffers
        # must belong to the graph, so nothing is shared there
        cache = getattr(engine, "_capture_buffers", None)
        reuse = cache is not None and not (dev.type == "cuda" and torch.cuda.is_current_stream_capturing())
        held = cache.get((batch_size, tokens_per_example)) if reuse else None
        if held is None:
            held = (torch.zeros(self.MAX_GHOST, batch_size, dtype=torch.float32, device=dev),
                    torch.arange(0, (batch_size + 1) * tokens_per_example, tokens_per_example, dtype=torch.int32, device=dev))
            if reuse:
                cache[(batch_size, tokens_per_example)] = held
        else:
            held[0].zero_()
        self.parts, self.seg = held
        self.part_slots: list[str] = []
        self.records: list[tuple] = []
        self.status = engine.status
        self.direct_elems = sp.direct_elems

    # ---- called from layer backward passes --------------------------------------------------
    def _part(self, slot_name: str) -> torch.Tensor:
        i = len(self.part_slots)
        if i >= self.MAX_GHOST:
            raise RuntimeError("too many ghost captures in one backward pass")
        self.part_slots.append(slot_name)
        return self.parts[i]

    def add_linear(self, weight: torch.nn.Parameter, x2d: torch.Tensor, g2d: torch.Tensor) -> None:
        slot = self.engine.slot_of(weight)
        path = NORM_PATH if NORM_PATH != "auto" else ops.pick_norm_path(self.tokens, x2d.shape[1], g2d.shape[1])
        if path == "direct" and self.tokens % 64 == 0 and x2d.shape[0] == self.batch_size * self.tokens \
                and x2d.stride(1) == 1 and g2d.stride(1) == 1:
            # long sequences on a small layer: the per-example product itself is cheaper than the two Gram matrices
            ops.direct_norm2(x2d, g2d, self._part(slot.name), self.tokens, status=self.status)
        else:
            ops.ghost_norm(x2d, g2d, self._part(slot.name), self.tokens, status=self.status)
        self.records.append(("linear", slot, g2d, x2d))

    def add_embedding(self, weight: torch.nn.Parameter, ids: torch.Tensor, g2d: torch.Tensor) -> None:
        slot = self.engine.slot_of(weight)
        ops.ghost_norm(None, g2d, self._part(slot.name), self.tokens, ids=ids.reshape(-1).to(torch.int32),
                       status=self.status)
        self.records.append(("embedding", slot, g2d, ids.reshape(-1).to(torch.int64)))

    def add_grouped_linear(self, weight: torch.nn.Parameter, a_rows: torch.Tensor, g_rows: torch.Tensor,
                           expert_offs: torch.Tensor, seg: torch.Tensor, example_of_row: torch.Tensor, tokens: int) -> None:
        """Stacked expert weights ``[E, out, in]``: rows sorted by (expert, example).

        ``seg`` delimits the (expert, example) segments for the ragged ghost norm; ``expert_offs`` (cumulative row
        ends per expert) delimits the groups of the clip-weighted grouped weight-gradient GEMM.
        """
        slot = self.engine.slot_of(weight)
        E = weight.shape[0]
        seg_out = (torch.arange(seg.numel() - 1, device=seg.device, dtype=torch.int32) % self.batch_size).contiguous()
        ops.ghost_norm(a_rows, g_rows, self._part(slot.name + "#experts"), tokens, seg_offsets=seg, seg_out=seg_out,
                       status=self.status)
        groups = torch.zeros(E + 1, dtype=torch.int32, device=seg.device)
        groups[1:] = expert_offs
        self.records.append(("grouped", slot, g_rows, (a_rows, groups, example_of_row)))

    def pe_view(self, param: torch.nn.Parameter) -> torch.Tensor:
        """``[mb, numel]`` window of the per-example buffer that belongs to ``param``."""
        slot = self.engine.slot_of(param)
        if not slot.direct:
            raise RuntimeError(f"{slot.name} is not a direct parameter")
        return self.pe[:, slot.offset:slot.offset + slot.numel]

    def add_per_example_grad(self, layer: Any, pname: str, grad: torch.Tensor) -> None:
        param = getattr(layer, pname)
        self.pe_view(param).add_(grad.reshape(self.batch_size, -1))

    def add_lora(self, lora_a: torch.nn.Parameter, lora_b: torch.nn.Parameter, x2d: torch.Tensor,
                 xa_pad: torch.Tensor, g2d: torch.Tensor, q_pad: torch.Tensor) -> None:
        """Per-example ``dA_i = q_iᵀ x_i`` (``[r, in]``) and ``dB_i = g_iᵀ (s·xa)_i`` (``[out, r]``)."""
        sa, sb = self.engine.slot_of(lora_a), self.engine.slot_of(lora_b)
        if not (sa.direct and sb.direct):
            raise RuntimeError("LoRA factors must be direct parameters of the flat space")
        r, d_in = lora_a.shape
        stride = self.pe.stride(0)
        ops.wgrad_clip(x2d, q_pad, self.pe, seg_offsets=self.seg, num_groups=self.batch_size, out_offset=sa.offset,
                       ldm=1, ldn=d_in, n_valid=r, accumulate=False, group_stride=stride, block_n=64,
                       status=self.status)
        ops.wgrad_clip(g2d, xa_pad, self.pe, seg_offsets=self.seg, num_groups=self.batch_size, out_offset=sb.offset,
                       ldm=r, ldn=1, n_valid=r, accumulate=False, group_stride=stride, block_n=64,
                       status=self.status)

    def add_lora_qkv(self, factors, x2d: torch.Tensor, xa: torch.Tensor, g_parts, q_all: torch.Tensor) -> None:
        """The three LoRA pairs of one attention block: ``factors = ((A_q, B_q), (A_k, B_k), (A_v, B_v))`` sharing ``x2d``.

        When the flat space holds ``A_q, A_k, A_v`` back to back (it does, see ``FlatSpace``), their per-example
        gradients are ONE launch: ``[q_i | k_i | v_i]ᵀ x_i`` is the ``[3r, in]`` block that starts at ``A_q``'s offset,
        and ``x`` is read once instead of three times.  The ``dB`` products have different left operands and stay separate.
        """
        r, d_in = factors[0][0].shape
        slots = [self.engine.slot_of(a) for a, _ in factors]
        contiguous = all(sl.direct for sl in slots) and all(slots[j + 1].offset == slots[j].offset + r * d_in for j in range(2)) \
            and q_all.is_contiguous() and q_all.shape[1] == 3 * r
        if not contiguous:
            for j, (a, b) in enumerate(factors):
                self.add_lora(a, b, x2d, xa[:, j * r:(j + 1) * r], g_parts[j], q_all[:, j * r:(j + 1) * r])
            return
        stride = self.pe.stride(0)
        ops.wgrad_clip(x2d, q_all, self.pe, seg_offsets=self.seg, num_groups=self.batch_size, out_offset=slots[0].offset,
                       ldm=1, ldn=d_in, n_valid=3 * r, accumulate=False, group_stride=stride, block_n=64, status=self.status)
        for j, (_, b) in enumerate(factors):
            sb = self.engine.slot_of(b)
            if not sb.direct:
                raise RuntimeError("LoRA factors must be direct parameters of the flat space")
            ops.wgrad_clip(g_parts[j], xa[:, j * r:(j + 1) * r], self.pe, seg_offsets=self.seg, num_groups=self.batch_size,
                           out_offset=sb.offset, ldm=r, ldn=1, n_valid=r, accumulate=False, group_stride=stride, block_n=64,
                           status=self.status)

    def _tied_cross_term(self, slot_name: str) -> torch.Tensor | None:
        """``<g_embedding, g_head>`` per example for a weight used as input embedding AND output head.

        With head inputs ``h`` / output gradients ``dlogits`` and embedding output gradients ``e``:
        ``<g_emb, g_head> = sum_{t, t'} dlogits[t', ids[t]] * <e_t, h_t'>`` — one gather and one
        ``T x T x d`` batched product per example.
        """
        lin = [r for r in self.records if r[0] == "linear" and r[1].name == slot_name]
        emb = [r for r in self.records if r[0] == "embedding" and r[1].name == slot_name]
        if len(lin) != 1 or len(emb) != 1:
            return None
        _, _, dlogits, hidden = lin[0]
        _, _, e, ids = emb[0]
        B, T = self.batch_size, self.tokens
        if dlogits.shape[0] != B * T or e.shape[0] != B * T:
            return None
        picked = dlogits.unflatten(0, (B, T)).gather(2, ids.view(B, 1, T).expand(B, T, T))   # [b, t', t]; rows may be padded
        inner = torch.bmm(hidden.view(B, T, -1), e.view(B, T, -1).transpose(1, 2))           # [b, t', t]
        return (picked.float() * inner.float()).sum(dim=(1, 2))

    # ---- after backward -------------------------------------------------------------------------
    @torch.no_grad()
    def _ghost_norm2(self, rows_by_slot: dict[str, list[int]]) -> torch.Tensor:
        """Squared norms contributed by the ghost captures listed in ``rows_by_slot`` (all captures: one slice sum)."""
        norm2 = torch.zeros(self.batch_size, dtype=torch.float32, device=self.engine.device)
        rows_all = sorted(r for rows in rows_by_slot.values() for r in rows)
        if not rows_all:
            return norm2
        if rows_all == list(range(rows_all[0], rows_all[-1] + 1)):
            norm2 += self.parts[rows_all[0]:rows_all[-1] + 1].sum(0)
        else:
            norm2 += self.parts.index_select(0, self.engine.index_tensor(rows_all)).sum(0)
        for name, rows in rows_by_slot.items():
            if len(rows) == 1:
                continue
            cross = self._tied_cross_term(name) if len(rows) == 2 else None
            if cross is not None:     # exact: |a + b|^2 = |a|^2 + |b|^2 + 2<a, b>   (the squares are in the sum above)
                norm2 += 2.0 * cross
            else:                     # (sum of the pieces' norms)^2 bounds the true squared norm
                pieces = torch.stack([self.parts[r] for r in rows])
                norm2 += pieces.clamp_min(0).sqrt().sum(0) ** 2 - pieces.sum(0)
        return norm2

    def finalize(self, clipping_norm: "float | Mapping[str, float]", *, mode: str = "clip",
                 gamma: float = 0.01) -> dict[str, torch.Tensor]:
        """Turn captured norms into clip factors and launch every deferred clip-weighted weight gradient.

        With a mapping ``{group label: C_g}`` each clipping group (labels come from the engine's ``group_of``) is
        clipped on its own norm to its own threshold; the step's sensitivity is then ``sqrt(Σ C_g²)``.
        """
        eng, sp = self.engine, self.engine.space
        by_slot: dict[str, list[int]] = {}
        for i, name in enumerate(self.part_slots):
            by_slot.setdefault(name, []).append(i)
        per_group = isinstance(clipping_norm, Mapping)
        labels = sorted(clipping_norm) if per_group else [""]
        label_of = (lambda slot_name: sp.group_label[slot_name.split("#")[0]]) if per_group else (lambda slot_name: "")
        norms: dict[str, torch.Tensor] = {}
        scales: dict[str, torch.Tensor] = {}
        for g in labels:
            norm2 = self._ghost_norm2({n: r for n, r in by_slot.items() if label_of(n) == g})
            lo, hi = sp.direct_ranges.get(g, (0, 0)) if per_group else (0, self.direct_elems)
            if hi > lo:
                ops.rows_sumsq(self.pe[:, lo:hi], norm2)
            nrm = norm2.clamp_min(0).sqrt()
            C = float(clipping_norm[g]) if per_group else float(clipping_norm)
            c = C / (nrm + gamma) if mode == "auto" else (C / nrm).clamp(max=1.0)
            norms[g] = nrm
            scales[g] = torch.where(torch.isfinite(c), c, torch.zeros_like(c)) * CLIP_GUARD
        tgt = sp.grad_target()
        for g in labels:
            lo, hi = sp.direct_ranges.get(g, (0, 0)) if per_group else (0, self.direct_elems)
            if hi > lo:
                ops.clip_weighted_sum(self.pe[:, lo:hi], scales[g], tgt["out"], flat_offset=lo,
                                      peer_table=tgt["peer_table"], shard_elems=tgt["shard_elems"])
        if self.records:
            expanded: dict[str, torch.Tensor] = {}

            class _RowScale:                      # per-row factors, formed only for the record kinds that need them
                def __getitem__(_, g: str) -> torch.Tensor:
                    if g not in expanded:
                        expanded[g] = scales[g].repeat_interleave(self.tokens)
                    return expanded[g]
            row_scale = _RowScale()
            for kind, slot, g2d, other in self.records:
                g = label_of(slot.name)
                if kind == "grouped":
                    a_rows, groups, ex_row = other
                    E, d_out, d_in = slot.shape
                    ops.wgrad_clip(g2d, a_rows, tgt["out"], row_scale=scales[g].index_select(0, ex_row.long()),
                                   seg_offsets=groups, num_groups=E, splits=1, out_offset=slot.offset, ldm=d_in, ldn=1,
                                   accumulate=True, group_stride=d_out * d_in, peer_table=tgt["peer_table"],
                                   shard_elems=tgt["shard_elems"], status=self.status)
                elif kind == "linear":
                    if self.tokens % 64 == 0 and self.tokens >= 128 and g2d.shape[0] == self.batch_size * self.tokens:
                        # uniform examples: factor applied per example in the epilogue, operands untouched
                        ops.wgrad_clip_per_example(g2d, other, tgt["out"], ex_scale=scales[g], rows_per_example=self.tokens,
                                                   out_offset=slot.offset, ldm=slot.shape[1], accumulate=True,
                                                   peer_table=tgt["peer_table"], shard_elems=tgt["shard_elems"],
                                                   status=self.status)
                    else:
                        ops.wgrad_clip(g2d, other, tgt["out"], row_scale=row_scale[g], out_offset=slot.offset,
                                       ldm=slot.shape[1], ldn=1, accumulate=True, peer_table=tgt["peer_table"],
                                       shard_elems=tgt["shard_elems"], status=self.status)
                else:
                    ops.embedding_wgrad(g2d, other, tgt["out"], row_scale=row_scale[g], flat_offset=slot.offset,
                                        peer_table=tgt["peer_table"], shard_elems=tgt["shard_elems"])
        self.records = []
        if per_group:
            total = torch.sqrt(sum(n ** 2 for n in norms.values()))
            return {"norms": total, "scales": scales, "group_norms": norms}
        return {"norms": norms[""], "scales": scales[""]}


# ===================================================================================== layer functions

NORM_PATH = "auto"     # per-example norms of weight matrices: "ghost", "direct", or "auto" (ops.pick_norm_path per layer)
OWN_GEMM = True        # forward / data-gradient products of linear layers run on this library's tcgen05 GEMMs


def _own_gemm_ok(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> bool:
    """True when ``x Wᵀ`` (and ``dY W``) can run on the library's GEMM: bf16 CUDA operands whose rows TMA can address."""
    return (OWN_GEMM and x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.ndim == 2
            and weight.stride(1) == 1 and weight.stride(0) % 8 == 0 and weight.shape[0] % 8 == 0 and weight.shape[1] % 8 == 0
            and (weight.data_ptr() & 15) == 0 and (bias is None or (bias.dtype == torch.bfloat16 and bias.is_contiguous()))
            and ops.functional.kernels_enabled())


def _rows(x: torch.Tensor) -> torch.Tensor:
    """``x`` as a ``[rows, features]`` matrix with contiguous, 16-byte aligned rows."""
    x2d = x.reshape(-1, x.shape[-1])
    if x2d.stride(1) != 1 or x2d.stride(0) % 8 or (x2d.data_ptr() & 15):
        x2d = x2d.contiguous()
    return x2d


class _DPLinear(Function):
    """``y = x Wᵀ (+ b)`` with the weight gradient deferred to the capture."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        ctx.save_for_backward(x, weight)
        ctx.bias = bias
        ctx.own = _own_gemm_ok(x, weight, bias)
        if ctx.own:
            return ops.gemm(_rows(x), weight, bias=bias).view(*x.shape[:-1], weight.shape[0])
        return torch.nn.functional.linear(x, weight, bias)

    @staticmethod
    def backward(ctx, gy):
        x, weight = ctx.saved_tensors
        cap = current_capture()
        g2d = gy.reshape(-1, gy.shape[-1])
        g2d = g2d if g2d.is_contiguous() else g2d.contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            dx = ops.gemm(g2d, weight, b_layout="kn").view(x.shape) if ctx.own else gy @ weight
        x2d = x.reshape(-1, x.shape[-1])
        x2d = x2d if x2d.is_contiguous() else x2d.contiguous()
        if cap is None:
            dw = g2d.t() @ x2d
            db = g2d.sum(0) if ctx.bias is not None else None
            return dx, dw, db
        cap.add_linear(weight, x2d, g2d)
        if ctx.bias is not None:
            if g2d.dtype == torch.bfloat16 and g2d.shape[1] % 8 == 0 and g2d.stride(0) % 8 == 0:
                ops.rows_group_sum_(cap.pe_view(ctx.bias), g2d, cap.batch_size)
            else:
                cap.pe_view(ctx.bias).add_(g2d.view(cap.batch_size, cap.tokens, -1).sum(1, dtype=torch.float32))
        return dx, None, None


class _FrozenLinear(Function):
    """``y = x Wᵀ (+ b)`` with frozen ``W``: forward and data gradient on the library's GEMM, no weight gradient."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        ctx.save_for_backward(weight)
        ctx.xshape = x.shape
        return ops.gemm(_rows(x), weight, bias=bias).view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, gy):
        (weight,) = ctx.saved_tensors
        if not ctx.needs_input_grad[0]:
            return None, None, None
        g2d = gy.reshape(-1, gy.shape[-1])
        g2d = g2d if g2d.is_contiguous() else g2d.contiguous()
        return ops.gemm(g2d, weight, b_layout="kn").view(ctx.xshape), None, None


def dp_linear(x: torch.Tensor, weight: torch.nn.Parameter, bias: torch.nn.Parameter | None = None) -> torch.Tensor:
    """``x W^T (+ b)`` whose weight gradient is deferred to the active capture."""
    if weight.requires_grad and x.is_cuda and current_capture() is not None:
        return _DPLinear.apply(x, weight, bias)
    if not weight.requires_grad and (bias is None or not bias.requires_grad) and _own_gemm_ok(x, weight, bias):
        return _FrozenLinear.apply(x, weight, bias)
    return torch.nn.functional.linear(x, weight, bias)


class _GLUUp(Function):
    """Gated-MLP up-projection ``act(x Wgᵀ) * (x Wuᵀ)`` as ONE GEMM launch with the activation in its epilogue.

    Backward: one element-wise pass gives ``dG`` and ``dU`` from the stored pre-activations, and
    ``dX = dG·Wg + dU·Wu`` is ONE two-segment GEMM launch.  Trainable ``Wg`` / ``Wu`` hand ``(x, dG)`` and ``(x, dU)``
    to the capture like any DP linear.
    """

    @staticmethod
    def forward(ctx, x, w_gate, w_up, act):
        x2d = _rows(x)
        h, g, u = ops.gemm_glu(x2d, w_gate, w_up, act=act)
        trainable = w_gate.requires_grad or w_up.requires_grad
        ctx.save_for_backward(g, u, w_gate, w_up, *((x2d,) if trainable else ()))
        ctx.act, ctx.xshape, ctx.trainable = act, x.shape, trainable
        return h.view(*x.shape[:-1], w_gate.shape[0])

    @staticmethod
    def backward(ctx, dh):
        g, u, w_gate, w_up = ctx.saved_tensors[:4]
        inter = g.shape[1]
        d2 = dh.reshape(-1, inter)
        d2 = d2 if d2.is_contiguous() else d2.contiguous()
        dg, du = ops.functional.glu_backward(d2, g, u, ctx.act)
        dx = None
        if ctx.needs_input_grad[0]:
            dx = ops.gemm_pair(dg, w_gate, b_layout="kn", a2=du, b2=w_up, b2_layout="kn").view(ctx.xshape)
        if ctx.trainable:
            x2d = ctx.saved_tensors[4]
            cap = current_capture()
            if cap is None:
                return dx, dg.t() @ x2d, du.t() @ x2d, None
            dgc, duc = dg.contiguous(), du.contiguous()
            if w_gate.requires_grad:
                cap.add_linear(w_gate, x2d, dgc)
            if w_up.requires_grad:
                cap.add_linear(w_up, x2d, duc)
        return dx, None, None, None


def glu_up(x: torch.Tensor, w_gate: torch.nn.Parameter, w_up: torch.nn.Parameter, act: str = "silu") -> torch.Tensor | None:
    """Fused gate/up projection with the gated activation, or ``None`` when the fused kernel does not apply (the caller
    then runs the two projections and the activation separately)."""
    if not (_own_gemm_ok(x, w_gate) and _own_gemm_ok(x, w_up) and w_gate.shape == w_up.shape
            and w_gate.stride(0) == w_up.stride(0)):
        return None
    trainable = w_gate.requires_grad or w_up.requires_grad
    if trainable and (current_capture() is None or w_gate.requires_grad != w_up.requires_grad):
        return None
    return _GLUUp.apply(x, w_gate, w_up, act)


class _GLUMLP(Function):
    """A whole FROZEN gated MLP ``(act(x Wgᵀ) * (x Wuᵀ)) Wdᵀ`` in four launches, forward and backward together.

    Forward: the fused gate/up launch (keeps the bf16 pre-activations) and the down projection.  Backward: the down
    projection's data-gradient GEMM turns its accumulator ``dH`` into ``dG`` and ``dU`` in its epilogue (neither ``h``
    nor ``dH`` is kept or written), and ``dX = dG·Wg + dU·Wu`` is one two-segment launch.  Against the separate
    functions this drops one element-wise pass over ``[T, I]`` tensors and a third of the MLP's saved activations.
    """

    @staticmethod
    def forward(ctx, x, w_gate, w_up, w_down, act):
        x2d = _rows(x)
        h, g, u = ops.gemm_glu(x2d, w_gate, w_up, act=act)
        y = ops.gemm(h, w_down)
        ctx.save_for_backward(g, u, w_gate, w_up, w_down)
        ctx.act, ctx.xshape = act, x.shape
        return y.view(*x.shape[:-1], w_down.shape[0])

    @staticmethod
    def backward(ctx, dy):
        g, u, w_gate, w_up, w_down = ctx.saved_tensors
        d2 = dy.reshape(-1, dy.shape[-1])
        d2 = d2 if d2.is_contiguous() else d2.contiguous()
        dg, du = ops.gemm_glu_bwd(d2, w_down, g, u, act=ctx.act)
        dx = None
        if ctx.needs_input_grad[0]:
            dx = ops.gemm_pair(dg, w_gate, b_layout="kn", a2=du, b2=w_up, b2_layout="kn").view(ctx.xshape)
        return dx, None, None, None, None


# Off: measured on 16384 x 14336 x 4096 (sustained) the fused launch takes 1.92 ms against 1.43 ms for the plain data-gradient
# GEMM + 0.43 ms for the element-wise GLU backward (1.86 ms): the epilogue's row-strided loads of the pre-activations make
# it longer than the tile's main loop.  Kept as a tested option.
FUSE_GLU_MLP = False


def glu_mlp(x: torch.Tensor, w_gate, w_up, w_down, act: str = "silu") -> torch.Tensor | None:
    """The frozen gated MLP as one autograd function, or ``None`` when it does not apply (any of the three weights
    trainable, shapes the kernels do not take): the caller then composes :func:`glu_up` and the down projection."""
    if not FUSE_GLU_MLP or w_gate.requires_grad or w_up.requires_grad or w_down.requires_grad:
        return None
    if not (_own_gemm_ok(x, w_gate) and _own_gemm_ok(x, w_up) and w_gate.shape == w_up.shape
            and w_gate.stride(0) == w_up.stride(0) and w_down.dtype == torch.bfloat16 and w_down.is_contiguous()
            and w_down.shape[1] == w_gate.shape[0] and w_gate.shape[0] % 64 == 0 and w_down.shape[0] % 8 == 0):
        return None
    return _GLUMLP.apply(x, w_gate, w_up, w_down, act)


class _DPEmbedding(Function):
    @staticmethod
    def forward(ctx, ids, weight):
        ctx.save_for_backward(ids, weight)
        return torch.nn.functional.embedding(ids, weight)

    @staticmethod
    def backward(ctx, gy):
        ids, weight = ctx.saved_tensors
        cap = current_capture()
        g2d = gy.reshape(-1, gy.shape[-1])
        g2d = g2d if g2d.is_contiguous() else g2d.contiguous()
        if cap is None:
            dw = torch.zeros_like(weight, dtype=torch.float32).index_add_(0, ids.reshape(-1), g2d.float())
            return None, dw.to(weight.dtype)
        cap.add_embedding(weight, ids, g2d)
        return None, None


def dp_embedding(ids: torch.Tensor, weight: torch.nn.Parameter) -> torch.Tensor:
    """Embedding lookup whose weight gradient is deferred to the active capture."""
    if weight.requires_grad and ids.is_cuda and current_capture() is not None:
        return _DPEmbedding.apply(ids, weight)
    return torch.nn.functional.embedding(ids, weight)


FUSE_LORA_GEMM = True      # LoRA linears run as ONE tcgen05 GEMM (base + low-rank segment) instead of GEMM + addmm


def _lora_gemm_ok(x2d, weight, lora_a, lora_b, bias) -> bool:
    r = lora_a.shape[0]
    return (x2d.is_cuda and x2d.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.is_contiguous()
            and lora_a.dtype == torch.bfloat16 and lora_b.dtype == torch.bfloat16 and lora_b.is_contiguous()
            and r % 8 == 0 and weight.shape[0] % 8 == 0 and weight.shape[1] % 8 == 0
            and (bias is None or bias.dtype == torch.bfloat16))


def _small_gemm(a: torch.Tensor, b: torch.Tensor, layout: str) -> torch.Tensor:
    """Rank-r side product of the LoRA path (``x·Aᵀ`` with ``layout="nk"``, ``g·B`` with ``"kn"``) on the single-CTA
    tcgen05 kernel when the operands qualify, so the adapter path launches no library GEMM either."""
    n = b.shape[0] if layout == "nk" else b.shape[1]
    if (OWN_GEMM and a.is_cuda and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.stride(1) == 1
            and a.stride(0) % 8 == 0 and b.is_contiguous() and n % 8 == 0 and a.shape[1] % 8 == 0 and (a.data_ptr() & 15) == 0
            and (b.data_ptr() & 15) == 0 and ops.functional.kernels_enabled()):
        return ops.gemm(a, b, b_layout=layout, kernel="single")
    return a @ (b.t() if layout == "nk" else b)


class _LoRALinear(Function):
    """``y = x Wᵀ + s·(x Aᵀ) Bᵀ`` with frozen ``W``; per-example ``dA``, ``dB`` go to the capture."""

    @staticmethod
    def forward(ctx, x, weight, bias, lora_a, lora_b, scaling):
        x2d = x.reshape(-1, x.shape[-1])
        x2d = x2d if x2d.is_contiguous() else x2d.contiguous()
        xa = _small_gemm(x2d, lora_a, "nk") * scaling     # s · x Aᵀ, kept for the backward pass
        if FUSE_LORA_GEMM and _lora_gemm_ok(x2d, weight, lora_a, lora_b, bias):
            # one tcgen05 pass: the low-rank product is a second K segment of the same accumulator tile
            y = ops.gemm(x2d, weight, a2=xa, b2=lora_b, bias=bias)
        else:
            y = torch.nn.functional.linear(x2d, weight, bias)
            y.addmm_(xa, lora_b.t())
        ctx.save_for_backward(x2d, xa, weight, lora_a, lora_b)
        ctx.scaling = scaling
        ctx.xshape = x.shape
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, gy):
        x2d, xa, weight, lora_a, lora_b = ctx.saved_tensors
        s = ctx.scaling
        g2d = gy.reshape(-1, gy.shape[-1])
        g2d = g2d if g2d.is_contiguous() else g2d.contiguous()
        q = _small_gemm(g2d, lora_b, "kn") * s                     # [R, r]
        dx = None
        if ctx.needs_input_grad[0]:
            if FUSE_LORA_GEMM and _lora_gemm_ok(g2d, weight, lora_a, lora_b, None):
                dx = ops.gemm_pair(g2d, weight, b_layout="kn", a2=q, b2=lora_a, b2_layout="kn")
            else:
                dx = g2d @ weight
                dx.addmm_(q, lora_a)
            dx = dx.view(ctx.xshape)
        cap = current_capture()
        if cap is None:
            return dx, None, None, (q.t() @ x2d), g2d.t() @ xa, None
        R, r = q.shape
        if r % 8 == 0:
            # rank-r operands go to the kernel as they are: TMA fills the rest of its 64-column box with zeros
            q_op, xa_op = (q if q.is_contiguous() else q.contiguous()), xa
        else:
            q_op = torch.zeros(R, LORA_PAD, dtype=q.dtype, device=q.device)
            q_op[:, :r] = q
            xa_op = torch.zeros(R, LORA_PAD, dtype=xa.dtype, device=xa.device)
            xa_op[:, :r] = xa
        xc = x2d if x2d.is_contiguous() else x2d.contiguous()
        cap.add_lora(lora_a, lora_b, xc, xa_op, g2d, q_op)
        return dx, None, None, None, None, None


GROUP_LORA_QKV = True      # LoRA on q, k and v of one block runs as grouped launches (see _LoRAQKV)


def stacked_weight_view(weights) -> torch.Tensor | None:
    """``[sum(out_i), in]`` view over weights that sit back to back in ONE allocation (see ``fuse_storage``), else None."""
    w0 = weights[0]
    if any(w.ndim != 2 or not w.is_contiguous() or w.shape[1] != w0.shape[1] or w.dtype != w0.dtype for w in weights):
        return None
    ptr = w0.data_ptr()
    for w in weights:
        if w.data_ptr() != ptr or w.untyped_storage().data_ptr() != w0.untyped_storage().data_ptr():
            return None
        ptr += w.numel() * w.element_size()
    return torch.as_strided(w0.detach(), (sum(w.shape[0] for w in weights), w0.shape[1]), (w0.shape[1], 1))


@torch.no_grad()
def fuse_storage(params) -> None:
    """Move the data of several (frozen) 2-D parameters with equal input width into one allocation, back to back, so that
    :func:`stacked_weight_view` can hand them to ONE GEMM launch.  Values are unchanged; nothing else refers to the old
    storage afterwards."""
    rows = sum(p.shape[0] for p in params)
    buf = torch.empty(rows, params[0].shape[1], dtype=params[0].dtype, device=params[0].device)
    lo = 0
    for p in params:
        buf[lo:lo + p.shape[0]].copy_(p.data)
        p.data = buf[lo:lo + p.shape[0]]
        lo += p.shape[0]


class _LoRAQKV(Function):
    """Query, key and value projections of one attention block with LoRA on all three, as grouped launches:

    forward   one rank-``3r`` side product ``x·[Aq;Ak;Av]ᵀ`` and ONE tcgen05 GEMM ``x·[Wq;Wk;Wv]ᵀ`` whose low-rank second
              K segment applies the block-diagonal ``[Bq, Bk, Bv]``;
    backward  one side product ``[dq|dk|dv]·blockdiag(B)``, ONE data-gradient GEMM ``[dq|dk|dv]·[Wq;Wk;Wv] + q·[Aq;Ak;Av]``
              (no three partial ``dx`` tensors to add up), and the per-example factor gradients to the capture.

    Counterpart of packages/opaque-patches/src/opaque/api/patches/kernels/lora.py:582-718 (three projections sharing X).
    """

    @staticmethod
    def forward(ctx, x, w_all, bias_all, scaling, aq, bq, ak, bk, av, bv):
        x2d = _rows(x)
        r = aq.shape[0]
        outs = (bq.shape[0], bk.shape[0], bv.shape[0])
        a_cat = torch.cat([aq, ak, av], dim=0)                                   # [3r, in]
        xa = _small_gemm(x2d, a_cat, "nk") * scaling                             # [R, 3r], kept for the backward pass
        b_block = torch.zeros(sum(outs), 3 * r, dtype=bq.dtype, device=bq.device)
        lo = 0
        for j, (b, n) in enumerate(zip((bq, bk, bv), outs)):
            b_block[lo:lo + n, j * r:(j + 1) * r] = b
            lo += n
        y = ops.gemm_pair(x2d, w_all, a2=xa, b2=b_block, bias=bias_all)
        ctx.save_for_backward(x2d, xa, w_all, a_cat, b_block, aq, bq, ak, bk, av, bv)
        ctx.scaling, ctx.xshape, ctx.outs = scaling, x.shape, outs
        q, k, v = torch.split(y, outs, dim=1)
        lead = x.shape[:-1]
        return q.unflatten(0, lead) if len(lead) > 1 else q, k.unflatten(0, lead) if len(lead) > 1 else k, \
            v.unflatten(0, lead) if len(lead) > 1 else v

    @staticmethod
    def backward(ctx, dq, dk, dv):
        x2d, xa, w_all, a_cat, b_block, aq, bq, ak, bk, av, bv = ctx.saved_tensors
        s, outs = ctx.scaling, ctx.outs
        r = aq.shape[0]
        R = x2d.shape[0]
        g_all = torch.cat([dq.reshape(R, outs[0]), dk.reshape(R, outs[1]), dv.reshape(R, outs[2])], dim=1)     # [R, sum(out)]
        q_all = _small_gemm(g_all, b_block, "kn") * s                            # [R, 3r]: (g_j B_j) s for each projection
        dx = None
        if ctx.needs_input_grad[0]:
            dx = ops.gemm_pair(g_all, w_all, b_layout="kn", a2=q_all, b2=a_cat, b2_layout="kn").view(ctx.xshape)
        cap = current_capture()
        if cap is not None:
            lo, parts = 0, []
            for j in range(3):
                parts.append(g_all[:, lo:lo + outs[j]])
                lo += outs[j]
            cap.add_lora_qkv(((aq, bq), (ak, bk), (av, bv)), x2d, xa, parts, q_all)
            return (dx,) + (None,) * 9
        grads = []
        lo = 0
        for j in range(3):
            g_j = g_all[:, lo:lo + outs[j]]
            lo += outs[j]
            grads += [q_all[:, j * r:(j + 1) * r].t() @ x2d, g_j.t() @ xa[:, j * r:(j + 1) * r]]
        return (dx, None, None, None, *grads)


def lora_qkv(x: torch.Tensor, q_proj, k_proj, v_proj):
    """``(q, k, v)`` of three LoRA-adapted projections sharing ``x`` through the grouped path, or ``None`` when it does not
    apply (different ranks / scalings, weights not stored back to back, biases on only some of them, CPU …)."""
    mods = (q_proj, k_proj, v_proj)
    if not GROUP_LORA_QKV or any(m.lora_A is None for m in mods) or not (x.is_cuda and x.dtype == torch.bfloat16 and ops.functional.kernels_enabled()):
        return None
    r = q_proj.lora_A.shape[0]
    if r % 8 or any(m.lora_A.shape[0] != r or m.scaling != q_proj.scaling or m.weight.requires_grad for m in mods):
        return None
    if any(m.lora_A.dtype != torch.bfloat16 or m.lora_B.dtype != torch.bfloat16 for m in mods):
        return None
    have_bias = [m.bias is not None for m in mods]
    if any(have_bias) and not all(have_bias):
        return None
    w_all = stacked_weight_view([m.weight for m in mods])
    if w_all is None or not _own_gemm_ok(x, w_all):
        return None
    bias_all = torch.cat([m.bias for m in mods]) if all(have_bias) else None
    if bias_all is not None and bias_all.requires_grad:
        return None
    return _LoRAQKV.apply(x, w_all, bias_all, q_proj.scaling, q_proj.lora_A, q_proj.lora_B, k_proj.lora_A, k_proj.lora_B,
                          v_proj.lora_A, v_proj.lora_B)


def lora_linear(x, weight, bias, lora_a, lora_b, scaling: float):
    """Frozen base linear plus LoRA factors; per-example factor gradients go to the active capture."""
    if x.is_cuda and x.dtype == torch.bfloat16 and ops.functional.kernels_enabled():
        return _LoRALinear.apply(x, weight, bias, lora_a, lora_b, scaling)
    y = torch.nn.functional.linear(x, weight, bias)
    return y + scaling * ((x @ lora_a.t()) @ lora_b.t())


# ===================================================================================== engine

@dataclasses.dataclass
class StepResult:
    loss: float
    grad_norm_mean: float
    clip_rate: float
    batch_size: int
    losses: torch.Tensor | None = None
    norms: torch.Tensor | None = None
    group_norms: dict[str, torch.Tensor] | None = None


class FusedDPEngine:
    """Owns the flat space, the capture buffers and the sharded DP optimizer for one model."""

    def __init__(self, model: torch.nn.Module, *, clipping_norm: float, noise_multiplier: float,
                 normalize_by: float, key: RngKey, step_config: DPStepConfig | None = None,
                 microbatch_size: int = 8, group: PeerGroup | None = None, mechanism: dict | None = None,
                 clipping_mode: str = "clip", gamma: float = 0.01,
                 direct: Callable[[str, torch.nn.Parameter], bool] | None = None,
                 group_of: Callable[[str], str] | None = None, adaptive: Any = None, cuda_graph: bool = False,
                 accumulate: str = "auto"):
        """``clipping_norm`` is a float, or ``{label: C_g}`` together with ``group_of(param_name) -> label`` for
        per-group clipping.  ``adaptive`` is an :class:`opaque_b200.dpsgd.clipping.AdaptiveClipState` (quantile
        tracking; its ``clipping_norm`` overrides the argument and is updated after every step from the cluster-wide
        count of clipped examples plus the state's own Gaussian draw)."""
        self.model = model
        self.device = next(model.parameters()).device
        self.group = group or PeerGroup(self.device)
        named = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
        self._named_trainable = named
        self._coverage_checked = False
        self._capture_buffers: dict[tuple[int, int], tuple[torch.Tensor, torch.Tensor]] = {}
        if not named:
            raise ValueError("the model has no trainable parameters")
        if isinstance(clipping_norm, Mapping):
            if group_of is None:
                raise ValueError("per-group clipping needs group_of(param_name) -> label")
            missing = {group_of(n) for n, _ in named} - set(clipping_norm)
            if missing:
                raise ValueError(f"no clipping norm for group(s) {sorted(missing)}")
        self.space = FlatSpace(named, self.group, direct=direct, group_of=group_of if isinstance(clipping_norm, Mapping) else None,
                               accumulate=accumulate)
        self.space.bind()
        self._slot_by_id = {id(p): self.space.slots[n] for n, p in named}
        self.opt = ShardedDPOptimizer(self.space, step_config or DPStepConfig(), key=key, mechanism=mechanism)
        self.clipping_norm, self.noise_multiplier, self.normalize_by = clipping_norm, noise_multiplier, normalize_by
        self.clipping_mode, self.gamma = clipping_mode, gamma
        self.cuda_graph = bool(cuda_graph)
        self._graphs: dict[Any, dict[str, Any]] = {}
        self._index_cache: dict[tuple, torch.Tensor] = {}
        self.adaptive = adaptive
        if adaptive is not None:
            self.clipping_norm = adaptive.clipping_norm.values if hasattr(adaptive.clipping_norm, "values") else adaptive.clipping_norm
        self.microbatch_size = microbatch_size
        self.status = self.group.status
        self._pe: torch.Tensor | None = None
        self.kernel_launches = 0

    def index_tensor(self, rows: list[int]) -> torch.Tensor:
        """Device copy of a small index list, cached (graph capture forbids fresh host-to-device copies)."""
        k = tuple(rows)
        t = self._index_cache.get(k)
        if t is None:
            t = self._index_cache[k] = torch.tensor(rows, dtype=torch.long, device=self.device)
        return t

    def slot_of(self, param: torch.nn.Parameter):
        return self._slot_by_id[id(param)]

    def pe_buffer(self, batch_size: int) -> torch.Tensor:
        width = max(self.space.direct_elems, 4)
        if self._pe is None or self._pe.shape[0] < batch_size:
            self._pe = torch.zeros(max(batch_size, self.microbatch_size), width, dtype=torch.float32,
                                   device=self.device)
        else:
            self._pe[:batch_size].zero_()
        return self._pe[:batch_size]

    def sensitivity(self) -> float:
        """L2 sensitivity of the clipped sum: ``C``, or ``sqrt(Σ C_g²)`` with per-group thresholds."""
        c = self.clipping_norm
        return math.sqrt(sum(float(v) ** 2 for v in c.values())) if isinstance(c, Mapping) else float(c)

    def accumulate(self, loss_fn: Callable[..., torch.Tensor], batch: dict[str, torch.Tensor]) -> StepResult:
        """Forward/backward all microbatches of ``batch`` and reduce clipped sums into the sharded gradient.

        ``loss_fn(**microbatch)`` returns one loss per example (``[mb]``).
        """
        first = next(iter(batch.values()))
        n = first.shape[0]
        losses, norms, group_norms = [], [], []
        for lo in range(0, n, self.microbatch_size):
            sub = {k: v[lo:lo + self.microbatch_size] for k, v in batch.items()}
            mb = next(iter(sub.values())).shape[0]
            if self.cuda_graph and self.adaptive is None and "labels" in sub:
                per_example, out = self._graphed_microbatch(loss_fn, sub, mb)
            else:
                per_example, out = self._microbatch(loss_fn, sub, mb)
            losses.append(per_example)
            norms.append(out["norms"])
            if "group_norms" in out:
                group_norms.append(out["group_norms"])
        if n:
            l_all, n_all = torch.cat(losses), torch.cat(norms)
            res = StepResult(float("nan"), float("nan"), float("nan"), n, l_all, n_all)
            if group_norms:
                res.group_norms = {g: torch.cat([d[g] for d in group_norms]) for g in group_norms[0]}
            return res
        return StepResult(0.0, 0.0, 0.0, 0, None, None)

    def _microbatch(self, loss_fn, sub: dict[str, torch.Tensor], mb: int):
        # rows of one privacy unit: a sequence [T], or several sequences that belong together ([2, T]: a preference pair)
        tokens = math.prod(sub["input_ids"].shape[1:]) if "input_ids" in sub else 1
        cap = Capture(self, mb, tokens)
        if not self._coverage_checked:
            for _, p in self._named_trainable:          # stale gradients of earlier, non-private use would trip the check below
                p.grad = None
        with trace_range("opaque::fused/microbatch"), activate(cap):
            per_example = loss_fn(**sub)
            per_example.sum().backward()
        if not self._coverage_checked:
            # DP-aware layers hand their parameter gradients to the capture and return None to autograd.  A trainable
            # parameter that autograd DID give a gradient was used through a plain op: its summed, unclipped gradient is
            # not part of the norms and would never reach the optimizer, so the first microbatch refuses such a model.
            self._coverage_checked = True
            stray = [n for n, p in self._named_trainable if p.grad is not None]
            if stray:
                raise RuntimeError("these trainable parameters are used outside the DP-aware layers (Linear, Embedding, "
                                   "RMSNorm, LayerNorm, LoRA, MoE experts) and cannot be clipped per example: "
                                   + ", ".join(stray[:8]) + (" ..." if len(stray) > 8 else "")
                                   + "; freeze them or use the reference engine")
        with trace_range("opaque::fused/clip"):
            out = cap.finalize(self.clipping_norm, mode=self.clipping_mode, gamma=self.gamma)
        return per_example.detach().float(), out

    def _graphed_microbatch(self, loss_fn, sub: dict[str, torch.Tensor], mb: int):
        """Replay the microbatch (forward, backward, norms, clip-weighted gradients) as ONE CUDA graph.

        Shapes are made static by padding the microbatch to ``microbatch_size`` rows whose labels are all ignored
        (zero loss, zero gradient, zero clip-weighted contribution).  The first microbatch of a shape runs eagerly
        (it also performs every kernel's one-time set-up), the second is captured and replayed, later ones only
        replay.  Launch-bound models (hundreds of small kernels per layer) stop being limited by the host.
        """
        # static sizes microbatch_size / {1, 2, 4, 8}: a short tail microbatch replays the smallest graph that holds it
        full = min(sz for sz in (max(self.microbatch_size >> k, 1) for k in range(4)) if sz >= mb)
        sig = (full,) + tuple((k, tuple(v.shape[1:]), v.dtype) for k, v in sorted(sub.items()))
        entry = self._graphs.get(sig)
        if entry is None:
            static = {k: torch.zeros((full,) + tuple(v.shape[1:]), dtype=v.dtype, device=v.device) for k, v in sub.items()}
            entry = self._graphs[sig] = {"static": static, "graph": None, "out": None}
        static = entry["static"]
        for k, v in sub.items():
            static[k][:mb].copy_(v)
            if mb < full:
                static[k][mb:].fill_(-100 if k == "labels" else 0)
        if entry["graph"] is None and not entry.get("warm"):
            entry["warm"] = True
            per_example, out = self._microbatch(loss_fn, static, full)
        else:
            if entry["graph"] is None:
                torch.cuda.synchronize(self.device)
                graph = torch.cuda.CUDAGraph()
                before = ops.lib.LAUNCHES
                with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                    entry["out"] = self._microbatch(loss_fn, static, full)
                entry["graph"], entry["launches"] = graph, ops.lib.LAUNCHES - before
                ops.lib.LAUNCHES = before                 # captured, not yet executed
            entry["graph"].replay()
            ops.lib.LAUNCHES += entry["launches"]         # kernels of this library that the replay launched
            per_example, out = entry["out"]
            per_example = per_example.clone()
            out = {k: ({g: t.clone() for g, t in v.items()} if isinstance(v, dict) else v.clone()) for k, v in out.items()}
        per_example = per_example[:mb]
        out = {k: ({g: t[:mb] for g, t in v.items()} if isinstance(v, dict) else v[:mb]) for k, v in out.items()}
        return per_example, out

    def prepare_graphs(self, loss_fn: Callable[..., torch.Tensor], example: dict[str, torch.Tensor]) -> int:
        """Capture the microbatch graph of every static size up front (``example`` gives shapes and dtypes only).

        The dummy rows carry ignored labels, so the passes add exactly zero to the gradient shard.  Without this the
        first occurrence of each tail size pays an eager pass plus a capture in the middle of training.
        """
        if not self.cuda_graph or self.adaptive is not None or "labels" not in example:
            return 0
        done = 0
        for size in sorted({max(self.microbatch_size >> k, 1) for k in range(4)}):
            sub = {}
            for k, v in example.items():
                row = torch.full_like(v[:1], -100) if k == "labels" else torch.zeros_like(v[:1])
                sub[k] = row.expand(size, *v.shape[1:]).contiguous()
            for _ in range(2):                      # eager pass (one-time kernel set-up), then capture + first replay
                self._graphed_microbatch(loss_fn, sub, size)
            done += 1
        return done

    def _adapt(self, res: StepResult) -> None:
        """Quantile-tracking threshold update from the cluster-wide number of clipped examples (one small reduction)."""
        from ..dpsgd.clipping import _updated
        from ..types import PerGroup
        st, used = self.adaptive, self.clipping_norm
        labels = sorted(used) if isinstance(used, Mapping) else [""]
        counts = torch.zeros(len(labels) + 1, dtype=torch.float64, device=self.device)
        if res.batch_size:
            counts[-1] = res.batch_size
            for i, g in enumerate(labels):
                nrm = res.group_norms[g] if isinstance(used, Mapping) else res.norms
                counts[i] = (nrm > float(used[g] if isinstance(used, Mapping) else used)).sum()
        if self.group.world > 1:
            torch.distributed.all_reduce(counts, group=self.group.pg)
        vals = counts.tolist()
        batch = int(vals[-1])
        if isinstance(used, Mapping):
            cur = PerGroup({n: self.space.group_label[n] for n in self.space.slots}, dict(used))
            nxt = _updated(st, cur, dict(zip(labels, vals[:-1])), batch, st.step)
            self.clipping_norm = dict(nxt.values)
            num: Any = dict(zip(labels, vals[:-1]))
        else:
            nxt = _updated(st, float(used), vals[0], batch, st.step)
            self.clipping_norm, cur, num = float(nxt), float(used), vals[0]
        self.adaptive = dataclasses.replace(st, clipping_norm=nxt, step=st.step + 1, _num_clipped=num, _batch_size=batch,
                                            _prev_clipping_norm=cur)

    def step(self, loss_fn: Callable[..., torch.Tensor], batch: dict[str, torch.Tensor], *,
             read_metrics: bool = True) -> StepResult:
        """One DP optimizer step: accumulate, then noise + AdamW-BC on the shards."""
        return self.apply(self.accumulate(loss_fn, batch), read_metrics=read_metrics)

    def apply(self, res: StepResult, *, read_metrics: bool = True) -> StepResult:
        """Second half of :meth:`step`: add noise to the accumulated clipped sum and update the parameters."""
        sens = self.sensitivity()
        sigma = 0.0 if self.noise_multiplier == 0 else self.noise_multiplier * sens
        with trace_range("opaque::fused/shard_step"):
            self.opt.step(noise_std=sigma, normalize_by=self.normalize_by)
        if read_metrics and res.batch_size:
            stats = torch.stack([res.losses.mean(), res.norms.mean(),
                                 (res.norms > sens).float().mean()]).tolist()   # one D2H read
            res.loss, res.grad_norm_mean, res.clip_rate = stats
        if read_metrics or self.group.world > 1:
            # With several ranks the status word is read after EVERY step, also for a rank whose Poisson batch was empty
            # and for callers that skip the metrics: a barrier that gave up made the shard step a no-op on this rank (the
            # kernels check the same word), and the job must stop here instead of training on with diverged replicas.
            self.group.check("fused DP step")
        if self.adaptive is not None:
            self._adapt(res)
        return res

    @torch.no_grad()
    def reset_gradients(self) -> None:
        """Discard everything accumulated since the last optimizer step on ALL ranks (call on every rank).

        Used when an accumulation is abandoned half-way (out of memory agreed on by the cluster) and will be replayed.
        """
        self.group.barrier()                    # peers' reductions into this shard have landed
        self.space.grad.local.zero_()
        if self.space.grad_full is not None:
            self.space.grad_full.zero_()
        self.group.barrier()                    # nobody accumulates again before every shard is clean
