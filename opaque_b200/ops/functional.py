"""Differentiable wrappers (``torch.autograd.Function``) of the transformer kernels.

On CUDA bf16 tensors the sm_100a kernels run; on CPU (or other dtypes) the plain PyTorch
reference of the same formula runs, so models built on these ops work everywhere and the
references double as test oracles.

Parity (signatures / semantics): packages/opaque-patches/src/opaque/api/patches/kernels/
rms_norm.py:630, fused_add_rms_norm.py:524, swiglu.py, geglu.py, rope_embedding.py:754-770,
cross_entropy.py:585-681.
"""
from __future__ import annotations

import contextlib
import math
import ctypes

import torch
from torch.autograd import Function

from . import lib

_MODES = {"llama": 0, "gemma": 1, "none": 1}


_PLAIN = 0      # > 0 inside ``plain_torch_ops()``: every op below takes its plain PyTorch path


@contextlib.contextmanager
def plain_torch_ops():
    """Run the model with plain PyTorch ops only (no custom autograd nodes, no kernels of this library).

    Needed under ``torch.func.vmap`` (the reference engine on a GPU) and used by the benchmark's restated-baseline arm.
    """
    global _PLAIN
    _PLAIN += 1
    try:
        yield
    finally:
        _PLAIN -= 1


def kernels_enabled() -> bool:
    return _PLAIN == 0


def _use_kernel(*ts: torch.Tensor) -> bool:
    return _PLAIN == 0 and all(t.is_cuda and t.dtype == torch.bfloat16 for t in ts)


def _param_grad_hook():
    """The fused DP engine's capture callback for small per-example parameter gradients, if active."""
    from ..engine import fused
    return fused.current_capture()


# =============================================================================== RMSNorm

def rms_norm_ref(x, weight, eps=1e-6, offset=0.0, casting_mode="llama", residual=None):
    """fp32 statement of (fused-add) RMSNorm; returns ``y`` or ``(y, s)``."""
    s = x if residual is None else (x.float() + residual.float()).to(x.dtype)
    sf = s.float()
    rstd = torch.rsqrt(sf.pow(2).mean(-1, keepdim=True) + eps)
    n = sf * rstd
    if casting_mode == "llama":
        n = n.to(x.dtype).float()
    y = (n * (offset + weight.float())).to(x.dtype)
    return y if residual is None else (y, s)


class _RMSNorm(Function):
    @staticmethod
    def forward(ctx, x, residual, weight, eps, offset, mode, layer):
        shape = x.shape
        H = shape[-1]
        x2 = x.reshape(-1, H)
        x2 = x2 if x2.is_contiguous() else x2.contiguous()
        r2 = None
        if residual is not None:
            r2 = residual.reshape(-1, H)
            r2 = r2 if r2.is_contiguous() else r2.contiguous()
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        s = torch.empty_like(x2) if r2 is not None else None
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        rc = lib.load().ob_rmsnorm_fwd(x2.data_ptr(), lib.ptr(r2), weight.data_ptr(), y.data_ptr(), lib.ptr(s),
                                       rstd.data_ptr(), rows, H, eps, offset, mode, lib.stream())
        lib.check(rc, "rmsnorm_fwd")
        ctx.save_for_backward(s if s is not None else x2, weight, rstd)
        ctx.meta = (shape, offset, layer, residual is not None)
        if s is not None:
            return y.view(shape), s.view(shape)
        return y.view(shape), None

    @staticmethod
    def backward(ctx, dy, ds):
        xs, weight, rstd = ctx.saved_tensors
        shape, offset, layer, fused_add = ctx.meta
        H = shape[-1]
        dy2 = dy.reshape(-1, H)
        dy2 = dy2 if dy2.is_contiguous() else dy2.contiguous()
        ds2 = None
        if ds is not None:
            ds2 = ds.reshape(-1, H)
            ds2 = ds2 if ds2.is_contiguous() else ds2.contiguous()
        rows = xs.shape[0]
        dx = torch.empty_like(xs)
        cap = _param_grad_hook() if weight.requires_grad else None
        dw_pe, dw = None, None
        n_ex, rows_per = 0, 0
        if cap is not None:
            n_ex, rows_per = cap.batch_size, rows // cap.batch_size
            dw_pe = torch.empty(n_ex, H, dtype=torch.float32, device=xs.device)
        elif weight.requires_grad:
            n_ex, rows_per = 1, rows
            dw_pe = torch.empty(1, H, dtype=torch.float32, device=xs.device)
        direct_pe = cap is not None and layer is not None and H % 8 == 0
        rc = lib.load().ob_rmsnorm_bwd(dy2.data_ptr(), xs.data_ptr(), weight.data_ptr(), rstd.data_ptr(),
                                       lib.ptr(ds2), dx.data_ptr(), None if direct_pe else lib.ptr(dw_pe), None, n_ex, rows_per,
                                       rows, H, offset, lib.stream())
        lib.check(rc, "rmsnorm_bwd")
        if direct_pe:                # 16-byte-vector row sums straight into the capture's per-example buffer
            rows_group_sum_(cap.pe_view(layer.weight), dy2, cap.batch_size, x2d=xs, rstd=rstd)
        elif cap is not None:
            cap.add_per_example_grad(layer, "weight", dw_pe)
        elif dw_pe is not None:
            dw = dw_pe[0].to(weight.dtype)
        dxv = dx.view(shape)
        return dxv, (dxv if fused_add else None), dw, None, None, None, None


def rms_norm(x, weight, eps=1e-6, offset=0.0, casting_mode="llama", *, layer=None):
    """``y = x·rsqrt(mean(x²)+eps)·(offset + w)``."""
    if _use_kernel(x, weight) and x.shape[-1] % 8 == 0:
        return _RMSNorm.apply(x, None, weight, eps, offset, _MODES[casting_mode], layer)[0]
    return rms_norm_ref(x, weight, eps, offset, casting_mode)


def fused_add_rms_norm(x, residual, weight, eps=1e-6, offset=0.0, casting_mode="llama", *, layer=None):
    """``s = x + residual; y = rmsnorm(s)``; returns ``(y, s)``."""
    if _use_kernel(x, residual, weight) and x.shape[-1] % 8 == 0:
        return _RMSNorm.apply(x, residual, weight, eps, offset, _MODES[casting_mode], layer)
    return rms_norm_ref(x, weight, eps, offset, casting_mode, residual=residual)


# =============================================================================== LayerNorm

def rows_group_sum_(out: torch.Tensor, g2d: torch.Tensor, num_examples: int, *, x2d: torch.Tensor | None = None,
                    mean: torch.Tensor | None = None, rstd: torch.Tensor | None = None,
                    out_plain: torch.Tensor | None = None) -> None:
    """``out[e] += Σ_{rows of example e} g`` (or ``g·(x−mean)·rstd`` when statistics are given); ``out`` fp32 ``[B, N]``
    (any row pitch), ``g2d`` bf16 ``[B·T, N]``.  With statistics, ``out_plain`` also receives the plain sums ``Σ g`` of
    the same pass (a LayerNorm's weight and bias gradients in one read of ``g``)."""
    rows, N = g2d.shape
    for o in (out, out_plain):
        if o is not None and (o.dtype != torch.float32 or o.shape != (num_examples, N) or o.stride(1) != 1):
            raise ValueError("rows_group_sum_: out must be fp32 [examples, N]")
    if rows % num_examples:
        raise ValueError("rows_group_sum_: rows must be a multiple of examples")
    mode = 0 if x2d is None else (1 if mean is not None else 2)          # 2: g * x * rstd (RMSNorm weight gradient)
    if mode == 0 and out_plain is not None:
        raise ValueError("rows_group_sum_: out_plain needs x2d (without it, out already is the plain sum)")
    rc = lib.load().ob_rows_group_sum(g2d.data_ptr(), lib.ptr(x2d), lib.ptr(mean), lib.ptr(rstd), num_examples,
                                      rows // num_examples, N, g2d.stride(0), out.data_ptr(), out.stride(0), mode,
                                      lib.ptr(out_plain), 0 if out_plain is None else out_plain.stride(0), lib.stream())
    lib.check(rc, "rows_group_sum")


def merge_heads3(gq: torch.Tensor, gk: torch.Tensor, gv: torch.Tensor) -> torch.Tensor:
    """Three ``[B, heads, T, hd]`` bf16 tensors (any batch / head / token strides, contiguous head vectors) gathered into
    one ``[B, T, 3·heads·hd]`` tensor in ONE launch: the gradient of splitting a fused q/k/v projection into heads."""
    B, H, T, hd = gq.shape
    ok = all(t.is_cuda and t.dtype == torch.bfloat16 and t.shape == gq.shape and t.stride(3) == 1 and
             t.data_ptr() % 16 == 0 and all(s % 8 == 0 for s in t.stride()[:3]) for t in (gq, gk, gv)) and hd % 8 == 0
    out = torch.empty(B, T, 3 * H * hd, dtype=gq.dtype, device=gq.device)
    if not ok or not kernels_enabled():
        v5 = out.view(B, T, 3, H, hd)
        for i, g in enumerate((gq, gk, gv)):
            v5[:, :, i].copy_(g.transpose(1, 2))
        return out
    strides = (ctypes.c_longlong * 9)(*[s for t in (gq, gk, gv) for s in (t.stride(0), t.stride(1), t.stride(2))])
    rc = lib.load().ob_merge_heads3(gq.data_ptr(), gk.data_ptr(), gv.data_ptr(), strides, out.data_ptr(), B, T, H, hd,
                                    lib.sm_count(), lib.stream())
    lib.check(rc, "merge_heads3")
    return out


class _LayerNorm(Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps, layer):
        shape = x.shape
        H = shape[-1]
        x2 = x.reshape(-1, H)
        x2 = x2 if x2.is_contiguous() else x2.contiguous()
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        stats = torch.empty(2, rows, dtype=torch.float32, device=x.device)
        rc = lib.load().ob_layernorm_fwd(x2.data_ptr(), weight.data_ptr(), lib.ptr(bias), y.data_ptr(), stats[0].data_ptr(),
                                         stats[1].data_ptr(), rows, H, eps, lib.stream())
        lib.check(rc, "layernorm_fwd")
        ctx.save_for_backward(x2, weight, stats)
        ctx.meta = (shape, layer, bias is not None)
        return y.view(shape)

    @staticmethod
    def backward(ctx, dy):
        x2, weight, stats = ctx.saved_tensors
        shape, layer, has_bias = ctx.meta
        H = shape[-1]
        dy2 = dy.reshape(-1, H)
        dy2 = dy2 if dy2.is_contiguous() else dy2.contiguous()
        rows = x2.shape[0]
        dx = torch.empty_like(x2)
        rc = lib.load().ob_layernorm_bwd_dx(dy2.data_ptr(), x2.data_ptr(), weight.data_ptr(), stats[0].data_ptr(),
                                            stats[1].data_ptr(), dx.data_ptr(), rows, H, lib.stream())
        lib.check(rc, "layernorm_bwd_dx")
        cap = _param_grad_hook() if weight.requires_grad else None
        dw = db = None
        if cap is not None:                      # per-example gradients straight into the capture's buffer rows
            rows_group_sum_(cap.pe_view(layer.weight), dy2, cap.batch_size, x2d=x2, mean=stats[0], rstd=stats[1],
                            out_plain=cap.pe_view(layer.bias) if has_bias else None)
        elif weight.requires_grad:
            acc = torch.zeros(2, 1, H, dtype=torch.float32, device=x2.device)
            rows_group_sum_(acc[0], dy2, 1, x2d=x2, mean=stats[0], rstd=stats[1], out_plain=acc[1])
            dw, db = acc[0, 0].to(weight.dtype), (acc[1, 0].to(weight.dtype) if has_bias else None)
        return dx.view(shape), dw, db, None, None


def layer_norm(x, weight, bias=None, eps=1e-5, *, layer=None):
    """LayerNorm over the last dimension; under a capture the weight / bias gradients are produced per example."""
    if _use_kernel(x, weight) and x.shape[-1] % 8 == 0 and (bias is None or bias.dtype == torch.bfloat16):
        return _LayerNorm.apply(x, weight, bias, eps, layer)
    return torch.nn.functional.layer_norm(x, (x.shape[-1],), weight, bias, eps)


# =============================================================================== plain activations

_ACTS = {"silu": 0, "gelu": 1, "gelu_tanh": 2, "relu": 3}


class _Activation(Function):
    @staticmethod
    def forward(ctx, x, act):
        xc = x if x.is_contiguous() else x.contiguous()
        out = torch.empty_like(xc)
        rc = lib.load().ob_activation(xc.data_ptr(), None, out.data_ptr(), xc.numel(), act, lib.sm_count(), lib.stream())
        lib.check(rc, "activation")
        ctx.save_for_backward(xc)
        ctx.act = act
        return out

    @staticmethod
    def backward(ctx, dy):
        (xc,) = ctx.saved_tensors
        dyc = dy if dy.is_contiguous() else dy.contiguous()
        dx = torch.empty_like(xc)
        rc = lib.load().ob_activation(xc.data_ptr(), dyc.data_ptr(), dx.data_ptr(), xc.numel(), ctx.act, lib.sm_count(),
                                      lib.stream())
        lib.check(rc, "activation_bwd")
        return dx, None


def activation(x, kind: str = "gelu_tanh"):
    """``silu`` / ``gelu`` / ``gelu_tanh`` / ``relu`` with a one-pass backward (the input is the only saved tensor)."""
    if _use_kernel(x) and x.numel() % 8 == 0 and lib.available():
        return _Activation.apply(x, _ACTS[kind])
    if kind == "silu":
        return torch.nn.functional.silu(x)
    if kind == "relu":
        return torch.relu(x)
    return torch.nn.functional.gelu(x, approximate="tanh" if kind == "gelu_tanh" else "none")


# =============================================================================== gated activations

ACTIVATION_SWIGLU, ACTIVATION_GEGLU_EXACT, ACTIVATION_GEGLU_APPROX = 0, 1, 2


def glu_ref(gate, up, act=0):
    """PyTorch reference of the gated activations (``swiglu`` / ``geglu``)."""
    g = gate.float()
    if act == 0:
        a = torch.nn.functional.silu(g)
    elif act == 1:
        a = torch.nn.functional.gelu(g)
    else:
        a = torch.nn.functional.gelu(g, approximate="tanh")
    return (a * up.float()).to(gate.dtype)


class _GLU(Function):
    @staticmethod
    def forward(ctx, gate, up, act):
        I = gate.shape[-1]
        g2, u2 = gate.reshape(-1, I), up.reshape(-1, I)
        if g2.stride(1) != 1 or u2.stride(1) != 1 or g2.stride(0) != u2.stride(0):
            g2, u2 = g2.contiguous(), u2.contiguous()
        out = torch.empty(g2.shape, dtype=gate.dtype, device=gate.device)
        rc = lib.load().ob_glu_fwd(g2.data_ptr(), u2.data_ptr(), out.data_ptr(), g2.shape[0], I, g2.stride(0), act,
                                   lib.sm_count(), lib.stream())
        lib.check(rc, "glu_fwd")
        ctx.save_for_backward(g2, u2)
        ctx.meta = (gate.shape, act)
        return out.view(gate.shape)

    @staticmethod
    def backward(ctx, dh):
        g2, u2 = ctx.saved_tensors
        shape, act = ctx.meta
        I = shape[-1]
        d2 = dh.reshape(-1, I)
        d2 = d2 if d2.is_contiguous() else d2.contiguous()
        both = torch.empty(g2.shape[0], 2 * I, dtype=g2.dtype, device=g2.device)
        dg, du = both[:, :I], both[:, I:]
        rc = lib.load().ob_glu_bwd(d2.data_ptr(), g2.data_ptr(), u2.data_ptr(), dg.data_ptr(), du.data_ptr(),
                                   g2.shape[0], I, g2.stride(0), 2 * I, act, lib.sm_count(), lib.stream())
        lib.check(rc, "glu_bwd")
        return dg.view(shape), du.view(shape), None


_GLU_ACT_CODE = {"silu": ACTIVATION_SWIGLU, "gelu": ACTIVATION_GEGLU_EXACT, "gelu_pytorch_tanh": ACTIVATION_GEGLU_APPROX,
                 "gelu_tanh": ACTIVATION_GEGLU_APPROX}


def glu_backward(dh: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, act: str = "silu"):
    """``(dGate, dUp)`` of ``act(gate) * up`` for row-major bf16 matrices (views of one ``[rows, 2I]`` buffer)."""
    I = gate.shape[1]
    both = torch.empty(gate.shape[0], 2 * I, dtype=gate.dtype, device=gate.device)
    dg, du = both[:, :I], both[:, I:]
    rc = lib.load().ob_glu_bwd(dh.data_ptr(), gate.data_ptr(), up.data_ptr(), dg.data_ptr(), du.data_ptr(), gate.shape[0], I,
                               gate.stride(0), 2 * I, _GLU_ACT_CODE[act], lib.sm_count(), lib.stream())
    lib.check(rc, "glu_bwd")
    return dg, du


def swiglu(gate, up):
    """``silu(gate)·up``."""
    if _use_kernel(gate, up) and gate.shape[-1] % 8 == 0:
        return _GLU.apply(gate, up, ACTIVATION_SWIGLU)
    return glu_ref(gate, up, 0)


def geglu(gate, up, approximate=False):
    """``gelu(gate) * up`` (erf or tanh form) with a fused backward."""
    act = ACTIVATION_GEGLU_APPROX if approximate else ACTIVATION_GEGLU_EXACT
    if _use_kernel(gate, up) and gate.shape[-1] % 8 == 0:
        return _GLU.apply(gate, up, act)
    return glu_ref(gate, up, act)


# =============================================================================== RoPE

def rope_inverse_frequencies(head_dim: int, theta: float, scaling: dict | None = None, *, max_pos: int | None = None,
                             device=None) -> tuple[torch.Tensor, float]:
    """Inverse frequencies ``[head_dim/2]`` (fp32) and the factor that multiplies ``cos`` / ``sin``.

    ``scaling`` follows the Hugging Face ``rope_scaling`` / ``rope_parameters`` dictionaries:
    ``linear`` (positions divided by ``factor``), ``dynamic`` (NTK: the base grows once ``max_pos`` exceeds the original
    context), ``llama3`` (long wavelengths divided by ``factor``, a smooth blend between ``low_freq_factor`` and
    ``high_freq_factor``) and ``yarn`` (interpolation blended with extrapolation over a correction range, with an
    attention factor).  Anything else is refused.
    """
    half = torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim
    inv = 1.0 / (theta ** half)
    kind = (scaling or {}).get("rope_type", (scaling or {}).get("type", "default")) or "default"
    if kind == "default":
        return inv, 1.0
    factor = float(scaling.get("factor", 1.0))
    original = scaling.get("original_max_position_embeddings")
    if kind == "linear":
        return inv / factor, 1.0
    if kind == "dynamic":
        original = int(original or max_pos or 0)
        if max_pos and original and max_pos > original:
            base = theta * ((factor * max_pos / original) - (factor - 1.0)) ** (head_dim / (head_dim - 2))
            inv = 1.0 / (base ** half)
        return inv, 1.0
    if kind == "llama3":
        low, high = float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
        old = float(original)
        wavelen = 2.0 * math.pi / inv
        smooth = ((old / wavelen - low) / (high - low)).clamp(0.0, 1.0)
        blended = (1.0 - smooth) * inv / factor + smooth * inv
        out = torch.where(wavelen > old / low, inv / factor, torch.where(wavelen < old / high, inv, blended))
        return out, 1.0
    if kind == "yarn":
        original = float(original or max_pos)
        beta_fast, beta_slow = float(scaling.get("beta_fast") or 32.0), float(scaling.get("beta_slow") or 1.0)
        att = scaling.get("attention_factor")
        ms, ms_all = scaling.get("mscale"), scaling.get("mscale_all_dim")

        def mscale(f, m=1.0):
            return 1.0 if f <= 1.0 else 0.1 * m * math.log(f) + 1.0
        if att is None:
            att = mscale(factor, ms) / mscale(factor, ms_all) if (ms and ms_all) else mscale(factor)

        def correction_dim(rotations):
            return head_dim * math.log(original / (rotations * 2.0 * math.pi)) / (2.0 * math.log(theta))
        lo, hi = correction_dim(beta_fast), correction_dim(beta_slow)
        if scaling.get("truncate", True):
            lo, hi = math.floor(lo), math.ceil(hi)
        lo, hi = max(lo, 0), min(hi, head_dim - 1)
        if lo == hi:
            hi += 0.001
        ramp = ((torch.arange(head_dim // 2, dtype=torch.float32, device=device) - lo) / (hi - lo)).clamp(0.0, 1.0)
        keep = 1.0 - ramp                                   # 1 where the dimension extrapolates (high frequencies)
        out = (inv / factor) * (1.0 - keep) + inv * keep
        return out, float(att)
    raise NotImplementedError(f"rope scaling {kind!r} is not implemented (linear, dynamic, llama3 and yarn are)")


def rope_tables(head_dim: int, max_pos: int, theta: float = 10000.0, device=None, scaling: dict | None = None,
                rotary_dim: int | None = None):
    """fp32 ``cos, sin`` tables of shape ``[max_pos, head_dim/2]`` (``scaling``: see ``rope_inverse_frequencies``).

    With ``rotary_dim < head_dim`` (partial rotary embedding) only the first ``rotary_dim/2`` pairs ``(i, i + head_dim/2)``
    rotate; the remaining columns hold ``cos = 1, sin = 0``, which leaves those pairs untouched.
    """
    rot = head_dim if rotary_dim is None else int(rotary_dim)
    if rot % 2 or not 0 < rot <= head_dim:
        raise ValueError("rotary_dim must be even and in (0, head_dim]")
    inv, att = rope_inverse_frequencies(rot, theta, scaling, max_pos=max_pos, device=device)
    ang = torch.arange(max_pos, dtype=torch.float32, device=device)[:, None] * inv[None, :]
    cos, sin = ang.cos() * att, ang.sin() * att
    if rot < head_dim:
        pad = (head_dim - rot) // 2
        cos = torch.cat([cos, torch.ones(max_pos, pad, dtype=torch.float32, device=device)], dim=1)
        sin = torch.cat([sin, torch.zeros(max_pos, pad, dtype=torch.float32, device=device)], dim=1)
    return cos.contiguous(), sin.contiguous()


def rope_qk_ref(q, k, cos, sin, pos=None, sign=1.0):
    """Rotate-half RoPE; ``q: [..., T, Hq, D]``, ``k: [..., T, Hk, D]``; ``pos`` indexes the tables."""
    T = q.shape[-3]
    if pos is None:
        c, s = cos[:T], sin[:T]
        c, s = c[:, None, :], s[:, None, :]
    else:
        c, s = cos[pos][..., None, :], sin[pos][..., None, :]
    s = s * sign

    def rot(x):
        half = x.shape[-1] // 2
        lo, hi = x[..., :half].float(), x[..., half:].float()
        return torch.cat([lo * c - hi * s, hi * c + lo * s], dim=-1).to(x.dtype)
    return rot(q), rot(k)


class _RoPE(Function):
    """Joint rotary embedding.  Inputs may be any 4-D ``[B, T, H, D]`` views with a contiguous last dimension (slices of a
    fused q|k|v projection, the ``[B, H, T, D]``-laid-out gradients an attention kernel returns): the kernel reads them
    through their strides and writes contiguous outputs, so nothing is copied before or after."""

    @staticmethod
    def forward(ctx, q, k, cos, sin, pos):
        ctx.save_for_backward(cos, sin, pos if pos is not None else torch.empty(0))
        ctx.has_pos = pos is not None
        return _RoPE._run(q, k, cos, sin, pos, 0)

    @staticmethod
    def _strided_ok(x):
        return (x.ndim == 4 and x.stride(-1) == 1 and x.shape[-1] % 16 == 0 and x.data_ptr() % 16 == 0
                and all(s % 8 == 0 for s in x.stride()[:3]))

    @staticmethod
    def _run(q, k, cos, sin, pos, backward):
        T, Hq, D = q.shape[-3], q.shape[-2], q.shape[-1]
        Hk = k.shape[-2]
        rows = q.numel() // (Hq * D)
        p32 = None
        if pos is not None:
            p32 = pos.reshape(-1).to(torch.int32)
        if _RoPE._strided_ok(q) and _RoPE._strided_ok(k) and cos.data_ptr() % 16 == 0 and sin.data_ptr() % 16 == 0 \
                and cos.is_contiguous() and sin.is_contiguous():
            qo = torch.empty(q.shape, dtype=q.dtype, device=q.device)
            ko = torch.empty(k.shape, dtype=k.dtype, device=k.device)
            rc = lib.load().ob_rope_qk_oop(q.data_ptr(), k.data_ptr(), qo.data_ptr(), ko.data_ptr(), cos.data_ptr(),
                                           sin.data_ptr(), lib.ptr(p32), rows, T, Hq, Hk, D, q.stride(0), q.stride(1),
                                           q.stride(2), k.stride(0), k.stride(1), k.stride(2), backward, lib.sm_count(),
                                           lib.stream())
            lib.check(rc, "rope_qk")
            return qo, ko
        # general case: one copy into contiguous storage, rotated in place
        q, k = q.clone(memory_format=torch.contiguous_format), k.clone(memory_format=torch.contiguous_format)
        rc = lib.load().ob_rope_qk(q.data_ptr(), k.data_ptr(), cos.data_ptr(), sin.data_ptr(), lib.ptr(p32), rows, T,
                                   Hq, Hk, D, Hq * D, Hk * D, backward, lib.sm_count(), lib.stream())
        lib.check(rc, "rope_qk")
        return q, k

    @staticmethod
    def backward(ctx, dq, dk):
        cos, sin, pos = ctx.saved_tensors
        dq, dk = _RoPE._run(dq, dk, cos, sin, pos if ctx.has_pos else None, 1)
        return dq, dk, None, None, None


def rope_qk(q, k, cos, sin, pos=None):
    """Joint rotary embedding of Q ``[B, T, Hq, D]`` and K ``[B, T, Hk, D]``."""
    if _use_kernel(q, k) and q.shape[-1] % 4 == 0 and cos.dtype == torch.float32:
        return _RoPE.apply(q, k, cos, sin, pos)
    return rope_qk_ref(q, k, cos, sin, pos)


# =============================================================================== cross-entropy

def cross_entropy_ref(logits, labels, *, ignore_index=-100, logit_softcapping=0.0, logit_scaling=0.0,
                      label_smoothing=0.0):
    """Per-row NLL (0 for ignored rows) in fp32."""
    z = logits.float()
    if logit_scaling:
        z = z * logit_scaling
    if logit_softcapping:
        z = logit_softcapping * torch.tanh(z / logit_softcapping)
    lse = torch.logsumexp(z, dim=-1)
    valid = (labels != ignore_index) & (labels >= 0) & (labels < z.shape[-1])
    safe = labels.clamp(0, z.shape[-1] - 1)
    picked = z.gather(-1, safe[..., None]).squeeze(-1)
    nll = lse - picked
    if label_smoothing:
        nll = (1 - label_smoothing) * nll + label_smoothing * (lse - z.mean(-1))
    return torch.where(valid, nll, torch.zeros_like(nll))


def cross_entropy_fused_(logits, labels, row_weight=None, *, ignore_index=-100, logit_softcapping=0.0,
                         logit_scaling=0.0, label_smoothing=0.0, write_grad=True):
    """Kernel entry: returns per-row NLL; with ``write_grad`` OVERWRITES ``logits`` by ``w_row·∂nll/∂logits``."""
    V = logits.shape[-1]
    z = logits.view(-1, V)
    if z.stride(1) != 1:
        raise ValueError("logits rows must be contiguous")
    rows = z.shape[0]
    lab = labels.reshape(-1).to(torch.int64).contiguous()
    nll = torch.empty(rows, dtype=torch.float32, device=z.device)
    rc = lib.load().ob_cross_entropy(z.data_ptr(), int(z.dtype == torch.float32), lab.data_ptr(), lib.ptr(row_weight),
                                     nll.data_ptr(), None, rows, V, z.stride(0), logit_scaling or 1.0,
                                     logit_softcapping, label_smoothing, ignore_index, int(write_grad), lib.stream())
    lib.check(rc, "cross_entropy")
    return nll.view(labels.shape)


class _CrossEntropy(Function):
    @staticmethod
    def forward(ctx, logits, labels, ignore_index, softcap, scale, smoothing):
        buf = logits.contiguous().clone()
        nll = cross_entropy_fused_(buf, labels, None, ignore_index=ignore_index, logit_softcapping=softcap,
                                   logit_scaling=scale, label_smoothing=smoothing, write_grad=True)
        ctx.save_for_backward(buf)
        return nll

    @staticmethod
    def backward(ctx, dnll):
        (buf,) = ctx.saved_tensors
        return buf * dnll.reshape(buf.shape[:-1] + (1,)).to(buf.dtype), None, None, None, None, None


def cross_entropy(logits, labels, *, ignore_index=-100, logit_softcapping=0.0, logit_scaling=0.0,
                  label_smoothing=0.0):
    """Per-token NLL (unreduced) with softcap / scaling / label smoothing; ignored tokens give 0."""
    if _PLAIN == 0 and logits.is_cuda and logits.dtype in (torch.bfloat16, torch.float32):
        return _CrossEntropy.apply(logits, labels, ignore_index, logit_softcapping, logit_scaling, label_smoothing)
    return cross_entropy_ref(logits, labels, ignore_index=ignore_index, logit_softcapping=logit_softcapping,
                             logit_scaling=logit_scaling, label_smoothing=label_smoothing)


def selective_log_softmax(logits, indices):
    """``log_softmax(logits)[indices]`` without materialising the softmax (``= −nll``)."""
    return -cross_entropy(logits, indices, ignore_index=-(2 ** 62))
