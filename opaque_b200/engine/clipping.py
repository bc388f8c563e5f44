"""Reference DP clipping engine: per-example gradients → clip → sum.

Design: per-example outputs are produced for a whole microbatch at once with
``torch.func.vmap`` (leaves shaped ``[mb, *shape]``); clipping is then a
*batched* operation — one fp32 sum of squares per leaf per example, a fp64
cross-leaf total, a guarded scale vector ``c[mb]`` and one ``Σ_i c_i·g_i``
contraction per leaf.  (The reference maps a per-example ``clip_pytree`` under
vmap; the batched form is the same arithmetic in far fewer kernels and is the
shape the fused CUDA path consumes.)

The scale keeps the bound on values *as stored*: the ratio ``C/‖g‖`` gives up
``2(u_store + norm_roundoff)`` relative and one subnormal ULP absolute before
``min(1, ·)``; non-finite per-example gradients are zeroed first and a
non-finite scale becomes 0.

Parity: packages/opaque-engine/src/opaque/api/engine/clipping/_pytree.py:106-142, 345-564;
_clipped_fun.py:137-350, 526-881; _clipped_grad.py:81-344; _auto.py:200; _per_group.py:41-153.
"""
from __future__ import annotations

import dataclasses
import math
from collections.abc import Callable, Sequence
from typing import Any

import torch

from ..functional import under_differentiating_transform
from ..pytree import (param_path, param_path_display, tree_flatten, tree_flatten_with_paths, tree_map,
                      tree_unflatten)
from ..types import ClippedPytree, ClipState, PerGroup, SecondMomentClippingOutput

_BLOCK = 2048          # width of the first stage of the two-stage leaf reduction
_BLOCK_MIN = 4096      # leaves longer than this are reduced in two stages


@dataclasses.dataclass(frozen=True)
class FixedClipState(ClipState):
    """Fixed clipping keeps no run state; the bound travels on ``ClippedPytree.max_norm``."""


@dataclasses.dataclass(frozen=True)
class AutoClipState(ClipState):
    """AUTO-S keeps no run state either."""


@dataclasses.dataclass(frozen=True)
class ClippingStats:
    num_clipped: Any
    clipping_rate: Any
    batch_size: int = 0
    all_finite: bool = True


@dataclasses.dataclass(frozen=True)
class ClippedFunAux:
    values: Any = None
    norms: Any = None
    clipped_norms: Any = None
    aux: Any = None
    clipping_rate: Any = None
    batch_size: int = 0
    group_norms: dict[str, torch.Tensor] | None = None

    @property
    def value_aux(self) -> Any:
        """The auxiliary outputs of the clipped function (``aux`` under the reference's field name)."""
        return self.aux


@dataclasses.dataclass(frozen=True)
class ClippedGradAux:
    """Diagnostics only (pre-noise); never feed them back into private computation."""
    loss_values: Any = None
    grad_norms: Any = None
    clipped_grad_norms: Any = None
    loss_aux: Any = None
    clipping_rate: Any = None
    batch_size: int = 0
    group_norms: dict[str, torch.Tensor] | None = None


@dataclasses.dataclass(frozen=True)
class ClipPytreeAux:
    norm: torch.Tensor
    group_norms: dict[str, torch.Tensor] | None = None


# ----------------------------------------------------------------------------- numerics

def _acc_dtype(leaves: Sequence[torch.Tensor], compute_dtype: torch.dtype | None) -> torch.dtype:
    if compute_dtype is not None:
        if not compute_dtype.is_floating_point:
            raise TypeError(f"compute_dtype must be a real floating-point dtype, got {compute_dtype!r}")
        return compute_dtype
    acc = torch.float32
    for x in leaves:
        if x.is_floating_point() and x.dtype == torch.float64:
            acc = torch.float64
    return acc


def _wide_dtype(leaves: Sequence[torch.Tensor]) -> torch.dtype:
    return torch.float32 if any(x.device.type == "mps" for x in leaves) else torch.float64


def _reduction_terms(numels: Sequence[int]) -> int:
    widest = max(numels, default=0)
    if widest <= 1:
        return 0
    if widest > _BLOCK_MIN:
        return _BLOCK + (widest + _BLOCK - 1) // _BLOCK
    return widest


def norm_roundoff(acc: torch.dtype, wide: torch.dtype, n_leaves: int, n_red: int) -> float:
    """Relative error bound of the computed norm (halved: it passes through a sqrt)."""
    u_acc = torch.finfo(acc).eps / 2
    u_wide = torch.finfo(wide).eps / 2
    return (u_acc + (max(n_leaves, 1) + n_red) * u_wide) / 2


def guard_scale(ratio: torch.Tensor, store: torch.dtype, roundoff: float, *, clamp: bool) -> torch.Tensor:
    """Shrink ``ratio`` so the stored, rounded product cannot exceed the bound; sanitise."""
    if store.is_floating_point or store.is_complex:
        fi = torch.finfo(store)
        ratio = ratio * (1.0 - 2.0 * (fi.eps / 2 + roundoff)) - fi.smallest_normal * fi.eps
    if clamp:
        ratio = torch.clamp(ratio, max=1.0)
    ratio = torch.where(torch.isfinite(ratio), ratio, torch.zeros_like(ratio))
    return torch.clamp(ratio, min=0.0)


def _batched_sq(x: torch.Tensor, acc: torch.dtype, wide: torch.dtype) -> torch.Tensor:
    """Per-example sum of squares of a ``[B, ...]`` leaf → ``[B]`` in ``wide``."""
    b = x.shape[0]
    flat = x.reshape(b, -1)
    if flat.is_complex():
        sq = flat.real.to(acc) ** 2 + flat.imag.to(acc) ** 2
    else:
        f = flat.to(acc)
        sq = f * f
    n = sq.shape[1]
    if n <= _BLOCK_MIN:
        return sq.sum(dim=1, dtype=wide)
    main = (n // _BLOCK) * _BLOCK
    total = sq[:, :main].reshape(b, -1, _BLOCK).sum(dim=-1, dtype=wide).sum(dim=-1, dtype=wide)
    if main < n:
        total = total + sq[:, main:].sum(dim=1, dtype=wide)
    return total


def _sanitize(x: torch.Tensor) -> torch.Tensor:
    return torch.nan_to_num(x, nan=0.0, posinf=0.0, neginf=0.0) if x.is_floating_point() or x.is_complex() else x


def _weighted_sum(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """``Σ_i w_i·x_i`` over the leading axis, the product rounded into ``x``'s dtype first.

    Rounding ``w_i·x_i`` to the storage dtype before summing is what the
    sensitivity bound is stated for: each record's stored contribution has
    norm at most ``C``.
    """
    shape = (x.shape[0],) + (1,) * (x.ndim - 1)
    scaled = w.to(x.dtype).reshape(shape) * x
    return scaled.sum(dim=0, dtype=torch.float32 if out_dtype in (torch.bfloat16, torch.float16) else out_dtype).to(out_dtype)


def _validate_groups(paths: Sequence[tuple], pg: PerGroup) -> None:
    have, want = set(paths), set(pg.groups)
    if have == want:
        return
    msg = ["PerGroup path keys must match the pytree tensor leaves exactly."]
    if have - want:
        msg.append(f"Leaves with no group assignment: {sorted(map(param_path_display, have - want))}.")
    if want - have:
        msg.append(f"Group paths with no matching leaf: {sorted(map(param_path_display, want - have))}.")
    raise ValueError(" ".join(msg))


def batched_clip_scales(batched: Any, bound: float | PerGroup, *, mode: str = "clip", gamma: float = 0.01,
                        compute_dtype: torch.dtype | None = None):
    """Per-example scales for a tree of ``[B, ...]`` leaves.

    Returns ``(scale_for_leaf, norms[B], group_norms | None, finite[B])`` where
    ``scale_for_leaf(path, dtype)`` gives the guarded ``[B]`` scale for a leaf.
    ``mode='clip'`` is ``min(1, C/‖g‖)``; ``mode='auto'`` is ``R/(‖g‖+γ)``.
    """
    paths, leaves, _ = tree_flatten_with_paths(batched)
    tens = [(p, x) for p, x in zip(paths, leaves) if isinstance(x, torch.Tensor)]
    if not tens:
        raise ValueError("nothing to clip: the tree has no tensor leaves")
    xs = [x for _, x in tens]
    acc, wide = _acc_dtype(xs, compute_dtype), _wide_dtype(xs)
    rnd = norm_roundoff(acc, wide, len(xs), _reduction_terms([x[0].numel() if x.shape[0] else 0 for x in xs]))
    sq = {p: _batched_sq(x, acc, wide) for p, x in tens}
    total = torch.stack(list(sq.values())).sum(dim=0)
    norms = total.sqrt()
    finite = torch.isfinite(norms)

    def ratio_of(norm: torch.Tensor, c: float) -> torch.Tensor:
        cc = torch.clamp(torch.as_tensor(c, dtype=norm.dtype, device=norm.device), min=0.0)
        return cc / (norm + gamma) if mode == "auto" else cc / norm

    if isinstance(bound, PerGroup):
        _validate_groups([p for p, _ in tens], bound)
        gsq: dict[str, torch.Tensor] = {}
        for p, _ in tens:
            g = bound.groups[p]
            gsq[g] = gsq[g] + sq[p] if g in gsq else sq[p]
        gnorm = {g: v.sqrt() for g, v in gsq.items()}
        gratio = {g: ratio_of(gnorm[g], bound.values[g]) for g in gnorm}

        def scale_for(path, dtype):
            return guard_scale(gratio[bound.groups[path]], dtype, rnd, clamp=(mode == "clip"))
        return scale_for, norms.to(acc), {g: v.to(acc) for g, v in gnorm.items()}, finite

    ratio = ratio_of(norms, float(bound))

    def scale_for(path, dtype):
        return guard_scale(ratio, dtype, rnd, clamp=(mode == "clip"))
    return scale_for, norms.to(acc), None, finite


def clip_pytree(pytree: Any, clipping_norm: float | PerGroup, return_zero: bool = False, *,
                compute_dtype: torch.dtype | None = None):
    """Clip ONE record's tree to L2 norm ``clipping_norm`` (guarded; non-finite values zeroed)."""
    lifted = tree_map(lambda t: _sanitize(t).unsqueeze(0) if isinstance(t, torch.Tensor) else t, pytree)
    scale_for, norms, gnorms, _ = batched_clip_scales(lifted, clipping_norm, compute_dtype=compute_dtype)
    paths, leaves, td = tree_flatten_with_paths(lifted)
    out = []
    for p, x in zip(paths, leaves):
        if not isinstance(x, torch.Tensor):
            out.append(x)
        elif return_zero:
            out.append(torch.zeros_like(x[0]))
        else:
            out.append((scale_for(p, x.dtype).to(x.dtype).reshape((1,) * x.ndim) * x)[0])
    aux = ClipPytreeAux(norms[0], None if gnorms is None else {g: v[0] for g, v in gnorms.items()})
    return tree_unflatten(td, out), aux


def auto_scale_pytree(pytree: Any, R: float | PerGroup = 1.0, gamma: float = 0.01, *,
                      compute_dtype: torch.dtype | None = None):
    """AUTO-S: rescale ONE record's tree by ``R/(‖g‖+γ)`` (no clamp to 1)."""
    lifted = tree_map(lambda t: _sanitize(t).unsqueeze(0) if isinstance(t, torch.Tensor) else t, pytree)
    scale_for, norms, gnorms, _ = batched_clip_scales(lifted, R, mode="auto", gamma=gamma, compute_dtype=compute_dtype)
    paths, leaves, td = tree_flatten_with_paths(lifted)
    out = [(scale_for(p, x.dtype).to(x.dtype).reshape((1,) * x.ndim) * x)[0] if isinstance(x, torch.Tensor) else x
           for p, x in zip(paths, leaves)]
    aux = ClipPytreeAux(norms[0], None if gnorms is None else {g: v[0] for g, v in gnorms.items()})
    return tree_unflatten(td, out), aux


# ----------------------------------------------------------------------------- per_group

def per_group(params: Any, /, patterns: dict[str, float] | None = None, *, fallback: float | None = None,
              **kwargs: float) -> PerGroup:
    """Assign each parameter leaf to a group by substring match on its dotted path.

    ``patterns`` (or keyword arguments) map a substring to that group's value;
    the first matching pattern wins; leaves matching nothing go to the
    ``"fallback"`` group when ``fallback`` is given and are an error otherwise.
    """
    table = dict(patterns or {})
    table.update(kwargs)
    if not table and fallback is None:
        raise ValueError("per_group needs at least one pattern or a fallback")
    paths, leaves, _ = tree_flatten_with_paths(params)
    groups: dict[tuple, str] = {}
    used: set[str] = set()
    for p, x in zip(paths, leaves):
        if not isinstance(x, torch.Tensor):
            continue
        name = param_path_display(p)
        hit = next((pat for pat in table if pat in name), None)
        if hit is None:
            if fallback is None:
                raise ValueError(f"parameter {name!r} matches no group pattern and no fallback was given")
            hit = "fallback"
        groups[p] = hit
        used.add(hit)
    values = {g: float(table[g]) for g in used if g != "fallback"}
    if "fallback" in used:
        values["fallback"] = float(fallback)
    for g, v in values.items():
        if v < 0 or math.isnan(v):
            raise ValueError(f"group {g!r} has an invalid bound {v}")
    return PerGroup(groups, values)


# ----------------------------------------------------------------------------- clipped_fun

def _as_tuple(x: int | Sequence[int]) -> tuple[int, ...]:
    return (x,) if isinstance(x, int) else tuple(x)


def _batch_size(args: Sequence[Any], batch_argnums: tuple[int, ...]) -> int:
    size = None
    for i in batch_argnums:
        for leaf in tree_flatten(args[i])[0]:
            if isinstance(leaf, torch.Tensor):
                if leaf.ndim == 0:
                    raise ValueError("batched arguments must have a leading batch axis")
                if size is None:
                    size = leaf.shape[0]
                elif leaf.shape[0] != size:
                    raise ValueError(f"inconsistent batch sizes: {size} vs {leaf.shape[0]}")
    if size is None:
        raise ValueError("no tensor found in the batched arguments")
    return size


def _slice(args: Sequence[Any], batch_argnums: tuple[int, ...], lo: int, hi: int) -> list[Any]:
    out = list(args)
    for i in batch_argnums:
        out[i] = tree_map(lambda t: t[lo:hi] if isinstance(t, torch.Tensor) else t, out[i])
    return out


def _scale_bound(bound: Any, f: float) -> Any:
    return bound * f if isinstance(bound, PerGroup) else float(bound) * f


def _square_bound(bound: Any) -> Any:
    return bound * bound if isinstance(bound, PerGroup) else float(bound) ** 2


def clipped_fun(fun: Callable, has_aux: bool = False, *, batch_argnums: int | Sequence[int] = 0,
                clipping_norm: float | PerGroup = 1.0, normalize_by: float = 1.0, return_aux: bool = False,
                return_stats: bool = False, second_moment: bool = False, microbatch_size: int | None = None,
                dtype: torch.dtype | None = None, compute_dtype: torch.dtype | None = None,
                _scale_fn: Callable | None = None, _mode: str = "clip", _gamma: float = 0.01,
                _state: ClipState | None = None):
    """Map ``fun`` over examples, clip each output tree, and sum.

    ``fun`` receives ONE example (no batch axis) in every ``batch_argnums``
    position and returns a tensor tree (plus aux when ``has_aux``).  The result
    is ``ClippedPytree(Σ_i clip(fun_i), max_norm=clipping_norm)/normalize_by``.
    A microbatch loop bounds memory; sums are accumulated in fp32 at least.
    """
    if normalize_by <= 0:
        raise ValueError(f"normalize_by must be > 0, got {normalize_by}.")
    if return_aux and return_stats:
        raise ValueError("return_stats cannot be combined with return_aux=True")
    if microbatch_size is not None and microbatch_size < 1:
        raise ValueError("microbatch_size must be >= 1")
    b_nums = _as_tuple(batch_argnums)
    if not b_nums:
        raise ValueError("Batch argnums must not be empty.")
    max_norm = _scale_bound(clipping_norm, 1.0 / normalize_by)

    def per_example(*args):
        out = fun(*args)
        return out if has_aux else (out, ())

    def transformed(*args: Any, state: ClipState | None = None):
        n = _batch_size(args, b_nums)
        in_dims = tuple(0 if i in b_nums else None for i in range(len(args)))
        mb = n if microbatch_size is None else min(microbatch_size, max(n, 1))
        sums: list[torch.Tensor] | None = None
        sq_sums: list[torch.Tensor] | None = None
        td = None
        values, aux_parts, norm_parts, cnorm_parts = [], [], [], []
        gnorm_parts: dict[str, list[torch.Tensor]] = {}
        num_clipped: Any = 0.0
        finite_all = True
        for lo in range(0, n, max(mb, 1)):
            hi = min(n, lo + mb)
            piece = _slice(args, b_nums, lo, hi)
            out, aux = torch.func.vmap(per_example, in_dims=in_dims, randomness="same")(*piece)
            paths, leaves, td = tree_flatten_with_paths(out)
            raw_finite = all(bool(torch.isfinite(x).all()) for x in leaves if isinstance(x, torch.Tensor)) \
                if return_stats else True
            finite_all = finite_all and raw_finite
            leaves = [_sanitize(x) if isinstance(x, torch.Tensor) else x for x in leaves]
            batched = tree_unflatten(td, leaves)
            if _scale_fn is not None:
                scale_for, norms, gnorms = _scale_fn(batched)
            else:
                scale_for, norms, gnorms, _ = batched_clip_scales(
                    batched, clipping_norm, mode=_mode, gamma=_gamma, compute_dtype=compute_dtype)
            part, part_sq = [], []
            for p, x in zip(paths, leaves):
                c = scale_for(p, x.dtype)
                out_dt = dtype or (torch.float32 if x.dtype in (torch.bfloat16, torch.float16) else x.dtype)
                part.append(_weighted_sum(x, c, out_dt))
                if second_moment:
                    shape = (x.shape[0],) + (1,) * (x.ndim - 1)
                    clipped_x = c.to(x.dtype).reshape(shape) * x
                    part_sq.append((clipped_x.to(out_dt) ** 2).sum(dim=0))
            sums = part if sums is None else [a + b for a, b in zip(sums, part)]
            if second_moment:
                sq_sums = part_sq if sq_sums is None else [a + b for a, b in zip(sq_sums, part_sq)]
            if isinstance(clipping_norm, PerGroup) and gnorms is not None and _mode == "clip":
                nc = {g: float((gnorms[g] > clipping_norm.values[g]).sum()) for g in gnorms}
                num_clipped = nc if not isinstance(num_clipped, dict) else {g: num_clipped[g] + nc[g] for g in nc}
            elif _mode == "clip" and not isinstance(clipping_norm, PerGroup):
                num_clipped = num_clipped + float((norms > float(clipping_norm)).sum())
            if return_aux:
                norm_parts.append(norms)
                if isinstance(clipping_norm, PerGroup):
                    cn2 = torch.zeros_like(norms, dtype=torch.float64)
                    for g, gn in gnorms.items():
                        gs = guard_scale((torch.as_tensor(clipping_norm.values[g], dtype=gn.dtype) / (gn + (_gamma if _mode == "auto" else 0.0))),
                                         torch.float32, 0.0, clamp=(_mode == "clip"))
                        cn2 = cn2 + (gs.double() * gn.double()) ** 2
                        gnorm_parts.setdefault(g, []).append(gn)
                    cnorm_parts.append(cn2.sqrt().to(norms.dtype))
                else:
                    first_path = next(p for p, x in zip(paths, leaves) if isinstance(x, torch.Tensor))
                    cnorm_parts.append(scale_for(first_path, torch.float32).to(norms.dtype) * norms)
                if has_aux:
                    aux_parts.append(aux)
        if sums is None:  # empty batch
            raise _EmptyBatch()
        inv = 1.0 / normalize_by
        tree = tree_unflatten(td, [s * inv if inv != 1.0 else s for s in sums])
        result: Any = ClippedPytree(tree, max_norm)
        if second_moment:
            sq_tree = tree_unflatten(td, [s * inv if inv != 1.0 else s for s in sq_sums])
            result = SecondMomentClippingOutput(result, ClippedPytree(sq_tree, _scale_bound(_square_bound(clipping_norm), inv)))
        new_state = state if state is not None else (_state or FixedClipState())
        rate = ({g: v / n for g, v in num_clipped.items()} if isinstance(num_clipped, dict) else num_clipped / n) if n else None
        if return_stats:
            return (result, ClippingStats(num_clipped, rate, n, finite_all)), new_state
        if return_aux:
            def cat_tree(parts):
                if not parts:
                    return None
                return tree_map(lambda *xs: torch.cat([x if x.ndim else x[None] for x in xs], dim=0), *parts)
            fa = ClippedFunAux(values=None, norms=torch.cat(norm_parts), clipped_norms=torch.cat(cnorm_parts),
                               aux=cat_tree(aux_parts), clipping_rate=rate, batch_size=n,
                               group_norms={g: torch.cat(v) for g, v in gnorm_parts.items()} or None)
            return (result, fa), new_state
        return result, new_state

    return transformed, (_state or FixedClipState())


class _EmptyBatch(Exception):
    pass


# ----------------------------------------------------------------------------- clipped_grad

def _zeros_like_args(args: Sequence[Any], argnums: tuple[int, ...], single: bool, dtype):
    def z(t):
        if not isinstance(t, torch.Tensor):
            return t
        dt = dtype or (torch.float32 if t.dtype in (torch.bfloat16, torch.float16) else t.dtype)
        return torch.zeros_like(t, dtype=dt)
    trees = tuple(tree_map(z, args[i]) for i in argnums)
    return trees[0] if single else trees


def clipped_grad(loss_fn: Callable, argnums: int | Sequence[int] = 0, has_aux: bool = False, *,
                 clipping_norm: float | PerGroup, normalize_by: float = 1.0,
                 batch_argnums: int | Sequence[int] = 1, return_aux: bool = False, return_stats: bool = False,
                 second_moment: bool = False, pre_clipping_transform: Callable = lambda x: x,
                 microbatch_size: int | None = None, dtype: torch.dtype | None = None,
                 compute_dtype: torch.dtype | None = None, _scale_fn: Callable | None = None,
                 _mode: str = "clip", _gamma: float = 0.01, _state: ClipState | None = None,
                 _range_name: str = "opaque::clipped_grad"):
    """Per-example-clipped gradient of ``loss_fn``.

    ``loss_fn(*args)`` is written for ONE example and returns a scalar loss (and
    aux when ``has_aux``).  Returns ``(grad_fn, clip_state)`` with
    ``grad_fn(*args, state=clip_state) -> (ClippedPytree | (ClippedPytree, aux), state)``.
    An empty batch short-circuits to zeros.  Autograd recording is disabled
    unless the call sits inside a differentiating ``torch.func`` transform.
    """
    a_nums, b_nums = _as_tuple(argnums), _as_tuple(batch_argnums)
    if normalize_by <= 0:
        raise ValueError(f"normalize_by must be > 0, got {normalize_by}.")
    if not b_nums:
        raise ValueError("Batch argnums must not be empty.")
    if min(a_nums + b_nums) < 0:
        raise ValueError(f"argnums={a_nums} and batch_argnums={b_nums} must be >= 0.")
    if set(a_nums) & set(b_nums):
        raise ValueError(f"Cannot compute clipped gradients for argnums that have a batch axis: "
                         f"argnums={a_nums} batch_argnums={b_nums}")
    if return_aux and return_stats:
        raise ValueError("return_stats cannot be combined with return_aux=True")
    single = isinstance(argnums, int)

    def loss_with_aux(*args):
        out = loss_fn(*args)
        loss, aux = out if has_aux else (out, ())
        return loss, (loss.detach(), aux)

    g_and_v = torch.func.grad(loss_with_aux, argnums=argnums, has_aux=True)

    def per_example(*args):
        grads, (loss, aux) = g_and_v(*args)
        return pre_clipping_transform(grads), (loss, aux)

    inner, init_state = clipped_fun(
        per_example, has_aux=True, batch_argnums=b_nums, clipping_norm=clipping_norm, normalize_by=normalize_by,
        return_aux=return_aux, return_stats=return_stats, second_moment=second_moment,
        microbatch_size=microbatch_size, dtype=dtype, compute_dtype=compute_dtype, _scale_fn=_scale_fn,
        _mode=_mode, _gamma=_gamma, _state=_state)
    max_norm = _scale_bound(clipping_norm, 1.0 / normalize_by)

    def grad_fn(*args: Any, state: ClipState | None = None):
        state = state if state is not None else init_state
        n = _batch_size(args, b_nums)
        if n == 0:
            zero = ClippedPytree(_zeros_like_args(args, a_nums, single, dtype), max_norm)
            out: Any = zero
            if second_moment:
                out = SecondMomentClippingOutput(zero, ClippedPytree(
                    _zeros_like_args(args, a_nums, single, dtype), _scale_bound(_square_bound(clipping_norm), 1.0 / normalize_by)))
            if return_stats:
                return (out, ClippingStats(0.0, None, 0, True)), state
            if return_aux:
                e = torch.zeros(0)
                return (out, ClippedGradAux(e, e, e, None, None, 0, None)), state
            return out, state
        with torch.profiler.record_function(_range_name):
            if under_differentiating_transform():
                res, new_state = inner(*args, state=state)
            else:
                with torch.no_grad():
                    res, new_state = inner(*args, state=state)
        if return_aux:
            tree, fa = res
            loss_vals, user_aux = fa.aux if fa.aux is not None else (None, None)
            return (tree, ClippedGradAux(loss_vals, fa.norms, fa.clipped_norms, user_aux if has_aux else None,
                                         fa.clipping_rate, fa.batch_size, fa.group_norms)), new_state
        return res, new_state

    return grad_fn, init_state


def auto_clipped_fun(fun: Callable, has_aux: bool = False, *, R: float | PerGroup = 1.0, gamma: float = 0.01,
                     **kw: Any):
    """AUTO-S variant of :func:`clipped_fun`: every example is rescaled to ``R·‖g‖/(‖g‖+γ)``."""
    if gamma <= 0:
        raise ValueError("gamma must be > 0")
    return clipped_fun(fun, has_aux, clipping_norm=R, _mode="auto", _gamma=gamma, _state=AutoClipState(), **kw)


def auto_clipped_grad(loss_fn: Callable, argnums: int | Sequence[int] = 0, has_aux: bool = False, *,
                      R: float | PerGroup = 1.0, gamma: float = 0.01, normalize_by: float = 1.0,
                      batch_argnums: int | Sequence[int] = 1, return_aux: bool = False, return_stats: bool = False,
                      pre_clipping_transform: Callable = lambda x: x, microbatch_size: int | None = None,
                      dtype: torch.dtype | None = None, second_moment: bool = False):
    """AUTO-S (Bu et al.): no threshold to tune; sensitivity is ``R``."""
    if gamma <= 0:
        raise ValueError("gamma must be > 0")
    return clipped_grad(loss_fn, argnums, has_aux, clipping_norm=R, normalize_by=normalize_by,
                        batch_argnums=batch_argnums, return_aux=return_aux, return_stats=return_stats,
                        second_moment=second_moment, pre_clipping_transform=pre_clipping_transform,
                        microbatch_size=microbatch_size, dtype=dtype, _mode="auto", _gamma=gamma,
                        _state=AutoClipState(), _range_name="opaque::auto_clipped_grad")


__all__ = [
    "AutoClipState", "ClipPytreeAux", "ClippedFunAux", "ClippedGradAux", "ClippingStats", "FixedClipState",
    "auto_clipped_fun", "auto_clipped_grad", "auto_scale_pytree", "batched_clip_scales", "clip_pytree",
    "clipped_fun", "clipped_grad", "guard_scale", "norm_roundoff", "per_group",
]
