"""Functional views of ``nn.Module`` and batch-dimension helpers.

``make_functional`` turns a module into ``fmodel(params, *args)`` backed by
``torch.func.functional_call``.  ``with_batch_dim`` adapts a function written
for batched inputs to the per-example calling convention of the vmap-based
reference engine (it re-adds a size-1 batch axis on the way in and removes it
on the way out).  ``empty_collate`` builds a zero-length batch with the right
trailing shapes for Poisson steps that sample nothing.

Parity: packages/opaque-engine/src/opaque/api/engine/functional/__init__.py:15-186, :219-360;
_collate.py:50-101; _transform_stack.py:9-20.
"""
from __future__ import annotations

import functools
from collections.abc import Callable, Sequence
from typing import Any

import torch
from torch import nn

from ..pytree import merge, partition, tree_map  # noqa: F401  (re-exported helpers)


def make_functional(mod: nn.Module, disable_autograd_tracking: bool = False,
                    partition_trainable: bool = False):
    """``(fmodel, params)`` or, with ``partition_trainable``, ``(fmodel, trainable, frozen)``.

    The tuple form takes parameters in ``named_parameters()`` order; the
    partitioned form takes a name → tensor dict (merge ``frozen`` and
    ``trainable`` before the call).  Buffers stay on the module.
    """
    named = dict(mod.named_parameters())
    values = {k: (v.detach() if disable_autograd_tracking else v) for k, v in named.items()}
    if partition_trainable:
        trainable = {k: values[k] for k, p in named.items() if p.requires_grad}
        frozen = {k: values[k] for k, p in named.items() if not p.requires_grad}

        def fmodel_named(params: dict, *args: Any, **kwargs: Any):
            return torch.func.functional_call(mod, params, args, kwargs)
        return fmodel_named, trainable, frozen

    names = tuple(values)

    def fmodel_positional(params: Sequence[torch.Tensor], *args: Any, **kwargs: Any):
        if len(params) != len(names):
            raise ValueError(f"expected {len(names)} parameter tensors, got {len(params)}")
        return torch.func.functional_call(mod, dict(zip(names, params)), args, kwargs)
    return fmodel_positional, tuple(values.values())


def _lift(x: Any, min_ndim: int | None) -> Any:
    if isinstance(x, torch.Tensor) and (min_ndim is None or x.ndim < min_ndim):
        return x.unsqueeze(0)
    return x


def _drop(x: Any) -> Any:
    if isinstance(x, torch.Tensor) and x.ndim >= 1 and x.shape[0] == 1:
        return x.squeeze(0)
    return x


def with_batch_dim(fn: Callable, batch_argnums: int | Sequence[int] = (), batch_kwargs: Sequence[str] = (),
                   *, min_ndim: int | None = None) -> Callable:
    """Call a batch-expecting ``fn`` on one example: unsqueeze inputs, squeeze outputs."""
    nums = (batch_argnums,) if isinstance(batch_argnums, int) else tuple(batch_argnums)
    names = tuple(batch_kwargs)

    @functools.wraps(fn)
    def wrapped(*args: Any, **kwargs: Any):
        args = list(args)
        for i in nums:
            if i < len(args):
                args[i] = tree_map(lambda t: _lift(t, min_ndim), args[i])
        for k in names:
            if k in kwargs:
                kwargs[k] = tree_map(lambda t: _lift(t, min_ndim), kwargs[k])
        return tree_map(_drop, fn(*args, **kwargs))
    return wrapped


def empty_collate(collate_fn: Any) -> Any:
    """Given a collate FUNCTION: the same function, except that an empty list of examples (an empty Poisson draw) gives a
    batch with the structure of the first non-empty batch it has seen and a zero-length batch dimension (an empty first
    call still reaches the wrapped function, which is the right place for that error).

    Given an EXAMPLE (anything not callable): a batch of zero examples shaped like it (one element of the dataset).

    Parity: packages/opaque-engine/src/opaque/api/engine/functional/_collate.py:50-101."""
    if callable(collate_fn) and not isinstance(collate_fn, torch.Tensor):
        import functools
        seen: list[Any] = []

        def empty_batch(x: Any):
            if isinstance(x, torch.Tensor):
                return x.new_zeros((0,) + tuple(x.shape[1:])) if x.ndim else x.new_zeros((0,))
            return x

        @functools.wraps(collate_fn)
        def wrapped(examples, *args, **kwargs):
            if len(examples) == 0 and seen:
                return tree_map(empty_batch, seen[0])
            out = collate_fn(examples, *args, **kwargs)
            if len(examples) and not seen:
                seen.append(tree_map(lambda x: x[:0].clone() if isinstance(x, torch.Tensor) and x.ndim else x, out))
            return out
        return wrapped
    example = collate_fn

    def zero_len(x: Any):
        if isinstance(x, torch.Tensor):
            return x.new_zeros((0,) + tuple(x.shape))
        if isinstance(x, (int, bool)):
            return torch.zeros(0, dtype=torch.long)
        if isinstance(x, float):
            return torch.zeros(0, dtype=torch.float32)
        if hasattr(x, "__array__"):
            t = torch.as_tensor(x)
            return t.new_zeros((0,) + tuple(t.shape))
        return x
    return tree_map(zero_len, example)


def under_differentiating_transform() -> bool:
    """True inside ``torch.func.grad`` / ``vjp`` / ``jvp`` (where ``no_grad`` must not be forced)."""
    try:
        from torch._C._functorch import TransformType, peek_interpreter_stack
        top = peek_interpreter_stack()
        if top is None:
            return False
        return top.key() in (TransformType.Grad, TransformType.Jvp)
    except Exception:
        return False


class _Recompute(torch.autograd.Function):
    """``fn(*inputs)`` whose backward pass recomputes the forward pass; usable under ``torch.func`` transforms."""
    generate_vmap_rule = True

    @staticmethod
    def forward(fn, diff_mask, *inputs):
        return fn(*inputs)

    @staticmethod
    def setup_context(ctx, inputs, output):
        ctx.fn, ctx.diff_mask = inputs[0], inputs[1]
        ctx.save_for_backward(*inputs[2:])

    @staticmethod
    def backward(ctx, grad_out):
        saved = ctx.saved_tensors
        diff = [t for t, d in zip(saved, ctx.diff_mask) if d]

        def of_diff(*primals):
            it = iter(primals)
            return ctx.fn(*[next(it) if d else t for t, d in zip(saved, ctx.diff_mask)])
        _, pull = torch.func.vjp(of_diff, *diff)
        grads = iter(pull(grad_out))
        return (None, None, *[next(grads) if d else None for d in ctx.diff_mask])


def functional_checkpoint(module: nn.Module, *args: Any) -> torch.Tensor:
    """Activation checkpointing that works under ``vmap(grad(...))``: run ``module(*args)`` without keeping its
    intermediates and recompute them in the backward pass.

    ``torch.utils.checkpoint`` relies on saved-tensor hooks (or an autograd node without a batching rule), neither of
    which ``torch.func`` supports.  Here every tensor argument and every trainable parameter of ``module`` (as currently
    bound, e.g. by ``functional_call``) becomes an explicit input of one autograd node with a generated batching rule;
    frozen parameters, non-tensor arguments and buffers are closed over.  The module must return one tensor.
    Parity: packages/opaque-patches/src/opaque/api/patches/torch/checkpoint of the reference (checkpointing under the
    per-example engine).
    """
    tensor_pos = [i for i, a in enumerate(args) if isinstance(a, torch.Tensor)]
    names, params, fixed = [], [], {}
    for n, p in module.named_parameters():
        if p.requires_grad:
            names.append(n)
            params.append(p)
        else:
            fixed[n] = p
    n_args = len(tensor_pos)

    def pure(*flat):
        call = list(args)
        for i, t in zip(tensor_pos, flat[:n_args]):
            call[i] = t
        return torch.func.functional_call(module, {**fixed, **dict(zip(names, flat[n_args:]))}, tuple(call))
    inputs = [args[i] for i in tensor_pos] + params
    diff_mask = tuple(bool(t.is_floating_point()) for t in inputs)
    return _Recompute.apply(pure, diff_mask, *inputs)


__all__ = ["empty_collate", "functional_checkpoint", "make_functional", "merge", "partition",
           "under_differentiating_transform", "with_batch_dim"]
