"""Data-parallel helpers over ``torch.distributed`` (NCCL on GPUs, gloo on CPU).

Everything here is a local no-op when no process group exists, so the same
training loop runs on one process and on eight.  The gradient path offered here
(``sum_gradients_`` = a reduction of the clipped sum) is the *baseline*
communication path; the fused path that reduce-scatters from the
weight-gradient kernel's epilogue lives in ``opaque_b200.parallel``.

Differences from the reference design: ``reduce_pytree_`` packs every leaf of
one dtype into a single flat buffer and issues ONE all-reduce per dtype (the
reference issues one per leaf), and ``sync_object`` packs all scalar fields of
a state into one all-reduce per reduction op instead of one per field.

Parity: packages/opaque-engine/src/opaque/api/engine/distributed/collectives.py,
gradients.py:46-193, _state.py:122-570, _shard.py:18-55.
"""
from __future__ import annotations

import dataclasses
import hashlib
import inspect
from collections.abc import Callable, Mapping, Sequence
from typing import Any

import torch
import torch.distributed as dist

from ..pytree import tree_flatten, tree_leaves, tree_map, tree_unflatten
from ..types import ClippedPytree, NoisedPytree, PerGroup, SecondMomentClippingOutput

_OPS = {"sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN,
        "product": dist.ReduceOp.PRODUCT, "mean": dist.ReduceOp.SUM}


def is_distributed() -> bool:
    """True when a process group with more than one rank is initialised."""
    return dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1


def get_rank() -> int:
    """Rank of this process (0 without a process group)."""
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def get_world_size() -> int:
    """Number of processes (1 without a process group)."""
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


process_index = get_rank
num_processes = get_world_size


def is_main_process() -> bool:
    """True on rank 0."""
    return get_rank() == 0


def barrier() -> None:
    """Block until every rank arrives (no-op in a single process)."""
    if is_distributed():
        dist.barrier()


wait_for_everyone = barrier


def _comm_device(device: torch.device | None = None) -> torch.device:
    """Where collective payloads must live for the active backend."""
    if device is not None:
        return torch.device(device)
    if dist.is_initialized() and dist.get_backend() == "nccl":
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


def all_reduce_(tensor: torch.Tensor, op: str = "sum") -> torch.Tensor:
    """In-place all-reduce (``mean`` = sum then divide); identity without a group."""
    if op not in _OPS:
        raise ValueError(f"unknown reduction op {op!r}; expected one of {sorted(_OPS)}")
    if not is_distributed():
        return tensor
    dist.all_reduce(tensor, op=_OPS[op])
    if op == "mean":
        tensor.div_(get_world_size())
    return tensor


def all_reduce(tensor: torch.Tensor, op: str = "sum") -> torch.Tensor:
    """Out-of-place ``all_reduce_``: returns the reduced copy of ``tensor``."""
    return all_reduce_(tensor.clone(), op)


def gather_for_metrics(tensor: torch.Tensor) -> torch.Tensor:
    """Concatenate a same-shaped tensor from every rank along dim 0."""
    if not is_distributed():
        return tensor
    t = tensor.contiguous()
    if t.ndim == 0:
        t = t[None]
    out = [torch.empty_like(t) for _ in range(get_world_size())]
    dist.all_gather(out, t)
    return torch.cat(out, dim=0)


# ----------------------------------------------------------------------------- scalars

def reduce_scalar(value: float | int, op: str = "sum", device: torch.device | None = None) -> float | int:
    """Reduce one Python scalar: integers stay exact (int64), floats use fp64 on CPU / fp32 on GPU."""
    if op not in _OPS:
        raise ValueError(f"unknown reduction op {op!r}")
    if not is_distributed():
        return value
    dev = _comm_device(device)
    is_int = isinstance(value, int) and not isinstance(value, bool)
    if is_int:
        dtype = torch.int64
    else:
        dtype = torch.float64 if dev.type == "cpu" else torch.float32
    t = torch.tensor([value], dtype=dtype, device=dev)
    dist.all_reduce(t, op=_OPS[op])
    out = t.item()
    if op == "mean":
        out = out / get_world_size()
    return int(out) if is_int and op != "mean" else float(out)


def _reduce_many(values: Sequence[float], op: str, device: torch.device | None) -> list[float]:
    dev = _comm_device(device)
    t = torch.tensor(list(values), dtype=torch.float64, device=dev)
    if dev.type != "cpu":
        # fp64 all-reduce is supported by NCCL and keeps int-valued counters exact to 2**53
        pass
    dist.all_reduce(t, op=_OPS[op])
    if op == "mean":
        t = t / get_world_size()
    return t.tolist()


def assert_scalar_equal(value: float | int, *, name: str = "value", atol: float = 0.0, rtol: float = 0.0,
                        compute_dtype: torch.dtype | None = None) -> None:
    """Raise on every rank when ``value`` differs anywhere (one packed min/max reduce)."""
    if not is_distributed():
        return
    lo, neg_hi = _reduce_many([float(value), -float(value)], "min", None)
    hi = -neg_hi
    if abs(hi - lo) > atol + rtol * max(abs(hi), abs(lo)):
        raise RuntimeError(f"{name} differs across ranks: min={lo!r} max={hi!r} (local {value!r})")


def _digest64(text: str) -> int:
    return int.from_bytes(hashlib.blake2b(text.encode(), digest_size=6).digest(), "little")


def assert_string_equal(value: str, *, name: str = "value") -> None:
    """Compare a string across ranks through a 48-bit hash (no pickled objects)."""
    if not is_distributed():
        return
    h = float(_digest64(value))
    lo, neg_hi = _reduce_many([h, -h], "min", None)
    if lo != -neg_hi:
        raise RuntimeError(f"{name} differs across ranks (local value {value!r})")


def _fingerprint(tree: Any) -> list[float]:
    total, sq, n = 0.0, 0.0, 0
    for x in tree_leaves(tree):
        if isinstance(x, torch.Tensor):
            xd = x.detach().double()
            total += float(xd.sum())
            sq += float((xd * xd).sum())
            n += x.numel()
    return [total, sq, float(n)]


def assert_pytree_equal(tree: Any, *, name: str = "pytree", atol: float = 0.0, rtol: float = 0.0) -> None:
    """Compare (sum, sum of squares, numel) fingerprints of a tree across ranks."""
    if not is_distributed():
        return
    fp = _fingerprint(tree)
    lows = _reduce_many(fp + [-v for v in fp], "min", None)
    k = len(fp)
    for i, label in enumerate(("sum", "sumsq", "numel")):
        lo, hi = lows[i], -lows[k + i]
        if abs(hi - lo) > atol + rtol * max(abs(hi), abs(lo)):
            raise RuntimeError(f"{name} {label} differs across ranks: min={lo!r} max={hi!r}")


# ----------------------------------------------------------------------------- gathers

def gather_tensors(tensor: torch.Tensor, *, dim: int = 0) -> torch.Tensor:
    """Concatenate possibly different-length tensors from all ranks (tensor collectives only).

    Lengths are exchanged with one small all-gather, payloads are padded to the
    longest and gathered with one tensor all-gather — no pickling and, on NCCL,
    no device-to-host copy of the payload.
    """
    if not is_distributed():
        return tensor
    world = get_world_size()
    dev = _comm_device()
    x = tensor.detach().movedim(dim, 0).contiguous().to(dev)
    sizes = torch.zeros(world, dtype=torch.int64, device=dev)
    mine = torch.tensor([x.shape[0]], dtype=torch.int64, device=dev)
    dist.all_gather_into_tensor(sizes, mine)
    sizes_l = sizes.tolist()
    cap = max(sizes_l)
    if cap == 0:
        return tensor
    padded = torch.zeros((cap,) + tuple(x.shape[1:]), dtype=x.dtype, device=dev)
    padded[: x.shape[0]] = x
    out = torch.empty((world * cap,) + tuple(x.shape[1:]), dtype=x.dtype, device=dev)
    dist.all_gather_into_tensor(out, padded)
    parts = [out[r * cap: r * cap + n] for r, n in enumerate(sizes_l)]
    return torch.cat(parts, dim=0).movedim(0, dim).to(tensor.device)


def gather_pytree(tree: Any, *, dim: int = 0) -> Any:
    """``gather_tensors`` applied to every tensor leaf of a tree."""
    return tree_map(lambda x: gather_tensors(x, dim=dim) if isinstance(x, torch.Tensor) else x, tree)


# ----------------------------------------------------------------------------- gradients

def _bound_key(b: Any) -> list[float]:
    if b is None:
        return [-1.0]
    if isinstance(b, PerGroup):
        return [float(v) for _, v in sorted(b.values.items())]
    return [float(b)]


def _check_metadata(tree: ClippedPytree) -> None:
    vals = _bound_key(tree.max_norm) + _bound_key(getattr(tree, "noise_stddev", None))
    lows = _reduce_many(vals + [-v for v in vals], "min", None)
    k = len(vals)
    for i in range(k):
        if lows[i] != -lows[k + i]:
            raise RuntimeError("clipping / noise metadata (max_norm, noise_stddev) differs across ranks")


def _scale_meta(b: Any, f: float) -> Any:
    if b is None:
        return None
    return b * f if isinstance(b, PerGroup) else float(b) * f


def _packed_all_reduce_(leaves: list[torch.Tensor], op: str) -> None:
    """One all-reduce per dtype over a flat concatenation of the leaves."""
    by_dtype: dict[tuple, list[torch.Tensor]] = {}
    for x in leaves:
        by_dtype.setdefault((x.dtype, x.device), []).append(x)
    for group in by_dtype.values():
        if len(group) == 1 and group[0].is_contiguous():
            all_reduce_(group[0], op)
            continue
        flat = torch.cat([g.reshape(-1) for g in group])
        all_reduce_(flat, op)
        off = 0
        for g in group:
            g.copy_(flat[off: off + g.numel()].view_as(g))
            off += g.numel()


def reduce_pytree_(pytree: Any, op: str = "sum", *, check_metadata: bool = True) -> Any:
    """In-place cross-rank reduction of a (wrapped) gradient tree.

    ``sum`` keeps ``max_norm`` (each record lives on one rank) and multiplies a
    noise σ by √W (independent noises add in variance); ``mean`` divides both by W.
    """
    tree = pytree
    if op not in ("sum", "mean"):
        raise ValueError("reduce_pytree_ supports op='sum' or 'mean'")
    if isinstance(tree, SecondMomentClippingOutput):
        return SecondMomentClippingOutput(reduce_pytree_(tree.grads, op, check_metadata=check_metadata),
                                          reduce_pytree_(tree.squared_grads, op, check_metadata=check_metadata))
    if not is_distributed():
        return tree
    world = get_world_size()
    wrapped = isinstance(tree, ClippedPytree)
    inner = tree.pytree if wrapped else tree
    if wrapped and check_metadata:
        _check_metadata(tree)
    leaves = [x for x in tree_leaves(inner) if isinstance(x, torch.Tensor)]
    _packed_all_reduce_(leaves, op)
    if not wrapped:
        return tree
    if isinstance(tree, NoisedPytree):
        f_noise = world ** 0.5 if op == "sum" else world ** -0.5
        f_norm = 1.0 if op == "sum" else 1.0 / world
        return dataclasses.replace(tree, max_norm=_scale_meta(tree.max_norm, f_norm),
                                   noise_stddev=_scale_meta(tree.noise_stddev, f_noise))
    if op == "mean":
        return dataclasses.replace(tree, max_norm=_scale_meta(tree.max_norm, 1.0 / world))
    return tree


def reduce_pytree(pytree: Any, op: str = "sum", **kw: Any) -> Any:
    """Out-of-place ``reduce_pytree_``."""
    tree = pytree
    if isinstance(tree, SecondMomentClippingOutput):
        return SecondMomentClippingOutput(reduce_pytree(tree.grads, op, **kw), reduce_pytree(tree.squared_grads, op, **kw))
    cloned = tree.clone() if isinstance(tree, ClippedPytree) else tree_map(
        lambda x: x.clone() if isinstance(x, torch.Tensor) else x, tree)
    return reduce_pytree_(cloned, op, **kw)


def sum_gradients_(gradients: Any) -> Any:
    """Sum a ``ClippedPytree`` over ranks in place (one packed all-reduce); the sensitivity metadata must agree on every rank."""
    tree = gradients
    return reduce_pytree_(tree, "sum")


def sum_gradients(gradients: Any) -> Any:
    """Out-of-place ``sum_gradients_``."""
    tree = gradients
    return reduce_pytree(tree, "sum")


# ----------------------------------------------------------------------------- state sync

_VALID = {"sum", "mean", "max", "min", "product", "assert_equal", "assert_optional_equal", "local"}


def _validate_op(name: str, op: Any) -> None:
    if isinstance(op, str):
        if op not in _VALID:
            raise ValueError(f"field_ops[{name!r}]={op!r} is not one of {sorted(_VALID)}")
        return
    if not callable(op):
        raise ValueError(f"field_ops[{name!r}] must be an op name or a callable fn(value, device)")
    try:
        inspect.signature(op, follow_wrapped=False).bind(None, None)
    except TypeError as err:
        raise ValueError(f"field_ops[{name!r}] must be callable as fn(value, device): {err}") from err
    except ValueError:
        pass


def sync_object(state: Any, field_ops: Mapping[str, Any], device: torch.device | None = None) -> Any:
    """Reduce the scalar fields of a dataclass across ranks; returns a new instance.

    The whole schema is validated on every rank BEFORE any collective is issued
    (a rank with a bad schema raises instead of leaving the others waiting), and
    fields are processed in declaration order.  Fields sharing a reduction op
    travel in one packed all-reduce.
    """
    if not dataclasses.is_dataclass(state) or isinstance(state, type):
        raise TypeError(f"state must be a dataclass instance, got {type(state)}")
    flds = dataclasses.fields(state)
    names = {f.name for f in flds}
    unknown, missing = set(field_ops) - names, names - set(field_ops)
    if unknown or missing:
        parts = []
        if unknown:
            parts.append(f"unknown fields: {sorted(unknown)}")
        if missing:
            parts.append(f"missing fields: {sorted(missing)}")
        raise ValueError("field_ops must define every dataclass field; " + "; ".join(parts) + ".")
    for f in flds:
        _validate_op(f.name, field_ops[f.name])
    # type checks are also schema checks: do them before touching the network
    for f in flds:
        op, v = field_ops[f.name], getattr(state, f.name)
        if isinstance(op, str) and op not in ("local", "assert_optional_equal"):
            if isinstance(v, bool) or not isinstance(v, (int, float)):
                raise TypeError(f"field_ops[{f.name!r}]={op!r} requires a float or int, got {type(v).__name__}.")
        if op == "assert_optional_equal" and v is not None and (isinstance(v, bool) or not isinstance(v, (int, float))):
            raise TypeError(f"field_ops[{f.name!r}]='assert_optional_equal' requires a float, int or None.")
    if not is_distributed():
        return state

    updates: dict[str, Any] = {}
    packed: dict[str, list[tuple[str, Any]]] = {}
    equal_checks: list[tuple[str, float]] = []
    for f in flds:
        op, v = field_ops[f.name], getattr(state, f.name)
        if op == "local":
            continue
        if callable(op):
            res = op(v, device)
            if isinstance(res, bool) or not isinstance(res, (int, float)):
                continue
            if isinstance(v, bool):
                raise TypeError(f"Callable field_ops[{f.name!r}] cannot update a bool field")
            updates[f.name] = int(res) if isinstance(v, int) else float(res)
        elif op == "assert_equal":
            equal_checks.append((f.name, float(v)))
        elif op == "assert_optional_equal":
            equal_checks.append((f.name + "?", float(v is not None)))
            equal_checks.append((f.name, float(v) if v is not None else 0.0))
        else:
            packed.setdefault(op, []).append((f.name, v))
    if equal_checks:
        vals = [v for _, v in equal_checks]
        lows = _reduce_many(vals + [-v for v in vals], "min", device)
        for i, (nm, _) in enumerate(equal_checks):
            if lows[i] != -lows[len(vals) + i]:
                what = "presence" if nm.endswith("?") else "value"
                raise RuntimeError(f"{type(state).__name__}.{nm.rstrip('?')} {what} mismatch across ranks.")
    for op, items in packed.items():
        red = _reduce_many([float(v) for _, v in items], op, device)
        for (nm, v), r in zip(items, red):
            updates[nm] = int(round(r)) if isinstance(v, int) else float(r)
    if updates:
        state = dataclasses.replace(state, **updates)
    return state


_SYNC_REGISTRY: dict[type, Callable[[Any], Any]] = {}


def register_sync_type(state_type: type, sync_fn: Callable[[Any], Any]) -> None:
    """Make ``sync()`` able to handle ``state_type`` (and its subclasses via the MRO)."""
    _SYNC_REGISTRY[state_type] = sync_fn


def _sync_one(state: Any) -> Any:
    for base in type(state).__mro__:
        fn = _SYNC_REGISTRY.get(base)
        if fn is not None:
            return fn(state)
    raise TypeError(f"no sync function registered for {type(state).__name__}; use register_sync_type")


def sync(*states: Any) -> Any:
    """Synchronise one or more state objects; types are resolved before any collective runs."""
    for s in states:
        if not any(b in _SYNC_REGISTRY for b in type(s).__mro__):
            raise TypeError(f"no sync function registered for {type(s).__name__}; use register_sync_type")
    out = tuple(_sync_one(s) for s in states)
    return out[0] if len(out) == 1 else out


# ----------------------------------------------------------------------------- sharding

def local_shard(dataset: Any, *, rank: int | None = None, world_size: int | None = None) -> Any:
    """Contiguous slice of ``dataset`` for this rank; the last rank takes the remainder."""
    r = get_rank() if rank is None else rank
    w = get_world_size() if world_size is None else world_size
    if w < 1 or not 0 <= r < w:
        raise ValueError(f"invalid rank/world_size: {r}/{w}")
    n = len(dataset)
    per = n // w
    lo = r * per
    hi = n if r == w - 1 else lo + per
    if isinstance(dataset, (torch.Tensor, list, tuple)) or hasattr(dataset, "__array__"):
        return dataset[lo:hi]
    if isinstance(dataset, torch.utils.data.Dataset):
        return torch.utils.data.Subset(dataset, range(lo, hi))
    return dataset[lo:hi]


__all__ = [
    "all_reduce", "all_reduce_", "assert_pytree_equal", "assert_scalar_equal", "assert_string_equal",
    "barrier", "gather_for_metrics", "gather_pytree", "gather_tensors", "get_rank", "get_world_size",
    "is_distributed", "is_main_process", "local_shard", "num_processes", "process_index",
    "reduce_pytree", "reduce_pytree_", "reduce_scalar", "register_sync_type", "sum_gradients",
    "sum_gradients_", "sync", "sync_object", "wait_for_everyone",
]

from ..utils.namespaces import submodule as _sub  # noqa: E402

_sub(__name__, "collectives", "Thin collectives.", {"all_reduce": all_reduce, "all_reduce_": all_reduce_, "barrier": barrier, "get_rank": get_rank,
                                                   "get_world_size": get_world_size, "is_distributed": is_distributed})
_sub(__name__, "gradients", "Gradient reductions over ranks.", {"reduce_pytree": reduce_pytree, "reduce_pytree_": reduce_pytree_,
                                                               "sum_gradients": sum_gradients, "sum_gradients_": sum_gradients_})
