"""A small self-contained pytree library (dict / list / tuple / NamedTuple / dataclass).

The reference delegates to ``optree``; this framework owns its tree walker so
the DP pipeline has no third-party dependency.  Dict children are visited in
sorted-key order (as optree does), ``None`` is an empty subtree, and a leaf is
anything that is not one of the container kinds.

Parity: packages/opaque-engine/src/opaque/api/engine/pytree.py (``global_norm``
at :336-432 accumulates in at least fp32 and combines leaves in fp64).
"""
from __future__ import annotations

import dataclasses
from collections import OrderedDict
from collections.abc import Callable, Iterable
from typing import Any

import torch

ParamPath = tuple[Any, ...]


def param_path(key: Any) -> ParamPath:
    """Normalise ``"a"`` → ``("a",)``; tuples pass through."""
    if isinstance(key, tuple):
        return key
    return (key,)


def param_path_display(path: ParamPath) -> str:
    """Dotted display form, integers rendered as ``[i]``."""
    out = ""
    for seg in path:
        if isinstance(seg, int):
            out += f"[{seg}]"
        else:
            out += ("." if out else "") + str(seg)
    return out


@dataclasses.dataclass(frozen=True)
class TreeDef:
    """Structure of a pytree: node kind, construction metadata and child defs."""

    kind: str                      # leaf | none | dict | odict | list | tuple | namedtuple | dataclass
    meta: Any = None               # keys / class
    children: tuple["TreeDef", ...] = ()

    @property
    def num_leaves(self) -> int:
        if self.kind == "leaf":
            return 1
        return sum(c.num_leaves for c in self.children)


_LEAF = TreeDef("leaf")
_NONE = TreeDef("none")


def _is_namedtuple(x: Any) -> bool:
    return isinstance(x, tuple) and hasattr(type(x), "_fields")


def _is_registered_dataclass(x: Any) -> bool:
    return type(x) in _DATACLASS_NODES


_DATACLASS_NODES: set[type] = set()


def register_dataclass_node(cls: type) -> type:
    """Opt a dataclass in as an *internal* node (its fields are children)."""
    _DATACLASS_NODES.add(cls)
    return cls


def _split(node: Any):
    """Return ``(kind, meta, [(key, child), ...])`` or None for a leaf."""
    if node is None:
        return "none", None, []
    if isinstance(node, OrderedDict):
        keys = list(node.keys())
        return "odict", tuple(keys), [(k, node[k]) for k in keys]
    if isinstance(node, dict):
        try:
            keys = sorted(node.keys())
        except TypeError:
            keys = list(node.keys())
        return "dict", tuple(keys), [(k, node[k]) for k in keys]
    if _is_namedtuple(node):
        return "namedtuple", type(node), [(f, getattr(node, f)) for f in type(node)._fields]
    if isinstance(node, tuple):
        return "tuple", None, list(enumerate(node))
    if isinstance(node, list):
        return "list", None, list(enumerate(node))
    if _is_registered_dataclass(node):
        names = [f.name for f in dataclasses.fields(node)]
        return "dataclass", (type(node), tuple(names)), [(n, getattr(node, n)) for n in names]
    return None


def tree_flatten_with_paths(tree: Any, is_leaf: Callable[[Any], bool] | None = None):
    """Return ``(paths, leaves, treedef)`` in deterministic depth-first order."""
    paths: list[ParamPath] = []
    leaves: list[Any] = []

    def rec(node: Any, path: ParamPath) -> TreeDef:
        if is_leaf is not None and is_leaf(node):
            paths.append(path)
            leaves.append(node)
            return _LEAF
        parts = _split(node)
        if parts is None:
            paths.append(path)
            leaves.append(node)
            return _LEAF
        kind, meta, kids = parts
        if kind == "none":
            return _NONE
        return TreeDef(kind, meta, tuple(rec(c, path + (k,)) for k, c in kids))

    td = rec(tree, ())
    return paths, leaves, td


def tree_flatten(tree: Any, is_leaf: Callable[[Any], bool] | None = None):
    """Leaves of ``tree`` in a fixed order, and the structure that ``tree_unflatten`` needs to rebuild it."""
    _, leaves, td = tree_flatten_with_paths(tree, is_leaf)
    return leaves, td


def tree_leaves(tree: Any, is_leaf: Callable[[Any], bool] | None = None) -> list[Any]:
    """Leaves of ``tree`` in the order ``tree_flatten`` uses."""
    return tree_flatten(tree, is_leaf)[0]


def tree_structure(tree: Any, is_leaf: Callable[[Any], bool] | None = None) -> TreeDef:
    """The structure of ``tree`` without its leaves."""
    return tree_flatten(tree, is_leaf)[1]


def tree_unflatten(treedef: TreeDef, leaves: Iterable[Any]) -> Any:
    """Rebuild a tree from a structure and a sequence of leaves."""
    it = iter(leaves)

    def rec(td: TreeDef) -> Any:
        k = td.kind
        if k == "leaf":
            return next(it)
        if k == "none":
            return None
        kids = [rec(c) for c in td.children]
        if k == "dict":
            return dict(zip(td.meta, kids))
        if k == "odict":
            return OrderedDict(zip(td.meta, kids))
        if k == "list":
            return kids
        if k == "tuple":
            return tuple(kids)
        if k == "namedtuple":
            return td.meta(*kids)
        if k == "dataclass":
            cls, names = td.meta
            return cls(**dict(zip(names, kids)))
        raise ValueError(f"unknown tree node kind {k!r}")

    out = rec(treedef)
    return out


def tree_map(fn: Callable[..., Any], tree: Any, *rest: Any,
             is_leaf: Callable[[Any], bool] | None = None) -> Any:
    """Apply ``fn`` leaf-wise; extra trees must share ``tree``'s structure."""
    leaves, td = tree_flatten(tree, is_leaf)
    others = []
    for other in rest:
        o_leaves, o_td = tree_flatten(other, is_leaf)
        if len(o_leaves) != len(leaves):
            raise ValueError("tree_map: trees do not have the same structure")
        others.append(o_leaves)
    return tree_unflatten(td, [fn(*xs) for xs in zip(leaves, *others)])


def tree_map_with_path(fn: Callable[..., Any], tree: Any, *rest: Any,
                       is_leaf: Callable[[Any], bool] | None = None) -> Any:
    """Like :func:`tree_map` but ``fn(path, leaf, *others)``."""
    paths, leaves, td = tree_flatten_with_paths(tree, is_leaf)
    others = [tree_flatten(o, is_leaf)[0] for o in rest]
    for o in others:
        if len(o) != len(leaves):
            raise ValueError("tree_map_with_path: trees do not have the same structure")
    return tree_unflatten(td, [fn(p, *xs) for p, *xs in zip(paths, leaves, *others)])


def partition(predicate: Callable[[ParamPath, Any], bool], tree: Any):
    """Split ``tree`` into two trees of identical structure.

    Leaves failing the predicate become ``None`` in the first tree and vice
    versa, so :func:`merge` can zip them back together.
    """
    paths, leaves, td = tree_flatten_with_paths(tree)
    keep = [predicate(p, x) for p, x in zip(paths, leaves)]
    yes = _unflatten_sparse(td, [x if k else None for x, k in zip(leaves, keep)])
    no = _unflatten_sparse(td, [None if k else x for x, k in zip(leaves, keep)])
    return yes, no


def _unflatten_sparse(td: TreeDef, leaves: list[Any]) -> Any:
    return tree_unflatten(td, leaves)


def merge(*trees: Any) -> Any:
    """Inverse of :func:`partition`: first non-``None`` leaf wins per position."""
    if not trees:
        raise ValueError("merge() needs at least one tree")

    def rec(nodes: list[Any]) -> Any:
        present = [n for n in nodes if n is not None]
        if not present:
            return None
        first = present[0]
        parts = _split(first)
        if parts is None:
            return first
        kind, meta, kids = parts
        merged_children = []
        for key, _ in kids:
            sub = []
            for n in nodes:
                if n is None:
                    sub.append(None)
                elif kind in ("dict", "odict"):
                    sub.append(n.get(key))
                elif kind in ("namedtuple", "dataclass"):
                    sub.append(getattr(n, key))
                else:
                    sub.append(n[key])
            merged_children.append(rec(sub))
        if kind == "dict":
            return dict(zip(meta, merged_children))
        if kind == "odict":
            return OrderedDict(zip(meta, merged_children))
        if kind == "list":
            return merged_children
        if kind == "tuple":
            return tuple(merged_children)
        if kind == "namedtuple":
            return meta(*merged_children)
        cls, names = meta
        return cls(**dict(zip(names, merged_children)))

    return rec(list(trees))


def _acc_dtype(dtype: torch.dtype) -> torch.dtype:
    return torch.float64 if dtype == torch.float64 else torch.float32


def global_norm(tree: Any, *, accumulate_dtype: torch.dtype | None = None) -> torch.Tensor:
    """L2 norm over every tensor leaf.

    Each leaf's sum of squares is taken in at least fp32; the cross-leaf sum is
    carried in fp64 (fp32 where the device has no fp64, e.g. MPS) so a model
    with thousands of leaves does not lose low-order bits.
    """
    leaves = [x for x in tree_leaves(tree) if isinstance(x, torch.Tensor)]
    if not leaves:
        return torch.zeros((), dtype=torch.float32)
    dev = leaves[0].device
    wide = torch.float32 if dev.type == "mps" else torch.float64
    if accumulate_dtype is not None:
        wide = accumulate_dtype
    total = torch.zeros((), dtype=wide, device=dev)
    for x in leaves:
        xs = x.detach().to(_acc_dtype(x.dtype))
        total = total + (xs * xs).sum().to(wide)
    out_dtype = torch.float64 if all(x.dtype == torch.float64 for x in leaves) else torch.float32
    return total.sqrt().to(out_dtype)


__all__ = [
    "ParamPath", "TreeDef", "global_norm", "merge", "param_path", "param_path_display",
    "partition", "register_dataclass_node", "tree_flatten", "tree_flatten_with_paths",
    "tree_leaves", "tree_map", "tree_map_with_path", "tree_structure", "tree_unflatten",
]
