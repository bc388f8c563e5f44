"""Minimal stand-in for the third-party ``optree`` package (only what the reference arm calls).

Semantics follow optree's defaults: ``dict`` keys are visited in sorted order, ``None`` is an internal node without
leaves, tuples / lists / namedtuples / OrderedDict / defaultdict are nodes, everything else is a leaf.
"""
from __future__ import annotations

import collections
from typing import Any, Callable

__version__ = "0.0-standin"


def _is_namedtuple(x: Any) -> bool:
    return isinstance(x, tuple) and hasattr(type(x), "_fields")


def _sorted_keys(d: dict) -> list:
    try:
        return sorted(d)
    except TypeError:
        return list(d)


class PyTreeSpec:
    """Structure of a pytree: node kind, node metadata and child specs (``kind == 'leaf'`` for leaves)."""

    __slots__ = ("kind", "meta", "children", "num_leaves")

    def __init__(self, kind: str, meta: Any, children: list["PyTreeSpec"]):
        self.kind, self.meta, self.children = kind, meta, children
        self.num_leaves = 1 if kind == "leaf" else sum(c.num_leaves for c in children)

    def _key(self):
        meta = self.meta
        if self.kind == "dict":
            meta = (meta[0], tuple(meta[1]))
        return (self.kind, meta, tuple(c._key() for c in self.children))

    def __eq__(self, other):
        return isinstance(other, PyTreeSpec) and self._key() == other._key()

    def __ne__(self, other):
        return not self == other

    def __hash__(self):
        try:
            return hash(self._key())
        except TypeError:
            return hash((self.kind, self.num_leaves))

    def __repr__(self):
        return f"PyTreeSpec({self._render()})"

    def _render(self) -> str:
        if self.kind == "leaf":
            return "*"
        if self.kind == "none":
            return "None"
        inner = [c._render() for c in self.children]
        if self.kind == "dict":
            return "{" + ", ".join(f"{k!r}: {v}" for k, v in zip(self.meta[1], inner)) + "}"
        if self.kind == "list":
            return "[" + ", ".join(inner) + "]"
        return "(" + ", ".join(inner) + ")"

    def unflatten(self, leaves):
        return tree_unflatten(self, leaves)


def _flatten(tree: Any, leaves: list, paths: list | None, path: tuple, is_leaf: Callable | None) -> PyTreeSpec:
    if is_leaf is not None and is_leaf(tree):
        leaves.append(tree)
        if paths is not None:
            paths.append(path)
        return PyTreeSpec("leaf", None, [])
    if tree is None:
        return PyTreeSpec("none", None, [])
    if isinstance(tree, dict):
        keys = list(tree) if isinstance(tree, collections.OrderedDict) else _sorted_keys(tree)
        kids = [_flatten(tree[k], leaves, paths, path + (k,), is_leaf) for k in keys]
        extra = tree.default_factory if isinstance(tree, collections.defaultdict) else None
        return PyTreeSpec("dict", ((type(tree), extra), keys), kids)
    if _is_namedtuple(tree):
        kids = [_flatten(v, leaves, paths, path + (i,), is_leaf) for i, v in enumerate(tree)]
        return PyTreeSpec("namedtuple", type(tree), kids)
    if isinstance(tree, (list, tuple)):
        kids = [_flatten(v, leaves, paths, path + (i,), is_leaf) for i, v in enumerate(tree)]
        return PyTreeSpec("list" if isinstance(tree, list) else "tuple", type(tree), kids)
    leaves.append(tree)
    if paths is not None:
        paths.append(path)
    return PyTreeSpec("leaf", None, [])


def tree_flatten(tree: Any, is_leaf: Callable | None = None, **_: Any):
    leaves: list = []
    spec = _flatten(tree, leaves, None, (), is_leaf)
    return leaves, spec


def tree_flatten_with_path(tree: Any, is_leaf: Callable | None = None, **_: Any):
    leaves: list = []
    paths: list = []
    spec = _flatten(tree, leaves, paths, (), is_leaf)
    return paths, leaves, spec


def tree_leaves(tree: Any, is_leaf: Callable | None = None, **_: Any) -> list:
    return tree_flatten(tree, is_leaf)[0]


def tree_structure(tree: Any, is_leaf: Callable | None = None, **_: Any) -> PyTreeSpec:
    return tree_flatten(tree, is_leaf)[1]


def _build(spec: PyTreeSpec, it) -> Any:
    if spec.kind == "leaf":
        return next(it)
    if spec.kind == "none":
        return None
    kids = [_build(c, it) for c in spec.children]
    if spec.kind == "dict":
        (cls, extra), keys = spec.meta
        if cls is collections.defaultdict:
            return collections.defaultdict(extra, zip(keys, kids))
        return cls(zip(keys, kids))
    if spec.kind == "namedtuple":
        return spec.meta(*kids)
    return spec.meta(kids)


def tree_unflatten(treespec: PyTreeSpec, leaves) -> Any:
    leaves = list(leaves)
    if len(leaves) != treespec.num_leaves:
        raise ValueError(f"treespec expects {treespec.num_leaves} leaves, got {len(leaves)}")
    return _build(treespec, iter(leaves))


def tree_map(func: Callable, tree: Any, *rests: Any, is_leaf: Callable | None = None, **_: Any) -> Any:
    leaves, spec = tree_flatten(tree, is_leaf)
    cols = [leaves]
    for other in rests:
        ol, ospec = tree_flatten(other, is_leaf)
        if ospec != spec:
            raise ValueError(f"tree structures differ: {spec} vs {ospec}")
        cols.append(ol)
    return tree_unflatten(spec, [func(*xs) for xs in zip(*cols)])


def tree_map_(func: Callable, tree: Any, *rests: Any, is_leaf: Callable | None = None, **_: Any) -> Any:
    tree_map(func, tree, *rests, is_leaf=is_leaf)
    return tree
