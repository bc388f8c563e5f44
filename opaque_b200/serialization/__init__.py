"""Flat, path-keyed state dictionaries for any state object.

``state_dict(obj)`` flattens an object into ``{"a.b[0].c": leaf}``;
``from_state_dict(template, sd)`` rebuilds an object of the template's shape.
Types with a registered handler are serialised by that handler (exact type
first, then the MRO); containers and primitives are walked structurally; any
other leaf raises ``TypeError`` so state is never dropped silently.

Parity: packages/opaque-base/src/opaque/api/base/serialization/_dispatch.py:83-106,
_registry.py:27-81, _structural.py:50-115.
"""
from __future__ import annotations

import dataclasses
from collections.abc import Callable, Mapping
from typing import Any

SerializedState = dict[str, Any]
StateDictFn = Callable[[Any], SerializedState]
FromStateDictFn = Callable[[Any, Mapping[str, Any]], Any]
Serializer = tuple[StateDictFn, FromStateDictFn]

_HANDLERS: dict[type, Serializer] = {}
_SCALARS = (bool, int, float, str, type(None))


def register_serializer(typ: type, state_dict_fn: StateDictFn, from_state_dict_fn: FromStateDictFn) -> None:
    """Attach a ``(save, load)`` pair to ``typ`` (and, through the MRO, its subclasses).

    ``state_dict_fn(obj)`` returns keys *relative* to the object (``""`` occupies the
    object's own slot); ``from_state_dict_fn(template, sub)`` receives the same relative keys.
    """
    _HANDLERS[typ] = (state_dict_fn, from_state_dict_fn)


def register_template_restored(typ: type) -> None:
    """Declare ``typ`` inert: nothing is written and the template's value is reused."""
    _HANDLERS[typ] = (lambda obj: {}, lambda template, sub: template)


def lookup_serializer(typ: type) -> Serializer | None:
    """Exact-type lookup only."""
    return _HANDLERS.get(typ)


def resolve_serializer(typ: type) -> Serializer | None:
    """Exact type, then each base class in MRO order."""
    cls = typ
    for base in getattr(cls, "__mro__", (cls,)):
        hit = _HANDLERS.get(base)
        if hit is not None:
            return hit
    return None


def _child(prefix: str, part: str) -> str:
    if not prefix:
        return part
    if not part:
        return prefix
    return prefix + part if part[0] == "[" else prefix + "." + part


def _slice(sd: Mapping[str, Any], prefix: str) -> dict[str, Any]:
    if not prefix:
        return dict(sd)
    n = len(prefix)
    picked: dict[str, Any] = {}
    for key, value in sd.items():
        if not key.startswith(prefix):
            continue
        rest = key[n:]
        if rest == "":
            picked[""] = value
        elif rest[0] == ".":
            picked[rest[1:]] = value
        elif rest[0] == "[":
            picked[rest] = value
    return picked


def _is_namedtuple(x: Any) -> bool:
    return isinstance(x, tuple) and hasattr(type(x), "_fields")


def _children(node: Any):
    """Yield ``(relative_key, child)`` pairs of a structural container, or None."""
    if dataclasses.is_dataclass(node) and not isinstance(node, type):
        return [(f.name, getattr(node, f.name)) for f in dataclasses.fields(node)]
    if _is_namedtuple(node):
        return [(name, getattr(node, name)) for name in type(node)._fields]
    if isinstance(node, (tuple, list)):
        return [(f"[{i}]", v) for i, v in enumerate(node)]
    if isinstance(node, Mapping):
        return [(str(k), v) for k, v in node.items()]
    return None


def _fail(node: Any, where: str, verb: str) -> TypeError:
    loc = repr(where) if where else "the root"
    t = type(node)
    return TypeError(
        f"cannot {verb} a {t.__module__}.{t.__qualname__} at {loc}: no serializer is "
        "registered for it and it is neither a container nor a primitive; use "
        "register_serializer, or register_template_restored if it carries no run state"
    )


def state_dict(obj: Any) -> SerializedState:
    """Flatten ``obj`` into a path-keyed dict (iterative, safe for deep spines)."""
    out: SerializedState = {}
    stack: list[tuple[Any, str]] = [(obj, "")]
    while stack:
        node, where = stack.pop()
        handler = resolve_serializer(type(node))
        if handler is not None:
            for rel, val in handler[0](node).items():
                out[_child(where, rel)] = val
            continue
        kids = _children(node)
        if kids is not None:
            for rel, child in reversed(kids):
                stack.append((child, _child(where, rel)))
            continue
        if isinstance(node, _SCALARS):
            out[where] = node
            continue
        raise _fail(node, where, "serialize")
    return out


def _load(template: Any, sd: Mapping[str, Any], where: str) -> Any:
    handler = resolve_serializer(type(template))
    if handler is not None:
        try:
            return handler[1](template, _slice(sd, where))
        except Exception as exc:  # name the failing leaf for the caller
            exc.add_note(f"while restoring {where!r}" if where else "while restoring the root")
            raise
    if dataclasses.is_dataclass(template) and not isinstance(template, type):
        new = {f.name: _load(getattr(template, f.name), sd, _child(where, f.name))
               for f in dataclasses.fields(template) if f.init}
        return dataclasses.replace(template, **new)
    if _is_namedtuple(template):
        return type(template)(*(_load(getattr(template, n), sd, _child(where, n))
                                for n in type(template)._fields))
    if isinstance(template, tuple):
        return tuple(_load(v, sd, f"{where}[{i}]") for i, v in enumerate(template))
    if isinstance(template, list):
        return [_load(v, sd, f"{where}[{i}]") for i, v in enumerate(template)]
    if isinstance(template, Mapping):
        return {k: _load(v, sd, _child(where, str(k))) for k, v in template.items()}
    if isinstance(template, _SCALARS):
        return sd.get(where, template)
    raise _fail(template, where, "restore")


def from_state_dict(template: Any, sd: Mapping[str, Any]) -> Any:
    """Rebuild an object shaped like ``template`` from ``sd``.

    Leaves missing from ``sd`` keep the template's value, so files written
    before a field existed still load.
    """
    return _load(template, sd, "")


__all__ = [
    "FromStateDictFn", "SerializedState", "Serializer", "StateDictFn",
    "from_state_dict", "lookup_serializer", "register_serializer",
    "register_template_restored", "resolve_serializer", "state_dict",
]
