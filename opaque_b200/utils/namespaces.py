"""Sub-namespaces that exist for import-path parity with the reference library.

The reference spreads some façades over small sub-packages (``opaque.alignment.dpo.loss``, ``opaque.dpsgd.accounting.
mechanisms``, ``opaque.auditing.one_run``, …).  Here those names live in one module per façade; :func:`submodule` makes
the deeper import paths work as well — ``from opaque_b200.alignment.dpo.loss import sigmoid_loss`` — by registering a
module object under the dotted name (``import a.b.c`` looks in ``sys.modules`` before it asks ``a.b`` for a path).
"""
from __future__ import annotations

import sys
import types
from typing import Any, Callable


class _CallableModule(types.ModuleType):
    """A namespace that can also be called (``auditing.one_run(...)`` is a function AND ``auditing.one_run.one_run`` exists)."""

    _call: Callable[..., Any] | None = None

    def __call__(self, *args: Any, **kwargs: Any) -> Any:
        if self._call is None:
            raise TypeError(f"module {self.__name__!r} is not callable")
        return self._call(*args, **kwargs)


def submodule(parent: str, name: str, doc: str, members: dict[str, Any], *, bind: bool = True,
              call: Callable[..., Any] | None = None) -> types.ModuleType:
    """Register ``{parent}.{name}`` holding ``members``; ``bind`` also sets it as an attribute of the parent module (leave
    it off where the attribute name is taken by something else, e.g. a global import of the parent).  ``call`` makes the
    namespace itself callable."""
    full = f"{parent}.{name}"
    mod = _CallableModule(full, doc) if call is not None else types.ModuleType(full, doc)
    if call is not None:
        mod._call = call
    for key, value in members.items():
        setattr(mod, key, value)
    mod.__all__ = sorted(members)
    mod.__package__ = parent
    sys.modules[full] = mod
    if bind and parent in sys.modules:
        setattr(sys.modules[parent], name, mod)
    return mod


__all__ = ["submodule"]
