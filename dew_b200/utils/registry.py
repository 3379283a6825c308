"""One alias registry per kind: ``register("name")`` decorators and loud lookups.

Unknown names raise with the list of known ones (reference: src/dew/registry.py; design rule
"unknown names/fields raise", docs/design/api.md:43-52).
"""
from __future__ import annotations

from typing import Any, Callable, Dict

_REGISTRIES: Dict[str, Dict[str, Any]] = {}


def registry(kind: str) -> Dict[str, Any]:
    return _REGISTRIES.setdefault(kind, {})


def register(name: str, kind: str = "model") -> Callable[[Any], Any]:
    def deco(obj: Any) -> Any:
        table = registry(kind)
        if name in table and table[name] is not obj:
            raise ValueError(f"{kind} {name!r} is already registered")
        table[name] = obj
        return obj
    return deco


def lookup(name: str, kind: str = "model") -> Any:
    table = registry(kind)
    if name not in table:
        raise KeyError(f"unknown {kind} {name!r}; known: {sorted(table)}")
    return table[name]
