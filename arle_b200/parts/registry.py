"""Registry from a part spec's ``kind`` to the class that builds the part.

A new mixer, feed-forward, norm, position encoding or block arrangement is added
by writing its spec (a frozen dataclass with a class attribute ``kind``) and its
class, and calling ``register_part(kind, cls)``; nothing else in the package has
to change.  ``build_part(spec)`` is the only way parts are constructed.
"""
from __future__ import annotations

_PARTS = {}


def register_part(kind: str, cls: type) -> None:
    _PARTS[kind] = cls


def registered_parts():
    return sorted(_PARTS)


def build_part(spec):
    kind = getattr(spec, "kind", None)
    if kind not in _PARTS:
        raise KeyError(f"no part registered for kind {kind!r}; registered: {', '.join(registered_parts())}")
    return _PARTS[kind](spec)
