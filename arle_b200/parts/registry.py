"""Registry from a part spec's ``kind`` to the class that builds the part.

A new mixer, feed-forward, norm, position encoding or block arrangement is added
by writing its spec (a frozen dataclass with a class attribute ``kind``) and its
class, and calling ``register_part(kind, cls)``; nothing else in the package has
to change.  ``build_part(spec)`` is the only way parts are constructed.

Whole models are registered the same way: a ``ModelSpec`` names the ``kind`` of the
class that is built from it (``"decoder"`` unless it says otherwise), so an
architecture whose arrangement around the blocks differs (a scaled embedding,
capped logits) brings a class of its own with ``register_model(kind, cls)``.
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


_MODELS = {}


def register_model(kind: str, cls: type) -> None:
    """``cls(spec)`` must offer what ``DecoderModel`` offers the engine: ``spec``, ``dtype``,
    ``cache_needs``, ``state_needs``, ``weight_decls()``, ``load(tensors, dtype, device)``,
    ``forward(ctx) -> float32 logits at ctx.want_rows`` and ``weight_bytes_per_step()``."""
    _MODELS[kind] = cls


def registered_models():
    return sorted(_MODELS)


def build_model(spec):
    kind = getattr(spec, "kind", "decoder")
    if kind not in _MODELS:
        raise KeyError(f"no model class registered for kind {kind!r}; registered: {', '.join(registered_models())}")
    return _MODELS[kind](spec)
