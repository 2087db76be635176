"""Registries of the parts a layer is assembled from, by kind.

A kind maps to a class; `LayerSpec` names kinds, never classes, and no part knows the
model it ends up in.  New parts register themselves here (also from outside the
package) and are then usable by any architecture's builder.

Interfaces (see `parts.base`):
  norm              Norm
  position encoding PositionEncoding
  mixer             Mixer
  feed-forward      FeedForward
  arrangement       Arrangement (how norms, mixer, feed-forward and residuals are wired; declares its roles)
  embedding         Embedding (token ids -> hidden stream)
  head              Head (hidden stream -> logits)
"""
from __future__ import annotations

_REGISTRIES: dict[str, dict] = {
    "norm": {}, "position": {}, "mixer": {}, "feed_forward": {}, "arrangement": {}, "embedding": {}, "head": {},
}


def register(category: str, kind: str, *, replace: bool = False):
    """Class decorator: `@register("mixer", "gqa_attention")`."""
    if category not in _REGISTRIES:
        raise ValueError(f"unknown part category {category!r}; have {sorted(_REGISTRIES)}")

    def deco(cls):
        reg = _REGISTRIES[category]
        if kind in reg and not replace and reg[kind] is not cls:
            raise ValueError(f"{category} {kind!r} is already registered")
        reg[kind] = cls
        return cls
    return deco


def unregister(category: str, kind: str) -> None:
    _REGISTRIES[category].pop(kind, None)


def lookup(category: str, kind: str):
    _ensure_builtin()
    try:
        return _REGISTRIES[category][kind]
    except KeyError:
        raise KeyError(f"no {category} registered as {kind!r}; have {sorted(_REGISTRIES[category])}") from None


def kinds(category: str) -> list[str]:
    _ensure_builtin()
    return sorted(_REGISTRIES[category])


def _ensure_builtin() -> None:
    from . import norm, rope, attention, feed_forward, block, embedding, head  # noqa: F401
