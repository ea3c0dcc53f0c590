"""Registries of parts, one per category, keyed by the ``kind`` of a ``PartSpec``."""
from __future__ import annotations

from typing import Callable, Dict

CATEGORIES = ("norm", "position_encoding", "mixer", "feed_forward", "block", "embedding", "head")
_PARTS: Dict[str, Dict[str, Callable]] = {c: {} for c in CATEGORIES}


def register_part(category: str, kind: str, factory: Callable, replace: bool = False) -> None:
    """``factory(spec, env)`` (blocks: ``factory(layer_spec, env)``) builds the part."""
    if category not in _PARTS:
        raise ValueError(f"unknown part category {category!r}; categories: {CATEGORIES}")
    if kind in _PARTS[category] and not replace:
        raise ValueError(f"{category} {kind!r} is already registered")
    _PARTS[category][kind] = factory


def build_part(category: str, spec, env):
    kind = spec.block.kind if category == "block" else spec.kind
    try:
        factory = _PARTS[category][kind]
    except KeyError:
        raise KeyError(f"no {category} named {kind!r} is registered; "
                       f"registered: {sorted(_PARTS[category])}") from None
    return factory(spec, env)


def registered(category: str):
    return sorted(_PARTS[category])
