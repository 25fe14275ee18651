"""Registry of part classes: (category, kind) → class.

Categories: "embedding", "norm", "position", "mixer", "feed_forward", "block",
"head".  A new part is added by decorating its class with
``@register_part(category, kind)``; an architecture's builder then names that kind in
a :class:`~rustingstrata_b200.parts.spec.PartSpec`.  Tests register toy parts this way
without touching the package.
"""
from __future__ import annotations

from typing import Callable, Dict, Tuple, Type

CATEGORIES = ("embedding", "norm", "position", "mixer", "feed_forward", "block", "head")

_PARTS: Dict[Tuple[str, str], type] = {}


def register_part(category: str, kind: str, *, replace: bool = False) -> Callable[[type], type]:
    if category not in CATEGORIES:
        raise ValueError(f"unknown part category '{category}' (known: {', '.join(CATEGORIES)})")

    def deco(cls: type) -> type:
        key = (category, kind)
        if key in _PARTS and _PARTS[key] is not cls and not replace:
            raise ValueError(f"part {category}/{kind} is already registered as {_PARTS[key].__name__}")
        _PARTS[key] = cls
        cls.category = category
        cls.kind = kind
        return cls
    return deco


def part_class(category: str, kind: str) -> type:
    try:
        return _PARTS[(category, kind)]
    except KeyError:
        known = sorted(k for c, k in _PARTS if c == category)
        raise KeyError(f"no {category} part of kind '{kind}' is registered (known: {', '.join(known) or 'none'})") from None


def unregister_part(category: str, kind: str) -> None:
    _PARTS.pop((category, kind), None)


def registered_parts():
    return sorted(_PARTS)
