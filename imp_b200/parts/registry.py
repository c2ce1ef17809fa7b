"""Part kinds by category: mixer, feed_forward, norm, position, block, embedding, head.

A plan names parts by kind; this table resolves the names.  Registering a new
kind (from a test, a user's module, or a new file under imp_b200/parts/) is
all it takes to make it available to every architecture plan.
"""
from __future__ import annotations

from typing import Dict, Type

CATEGORIES = ("mixer", "feed_forward", "norm", "position", "block", "embedding", "head")

_PARTS: Dict[str, Dict[str, type]] = {c: {} for c in CATEGORIES}


def register_part(category: str, kind: str, cls: type, *, replace: bool = False) -> None:
    if category not in _PARTS:
        raise ValueError(f"unknown part category '{category}'; categories: {', '.join(CATEGORIES)}")
    if kind in _PARTS[category] and not replace:
        raise ValueError(f"{category} kind '{kind}' is already registered")
    _PARTS[category][kind] = cls


def unregister_part(category: str, kind: str) -> None:
    _PARTS[category].pop(kind, None)


def part_class(category: str, kind: str) -> type:
    _ensure_builtin()
    try:
        return _PARTS[category][kind]
    except KeyError:
        known = ", ".join(sorted(_PARTS.get(category, {}))) or "(none)"
        raise ValueError(f"unknown {category} kind '{kind}'; known: {known}") from None


def known_parts(category: str):
    _ensure_builtin()
    return sorted(_PARTS[category])


def _ensure_builtin() -> None:
    from . import builtin  # noqa: F401  (registers the built-in kinds on import)
