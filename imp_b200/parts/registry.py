"""Part kinds by category: mixer, feed_forward, norm, position, block, embedding, head.

A plan names parts by kind; the table that resolves the names lives in the
library (csrc/host/parts.cpp).  `register_part` adds a kind written in Python
(a subclass of the classes in imp_b200/parts/base.py); that is all it takes to
make it available to every architecture plan.
"""
from __future__ import annotations

import json

from .. import capi

CATEGORIES = ("mixer", "feed_forward", "norm", "position", "block", "embedding", "head")


def register_part(category: str, kind: str, cls: type, *, replace: bool = False) -> None:
    if category not in CATEGORIES:
        raise ValueError(f"unknown part category '{category}'; categories: {', '.join(CATEGORIES)}")
    from .base import register_python_part
    if kind in known_parts(category) and not replace:
        raise ValueError(f"{category} kind '{kind}' is already registered")
    register_python_part(category, kind, cls, replace=replace)


def unregister_part(category: str, kind: str) -> None:
    capi.check(capi.load().imp_unregister_part(category.encode(), kind.encode()))


def known_parts(category: str):
    return sorted(json.loads(capi.text(capi.load().imp_known_parts(category.encode()))))
