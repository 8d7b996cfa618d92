"""Registries of part kinds.  A model description names parts by kind; ``build_part`` makes them."""
from __future__ import annotations

from .base import PartSpec

NORMS: dict = {}
POSITION_ENCODINGS: dict = {}
MIXERS: dict = {}
FEED_FORWARDS: dict = {}
ARRANGEMENTS: dict = {}

_TABLES = {"norm": NORMS, "position": POSITION_ENCODINGS, "mixer": MIXERS, "feed_forward": FEED_FORWARDS,
           "arrangement": ARRANGEMENTS}


def register_part(family: str, kind: str, cls) -> None:
    """``family``: norm, position, mixer, feed_forward or arrangement."""
    _TABLES[family][kind] = cls


def build_part(family: str, spec: PartSpec):
    table = _TABLES[family]
    try:
        cls = table[spec.kind]
    except KeyError:
        raise KeyError(f"no {family} part of kind {spec.kind!r} is registered; known: {sorted(table)}") from None
    return cls(**spec.params)
