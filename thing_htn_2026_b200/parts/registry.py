"""Registries of parts.  A part class is looked up by (family, kind); ``kind`` is the
``PartSpec.kind`` a configuration wrote into its plan.  Registering a new class is all it
takes to make a new mixer, feed-forward, norm, position encoding or block arrangement
available to every configuration."""

from __future__ import annotations

from typing import Callable, Dict, Tuple

FAMILIES = ("embedding", "mixer", "ffn", "norm", "position", "block", "head")

_PARTS: Dict[Tuple[str, str], type] = {}


def register_part(family: str, kind: str) -> Callable[[type], type]:
    if family not in FAMILIES:
        raise ValueError(f"unknown part family '{family}'; families: {', '.join(FAMILIES)}")

    def decorate(cls: type) -> type:
        if (family, kind) in _PARTS and _PARTS[(family, kind)] is not cls:
            raise ValueError(f"{family} '{kind}' is already registered")
        _PARTS[(family, kind)] = cls
        return cls

    return decorate


def part_class(family: str, kind: str) -> type:
    try:
        return _PARTS[(family, kind)]
    except KeyError:
        known = sorted(k for f, k in _PARTS if f == family)
        raise KeyError(f"no {family} named '{kind}' is registered; known: {', '.join(known)}") from None


def unregister_part(family: str, kind: str) -> None:
    _PARTS.pop((family, kind), None)
