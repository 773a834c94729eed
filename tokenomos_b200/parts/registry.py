"""Registries from a part's ``kind`` to the function that builds it.

A builder has the signature ``build(params: dict, tensors: dict[str, Tensor], rt: Runtime)``
and returns an object with the interface of its family (``parts.contract``). Registering a new
kind is all it takes to use it in a ``ModelSpec``; the framework's files do not change.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch


@dataclass(frozen=True)
class Runtime:
    """What every part is built for: the work dtype (storage of activations, matrices and
    caches) and the device."""

    dtype: torch.dtype
    device: torch.device


Builder = Callable[[dict, dict, Runtime], object]

MIXERS: dict[str, Builder] = {}
FEED_FORWARDS: dict[str, Builder] = {}
NORMS: dict[str, Builder] = {}
POSITIONS: dict[str, Builder] = {}
BLOCKS: dict[str, Callable] = {}

_FAMILIES = {
    "mixer": MIXERS,
    "feed_forward": FEED_FORWARDS,
    "norm": NORMS,
    "position": POSITIONS,
    "block": BLOCKS,
}


def register(family: str, kind: str, builder: Callable | None = None):
    """``register("mixer", "my_mixer", build_fn)`` or as a decorator without ``builder``."""
    if family not in _FAMILIES:
        raise ValueError(f"unknown part family {family!r}; families: {sorted(_FAMILIES)}")

    def put(fn):
        _FAMILIES[family][kind] = fn
        return fn

    return put if builder is None else put(builder)


def builder_of(family: str, kind: str) -> Callable:
    table = _FAMILIES[family]
    if kind not in table:
        raise ValueError(f"no {family} of kind {kind!r} is registered; known: {sorted(table)}")
    return table[kind]
