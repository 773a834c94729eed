"""Registries from a part's ``kind`` to the function that builds it.

A builder has the signature ``build(params: dict, tensors: dict[str, Tensor], rt: Runtime)``
and returns an object with the interface of its family (``parts.contract``). Registering a new
kind is all it takes to use it in a ``ModelSpec``; the framework's files do not change.
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Callable

import torch


@dataclass(frozen=True)
class Tuning:
    """Thresholds that pick between kernels that compute the same thing. They change speed,
    never results beyond rounding, and they belong to a device and a range of sizes, not to a
    part: the defaults were measured on a B200 (148 SMs) with 1,024- to 8,192-wide layers, in
    CUDA graphs, weights cycled beyond L2. ``for_device`` reads the SM count of another GPU.

    Dense products of 16-bit matrices, by rows of the input (``Linear.route``):
    ``skinny_rows``: up to here the register-streaming kernel, for any matrix;
    ``skinny_small_rows`` / ``skinny_small_n``: up to that many rows for matrices of at most that
    many output rows; ``skinny_tall_rows``: up to that many rows it also takes the tallest
    matrices (a vocabulary head); ``tc_tall_n`` / ``tc_tall_rows``: above, matrices at least
    ``tc_tall_n`` tall go to the TMA + tcgen05 kernel up to ``tc_tall_rows`` rows; ``tc_deep_k`` / ``tc_deep_rows``: matrices with an inner size of at
    least ``tc_deep_k`` (a feed-forward's down projection) go there above the skinny range up to
    ``tc_deep_rows`` rows; everything else is the library's.
    ``swiglu_fused_rows``: up to here gate/up and the activation are one kernel.
    Decode attention (``Attention.decode_splits``): about ``decode_keys`` keys of the longest
    allowed sequence per CTA; more CTAs than that gives while fewer than ``decode_fill`` would be
    on the GPU (never below ``decode_min_keys`` keys each); never more than
    ``decode_ctas_per_sm`` CTAs per SM (three fit by shared memory, and a few waves of them even
    out the last, partial one).
    ``decode_fused_rows``: up to that many decoded tokens a layer's norm + rotation + cache write,
    split attention, merge and gate are one kernel (``ops.attention_decode_fused``); beyond, the
    separate kernels overlap better (measured: -2.7 % of the step at 1 row, -5 % at 8, +1 % at 16,
    +5 % at 64). ``decode_fused_ctas_per_sm``: how many of its CTAs an SM holds (``Attention.fused_splits``).
    ``decode_fused_carveout``: the share of shared memory that
    kernel asks for (percent) while the products around it are the weight-streaming kernels (up to
    ``skinny_rows`` rows): an SM changes its split between shared memory and L1 only when empty,
    so a kernel that asks for another split than its neighbours cannot start under them, and the
    L1 it leaves is what their activation loads find; -1 leaves the choice to the driver, which
    it always is above ``skinny_rows`` rows.
    ``prefill_split_ctas_per_sm`` / ``prefill_split_scratch_mb``: how far a prompt portion's
    tiles may share their keys out over CTAs (``Attention.prefill_splits``).
    ``conv_tile``: tokens of a conv tile; up to 16 the tiled kernel takes them (one thread per
    token and 8 channels, a 2,048-token portion of 2,048 channels at memory speed).
    ``fuse_norms``: 16-bit models fold each pre-norm's weight into the columns of the projection
    that follows it when they are built, and steps of at most ``ops.SKINNY_FUSED_ROWS`` decoded
    tokens then run without norm kernels (``parts.block.PreNormBlock``); the environment variable
    ``TOKENOMOS_B200_FUSE_NORMS=0`` turns it off for a whole process."""

    sm_count: int = 148
    skinny_rows: int = 8
    skinny_small_rows: int = 16
    skinny_small_n: int = 4096
    skinny_tall_rows: int = 8
    tc_tall_n: int = 32768
    tc_tall_rows: int = 64
    tc_deep_k: int = 8192
    tc_deep_rows: int = 64
    swiglu_fused_rows: int = 8
    decode_keys: int = 1024
    decode_fill: int = 256
    decode_min_keys: int = 128
    decode_ctas_per_sm: int = 12
    decode_fused_rows: int = 8
    decode_fused_ctas_per_sm: int = 2
    decode_fused_carveout: int = 62
    prefill_split_ctas_per_sm: int = 2
    prefill_split_scratch_mb: int = 64
    conv_tile: int = 16
    fuse_norms: bool = True

    @classmethod
    def for_device(cls, device) -> "Tuning":
        device = torch.device(device)
        fuse = os.environ.get("TOKENOMOS_B200_FUSE_NORMS", "1") != "0"
        if device.type == "cuda" and torch.cuda.is_available():
            return cls(sm_count=torch.cuda.get_device_properties(device).multi_processor_count,
                       fuse_norms=fuse)
        return cls(fuse_norms=fuse)


DEFAULT_TUNING = Tuning()


@dataclass(frozen=True)
class Runtime:
    """What every part is built for: the work dtype (storage of activations, matrices and
    caches), the device, and the device's kernel-choice thresholds."""

    dtype: torch.dtype
    device: torch.device
    tuning: Tuning = DEFAULT_TUNING


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
