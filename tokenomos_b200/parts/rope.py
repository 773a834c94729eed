"""Rotary position encoding, rotate-half (neox) layout.

Frequencies ``inv_i = theta ** (-2 i / dim)`` for ``i < angles``, zero for the rest of
``dim / 2`` (a zero-tail partial rotation: those dims pass through with cos 1, sin 0), computed
once on the CPU in float32; the angle of a token is ``float(position) * inv_i`` and cos / sin are
rounded to the storage type (Tokenomos models/blocks/rope.py:33-35,51-59). The kernels compute
cos and sin from ``inv_freq`` and the positions, so the part only owns the frequency table.
"""

from __future__ import annotations

import torch

from tokenomos_b200.parts.registry import Runtime, register


class Rope:
    def __init__(self, head_dim: int, angles: int, theta: float, device, dim: int | None = None):
        dim = dim or head_dim
        if dim % 2 or dim > head_dim:
            raise ValueError(f"rotary width {dim} of head size {head_dim}")
        if not 0 <= angles <= dim // 2:
            raise ValueError(f"{angles} rotary angles of width {dim}")
        idx = torch.arange(0, 2 * angles, 2, dtype=torch.float32)
        inv = 1.0 / (theta ** (idx / dim))
        inv = torch.cat((inv, torch.zeros(dim // 2 - angles, dtype=torch.float32)))
        self.inv_freq = inv.to(device).contiguous()
        self.dim = dim

    def tables(self, ctx) -> torch.Tensor:
        """What the attention kernels take: the frequency table (positions come from ``ctx``)."""
        return self.inv_freq


@register("position", "rope")
def build_rope(params: dict, tensors: dict, rt: Runtime) -> Rope:
    return Rope(params["head_dim"], params["angles"], params["theta"], rt.device,
                params.get("dim"))
