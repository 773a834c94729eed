"""Rotary position encoding, rotate-half (neox) layout.

Frequencies ``inv_i = theta ** (-2 i / dim)`` for ``i < angles``, zero for the rest of
``dim / 2`` (a zero-tail partial rotation: those dims pass through with cos 1, sin 0), computed
once on the CPU in float32; the angle of a token is ``float(position) * inv_i`` and cos / sin are
rounded to the storage type (Tokenomos models/blocks/rope.py:33-35,51-59). One kernel norms the
q and k heads, rotates them by angles it computes from ``inv_freq`` and the positions, and
writes the new keys and values into the cache.
"""

from __future__ import annotations

import torch

from tokenomos_b200 import ops
from tokenomos_b200.parts.contract import HeadLayout, StepContext
from tokenomos_b200.parts.registry import Runtime, register


class Rope:
    capture_safe = True

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

    def rotate_half_frequencies(self) -> torch.Tensor:
        return self.inv_freq

    def encode_qk(self, qkv: torch.Tensor, ctx: StepContext, heads: HeadLayout,
                  pool: torch.Tensor | None, table: torch.Tensor | None) -> torch.Tensor:
        if self.dim > heads.head_dim:
            raise ValueError(f"rotary width {self.dim} above the head size {heads.head_dim}")
        return ops.qk_norm_rope_write(
            qkv, pool, heads.q_norm, heads.k_norm if heads.kv_heads else None, heads.eps,
            self.inv_freq, ctx.positions, ctx.tok_seq, table, heads.heads, heads.kv_heads,
            heads.head_dim, ctx.page_size)


@register("position", "rope")
def build_rope(params: dict, tensors: dict, rt: Runtime) -> Rope:
    return Rope(params["head_dim"], params["angles"], params["theta"], rt.device,
                params.get("dim"))
