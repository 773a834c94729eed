"""Gated short-convolution mixer: ``B, C, X = in_proj(x)``; ``y = conv(B * X)``, a causal
depthwise convolution of ``width`` taps within each sequence whose last ``width - 1`` inputs
are the request's state row; ``out_proj(C * y)`` (Tokenomos models/blocks/shortconv.py:39-59).
"""

from __future__ import annotations

import torch

from tokenomos_b200 import ops
from tokenomos_b200.parts.contract import SlotState, StepContext
from tokenomos_b200.parts.linear import Linear
from tokenomos_b200.parts.registry import Runtime, register

# tokens a conv tile walks in order; any value >= width - 1 is correct. Short tiles give the
# kernel more threads (a 2,048-token portion of 2,048 channels: 18 us at 8, 33 us at 32)
CONV_TILE = 8


class ShortConv:
    def __init__(self, in_proj: Linear, out_proj: Linear, conv: torch.Tensor,
                 conv_bias: torch.Tensor | None = None):
        """``conv`` [dim, width]: tap ``width - 1`` multiplies the current token."""
        self.in_proj, self.out_proj = in_proj, out_proj
        self.conv = conv.float().contiguous()
        self.conv_bias = conv_bias.float().contiguous() if conv_bias is not None else None
        self.dim, self.width = conv.shape
        if in_proj.out_features != 3 * self.dim or out_proj.in_features != self.dim:
            raise ValueError("short conv: projections do not match the conv's channel count")
        self.tile = max(CONV_TILE, self.width - 1)

    def state_specs(self) -> dict:
        return {"conv": SlotState((self.width - 1, self.dim))}

    def forward(self, x: torch.Tensor, ctx: StepContext, call: int) -> torch.Tensor:
        bcx = self.in_proj(x)
        seq, _, off, n = ctx.tiles(self.tile)
        y = ops.conv_gated(bcx, self.conv, self.conv_bias, ctx.states[(call, "conv")],
                           ctx.cu_seqlens, ctx.seq_ctx, ctx.seq_slot, seq, off, n)
        return self.out_proj(y)


@register("mixer", "short_conv")
def build_short_conv(params: dict, tensors: dict, rt: Runtime) -> ShortConv:
    conv = tensors["conv"]
    conv = conv.reshape(conv.shape[0], conv.shape[-1])
    if conv.shape[1] != params["width"]:
        raise ValueError(f"short conv: the weight has {conv.shape[1]} taps, the configuration "
                         f"says {params['width']}")
    return ShortConv(
        Linear(tensors["in_proj"], tensors.get("in_proj_bias")),
        Linear(tensors["out_proj"], tensors.get("out_proj_bias")),
        conv, tensors.get("conv_bias"))
