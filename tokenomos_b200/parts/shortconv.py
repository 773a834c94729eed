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

# channels per run when the in-projection's rows hold B, C and X of the same channels in turn
# (what the decode kernel's epilogue needs side by side)
RUN = 8


class ShortConv:
    capture_safe = True

    def __init__(self, in_proj: Linear, out_proj: Linear, conv: torch.Tensor,
                 conv_bias: torch.Tensor | None = None, run: int = 0):
        """``conv`` [dim, width]: tap ``width - 1`` multiplies the current token. ``run`` 0:
        ``in_proj``'s rows are all of B, then C, then X; ``run`` 8: runs of 8 channels of B, of C
        and of X in turn, so that a decode CTA that owns 24 rows holds all three of the same 8
        channels and can run the conv in its epilogue."""
        self.in_proj, self.out_proj, self.run = in_proj, out_proj, run
        self.conv = conv.float().contiguous()
        self.conv_bias = conv_bias.float().contiguous() if conv_bias is not None else None
        self.dim, self.width = conv.shape
        lo, hi = ops.CONV_WIDTHS
        if not lo <= self.width <= hi:
            raise ValueError(f"short conv: {self.width} taps; the conv kernels take {lo} to {hi}")
        if in_proj.out_features != 3 * self.dim or out_proj.in_features != self.dim:
            raise ValueError("short conv: projections do not match the conv's channel count")
        self.norm_folded = False
        # tokens a conv tile walks in order; any value >= width - 1 is correct
        self.tile = max(in_proj.tuning.conv_tile, self.width - 1)

    def state_specs(self) -> dict:
        return {"conv": SlotState((self.width - 1, self.dim))}

    def forward(self, x: torch.Tensor, ctx: StepContext, call: int) -> torch.Tensor:
        state = ctx.states[(call, "conv")]
        if (self.run == RUN and ctx.host.decode_only and 2 <= self.width <= 8
                and ops.gemm_skinny_ok(x, self.in_proj.weight)):
            # every sequence brings one token: projection and conv in one kernel
            y = ops.gemm_skinny_conv(x, self.in_proj.weight, self.in_proj.bias, self.conv, self.conv_bias,
                                     state, ctx.seq_ctx, ctx.seq_slot)
            return self.out_proj(y)
        bcx = self.in_proj(x)
        seq, tok0, off, n = ctx.tiles(self.tile)
        # (a step of single tokens has one-token tiles: the tiled kernel's blocks of 16 tokens
        # would be all but empty, the walking form takes them)
        cap = 0 if ctx.host.decode_only else self.tile
        y = ops.conv_gated(bcx, self.conv, self.conv_bias, state,
                           ctx.cu_seqlens, ctx.seq_ctx, ctx.seq_slot, seq, off, n, self.run, cap, tok0)
        return self.out_proj(y)


    # ---- the block's norm and residual add taken into the two products (parts.contract) ----

    def fold_norm(self, weight: torch.Tensor) -> bool:
        if self.in_proj.weight.dtype != torch.bfloat16 or not self.in_proj.tuning.fuse_norms:
            return False
        self.in_proj.fold_columns(weight)
        self.norm_folded = True
        return True

    def can_stream(self, rows: int, ctx: StepContext) -> bool:
        return (self.norm_folded and self.run == RUN and ctx.host.decode_only
                and rows <= ops.SKINNY_FUSED_ROWS and self.in_proj.in_features % 8 == 0
                and self.dim % 8 == 0)

    def forward_stream(self, stream: torch.Tensor, eps: float, ctx: StepContext, call: int) -> torch.Tensor:
        self.in_proj.note("skinny+norm")
        self.out_proj.note("skinny+add")
        state = ctx.states[(call, "conv")]
        y = ops.gemm_skinny_conv(stream, self.in_proj.weight, self.in_proj.bias, self.conv, self.conv_bias,
                                 state, ctx.seq_ctx, ctx.seq_slot, norm_eps=eps)
        return ops.gemm_skinny(y, self.out_proj.weight, self.out_proj.bias, residual=stream)


def interleave_bcx(w: torch.Tensor, run: int) -> torch.Tensor:
    """Rows (or entries) [B | C | X] of 3 d -> runs of ``run`` channels of B, of C and of X in turn."""
    d = w.shape[0] // 3
    parts = w.view(3, d // run, run, *w.shape[1:])
    return parts.transpose(0, 1).reshape(w.shape).contiguous()


@register("mixer", "short_conv")
def build_short_conv(params: dict, tensors: dict, rt: Runtime) -> ShortConv:
    conv = tensors["conv"]
    conv = conv.reshape(conv.shape[0], conv.shape[-1])
    if conv.shape[1] != params["width"]:
        raise ValueError(f"short conv: the weight has {conv.shape[1]} taps, the configuration "
                         f"says {params['width']}")
    w_in, b_in = tensors["in_proj"], tensors.get("in_proj_bias")
    run = 0
    if w_in.dtype == torch.bfloat16 and conv.shape[0] % RUN == 0:
        run = RUN
        w_in = interleave_bcx(w_in, RUN)
        b_in = interleave_bcx(b_in, RUN) if b_in is not None else None
    return ShortConv(
        Linear(w_in, b_in, rt.tuning),
        Linear(tensors["out_proj"], tensors.get("out_proj_bias"), rt.tuning),
        conv, tensors.get("conv_bias"), run)
