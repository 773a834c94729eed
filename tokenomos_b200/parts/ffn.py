"""Gated feed-forward: ``down(silu(gate(x)) * up(x))``, gate and up fused into one projection
(gate first) (Tokenomos models/blocks/ffn.py:25-32)."""

from __future__ import annotations

import torch

from tokenomos_b200 import ops
from tokenomos_b200.parts.linear import Linear
from tokenomos_b200.parts.registry import Runtime, register


# channels per run when gate and up rows alternate (what the decode kernel's epilogue pairs up)
RUN = 8


class SwiGLU:
    capture_safe = True

    def __init__(self, gate_up: Linear, down: Linear, run: int = 0):
        """``run`` 0: ``gate_up``'s rows are all gate rows, then all up rows. ``run`` 8: they
        alternate in runs of 8 channels, so that a decode CTA that owns 16 rows holds gate and up
        of the same 8 channels and can apply the activation in its epilogue."""
        if gate_up.out_features != 2 * down.in_features:
            raise ValueError("SwiGLU: gate_up must be twice as wide as down's input")
        self.gate_up, self.down, self.run = gate_up, down, run
        self.norm_folded = False

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        w = self.gate_up.weight
        # (up to 8 rows: with 9 to 16 the library's product and the activation kernel are faster,
        # 0.91 ms a decode step at 16 rows against 1.00 ms)
        if (self.run == RUN and x.shape[0] <= self.gate_up.tuning.swiglu_fused_rows
                and ops.gemm_skinny_ok(x, w)):
            act = ops.gemm_skinny(x, w, self.gate_up.bias, swiglu=True)
        else:
            act = ops.swiglu(self.gate_up(x), self.run)
        return self.down(act)


    # ---- the block's norm and residual add taken into the two products (parts.contract) ----

    def fold_norm(self, weight: torch.Tensor) -> bool:
        if self.gate_up.weight.dtype != torch.bfloat16 or not self.gate_up.tuning.fuse_norms:
            return False
        self.gate_up.fold_columns(weight)
        self.norm_folded = True
        return True

    def can_stream(self, rows: int) -> bool:
        t = self.gate_up.tuning
        return (self.norm_folded and self.run == RUN and rows <= min(ops.SKINNY_FUSED_ROWS, t.swiglu_fused_rows)
                and self.gate_up.in_features % 8 == 0 and self.down.in_features % 8 == 0)

    def forward_stream(self, stream: torch.Tensor, eps: float) -> torch.Tensor:
        self.gate_up.note("skinny+norm")
        self.down.note("skinny+add")
        act = ops.gemm_skinny(stream, self.gate_up.weight, self.gate_up.bias, swiglu=True, norm_eps=eps)
        return ops.gemm_skinny(act, self.down.weight, self.down.bias, residual=stream)


def interleave_rows(gate: torch.Tensor, up: torch.Tensor, run: int) -> torch.Tensor:
    """[I, K] gate and up -> [2 I, K] with ``run`` gate rows, the ``run`` up rows of the same
    channels, and so on."""
    inter, k = gate.shape
    both = torch.stack((gate.view(inter // run, run, k), up.view(inter // run, run, k)), dim=1)
    return both.reshape(2 * inter, k).contiguous()


@register("feed_forward", "swiglu")
def build_swiglu(params: dict, tensors: dict, rt: Runtime) -> SwiGLU:
    gate, up = tensors["gate"], tensors["up"]
    down = Linear(tensors["down"], tuning=rt.tuning)
    if gate.dtype == torch.bfloat16 and gate.shape[0] % RUN == 0:
        return SwiGLU(Linear(interleave_rows(gate, up, RUN), tuning=rt.tuning), down, RUN)
    return SwiGLU(Linear.fused([gate, up], tuning=rt.tuning), down)
