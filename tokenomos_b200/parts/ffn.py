"""Gated feed-forward: ``down(silu(gate(x)) * up(x))``, gate and up fused into one projection
(gate first) (Tokenomos models/blocks/ffn.py:25-32)."""

from __future__ import annotations

import torch

from tokenomos_b200 import ops
from tokenomos_b200.parts.linear import Linear
from tokenomos_b200.parts.registry import Runtime, register


class SwiGLU:
    def __init__(self, gate_up: Linear, down: Linear):
        if gate_up.out_features != 2 * down.in_features:
            raise ValueError("SwiGLU: gate_up must be twice as wide as down's input")
        self.gate_up, self.down = gate_up, down

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.down(ops.swiglu(self.gate_up(x)))


@register("feed_forward", "swiglu")
def build_swiglu(params: dict, tensors: dict, rt: Runtime) -> SwiGLU:
    return SwiGLU(Linear.fused([tensors["gate"], tensors["up"]]), Linear(tensors["down"]))
