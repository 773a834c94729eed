"""RMSNorm, with the residual add in the same kernel.

``rstd = 1 / sqrt(mean(x^2) + eps)`` over the full width, eps inside the root; 16-bit storage
rounds the normed value before the weight and the product after it; the residual sum is formed
in 32-bit and rounded once (Tokenomos models/blocks/norm.py:41-45; kernels/norm/fused.py:22-28,
69-82). The weight is kept in float32 (a 16-bit weight widens exactly).
"""

from __future__ import annotations

import torch

from tokenomos_b200 import ops
from tokenomos_b200.parts.registry import Runtime, register


class RMSNorm:
    capture_safe = True

    def __init__(self, weight: torch.Tensor, eps: float):
        self.weight = weight.float().contiguous()
        self.eps = float(eps)
        self.width = weight.numel()
        if self.width > ops.NORM_MAX_WIDTH:
            raise ValueError(f"RMSNorm: a width of {self.width} is above the {ops.NORM_MAX_WIDTH} the "
                             "norm kernel keeps in shared memory")

    def add_norm(self, x: torch.Tensor, residual: torch.Tensor | None, pre: "RMSNorm | None" = None):
        """``stream = residual + [pre](x)``; returns ``(norm(stream), stream)``."""
        return ops.add_rmsnorm(x, residual, self.weight, self.eps,
                               (pre.weight, pre.eps) if pre is not None else None)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return self.add_norm(x, None)[0]

    def folded(self) -> tuple[torch.Tensor, float, "RMSNorm"]:
        """For a block that takes this norm's weight into the projection after it: the weight,
        eps, and the norm that is left (the same statistics, weight one)."""
        return self.weight, self.eps, RMSNorm(torch.ones_like(self.weight), self.eps)


@register("norm", "rmsnorm")
def build_rmsnorm(params: dict, tensors: dict, rt: Runtime) -> RMSNorm:
    return RMSNorm(tensors["weight"], params["eps"])
