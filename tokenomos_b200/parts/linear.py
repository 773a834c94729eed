"""Dense projection ``y = x @ W.T (+ b)`` with the weight kept as loaded: ``[out, in]``.

Routes, by storage type:

- float32: the CUDA-core kernel with 32-bit FMA accumulation (``ops.gemm``). No tensor-core or
  reduced-precision mode can reach it, whatever the process-wide torch flags say.
- bfloat16: by shape (``route``): the hand-written weight-streaming kernel for a few rows
  (``ops.gemm_skinny``), the TMA + tcgen05 kernel for very tall matrices (``ops.gemm_tc``), else
  the library GEMM (cuBLAS through ``torch.nn.functional.linear``), as the reference engine does
  for every 16-bit projection (Tokenomos models/blocks/linear.py:236-254).
- a matrix stored in 32-bit in a 16-bit model stays 32-bit: the activation is widened for it.

Several matrices that read the same input are fused along the output axis at build time
(q/k/v, gate/up: Tokenomos models/blocks/linear.py:123-165).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from tokenomos_b200 import ops


class Linear:
    def __init__(self, weight: torch.Tensor, bias: torch.Tensor | None = None):
        """``weight`` [out, in] in the work dtype (or float32); ``bias`` float32 [out] or None."""
        self.weight = weight.contiguous()
        self.bias = bias
        self.out_features, self.in_features = weight.shape
        self._bias_lp = None
        if bias is not None and weight.dtype == torch.bfloat16:
            self._bias_lp = bias.to(torch.bfloat16)

    @classmethod
    def fused(cls, weights: list[torch.Tensor], biases: list[torch.Tensor | None] | None = None):
        """One projection from several that read the same input, outputs side by side."""
        biases = biases or [None] * len(weights)
        if any(b is not None for b in biases) and not all(b is not None for b in biases):
            raise ValueError("fused projection: either every part has a bias or none")
        bias = torch.cat(biases) if biases[0] is not None else None
        return cls(torch.cat(weights, dim=0), bias)

    def __call__(self, x: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
        w = self.weight
        if x.dtype != w.dtype:
            # a 32-bit matrix in a 16-bit model: widen the input, round the result once
            y = ops.gemm(x.float().contiguous(), w, self.bias, torch.float32)
            return y if out_dtype == torch.float32 else y.to(x.dtype)
        if w.dtype == torch.float32:
            return ops.gemm(x, w, self.bias, torch.float32)
        if not x.is_cuda:
            raise ops.KernelError("Linear: CUDA tensors only (there is no CPU path)")
        route = self.route(x)
        if route == "tc":
            return ops.gemm_tc(x, w, self.bias, out_dtype)
        if route == "skinny":
            return ops.gemm_skinny(x, w, self.bias, out_dtype)
        if out_dtype == torch.float32:
            return self._float_out(x)
        if self.in_features % 8 or (x.stride(0) % 8 and x.shape[0] > 1):
            return ops.gemm(x, w, self.bias, out_dtype or x.dtype)
        return F.linear(x, w, self._bias_lp)

    def route(self, x: torch.Tensor) -> str:
        """Which kernel takes ``x`` [M, in]: measured on a B200 with 2048- to 8192-wide matrices
        in CUDA graphs, the register-streaming kernel is the fastest up to 8 rows (and up to 16
        for matrices of a few thousand rows), the TMA + tcgen05 kernel for very tall matrices
        (the head) from 5 to 64 rows, the library elsewhere."""
        m, n = x.shape[0], self.out_features
        if m > 64:
            return "library"             # no slicing, no checks: prompt portions come here
        if not ops.gemm_skinny_ok(x[:1], self.weight):
            return "library"
        if m <= 4:
            return "skinny"              # the head too: 0.67 ms a decode step at one row against 0.70
        if n >= 32768 and m <= 64:
            return "tc"
        if m <= 8 or (m <= 16 and n <= 4096):
            return "skinny"
        return "library"

    def _float_out(self, x: torch.Tensor) -> torch.Tensor:
        """16-bit operands, 32-bit result (the head: logits are not rounded to 16-bit)."""
        if self.in_features % 8 == 0 and self.bias is None and x.is_contiguous():
            return torch.mm(x, self.weight.t(), out_dtype=torch.float32)
        return ops.gemm(x, self.weight, self.bias, torch.float32)
