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
from tokenomos_b200.parts.registry import DEFAULT_TUNING, Tuning


class Linear:
    def __init__(self, weight: torch.Tensor, bias: torch.Tensor | None = None,
                 tuning: Tuning = DEFAULT_TUNING):
        """``weight`` [out, in] in the work dtype (or float32); ``bias`` float32 [out] or None;
        ``tuning``: the thresholds ``route`` picks kernels by."""
        self.weight = weight.contiguous()
        self.bias = bias.float().contiguous() if bias is not None else None
        self.out_features, self.in_features = weight.shape
        self.tuning = tuning
        # which route took how many products (tests read it to see that every branch ran)
        self.routed: dict[str, int] = {}

    @classmethod
    def fused(cls, weights: list[torch.Tensor], biases: list[torch.Tensor | None] | None = None,
              tuning: Tuning = DEFAULT_TUNING):
        """One projection from several that read the same input, outputs side by side."""
        biases = biases or [None] * len(weights)
        if any(b is not None for b in biases) and not all(b is not None for b in biases):
            raise ValueError("fused projection: either every part has a bias or none")
        bias = torch.cat(biases) if biases[0] is not None else None
        return cls(torch.cat(weights, dim=0), bias, tuning)

    def note(self, route: str) -> None:
        """Count a product a part ran through a kernel of its own choice instead of ``route``."""
        self.routed[route] = self.routed.get(route, 0) + 1

    def fold_columns(self, scale: torch.Tensor) -> None:
        """``weight[n, k] *= scale[k]`` (the product formed in 32-bit, rounded once): a norm's
        weight taken into the projection that follows the norm."""
        w = self.weight
        self.weight = (w.float() * scale.float().to(w.device)[None, :]).to(w.dtype).contiguous()

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
        self.routed[route] = self.routed.get(route, 0) + 1
        if route == "tc":
            return ops.gemm_tc(x, w, self.bias, out_dtype)
        if route == "skinny":
            return ops.gemm_skinny(x, w, self.bias, out_dtype)
        if route == "simt":
            return ops.gemm(x, w, self.bias, out_dtype or x.dtype)
        # the library's product has no 32-bit bias: the bias is added to the 32-bit result and
        # the sum rounded once, as every other route does
        if out_dtype == torch.float32 or self.bias is not None:
            y = torch.mm(x, w.t(), out_dtype=torch.float32)
            if self.bias is not None:
                y += self.bias
            return y if out_dtype == torch.float32 else y.to(x.dtype)
        return F.linear(x, w)

    def route(self, x: torch.Tensor) -> str:
        """Which kernel takes ``x`` [M, in] (thresholds: ``Tuning``): the register-streaming
        kernel for a few rows, the TMA + tcgen05 kernel for very tall matrices (the head) and for
        deep ones (a down projection) at small batches, the library elsewhere; the CUDA-core
        kernel for shapes the others refuse."""
        t, m, n, k = self.tuning, x.shape[0], self.out_features, self.in_features
        if k % 8 or x.stride(1) != 1 or (x.stride(0) % 8 and m > 1) or x.data_ptr() % 16:
            return "simt"                # no 16-byte rows: neither the library nor TMA takes it
        if m > max(t.tc_tall_rows, t.tc_deep_rows, t.skinny_small_rows):
            return "library"             # no further checks: prompt portions come here
        skinny_ok = ops.gemm_skinny_ok(x[:1], self.weight)
        if skinny_ok and m <= t.skinny_tall_rows:
            return "skinny"              # the head too (0.67 ms a decode step at one row against
                                         # 0.70, 0.729 at 8 rows against 0.740 with the tcgen05 kernel)
        if n >= t.tc_tall_n and m <= t.tc_tall_rows and ops.gemm_tc_ok(x, self.weight):
            return "tc"
        if skinny_ok and (m <= t.skinny_rows or (m <= t.skinny_small_rows and n <= t.skinny_small_n
                                                 and k < t.tc_deep_k)):
            return "skinny"
        if k >= t.tc_deep_k and t.skinny_rows < m <= t.tc_deep_rows and ops.gemm_tc_ok(x, self.weight):
            return "tc"
        return "library"
