"""The matrix product y = a W^T (+ bias) behind every projection.

float32: the framework's own FMA kernel, true 32-bit.  bfloat16: operands in
bfloat16, accumulation in 32-bit; the result is bfloat16 or, where asked
(logits), float32.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from . import gemm_bf16


class Linear:
    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None):
        if weight.dim() != 2:
            raise ValueError("a projection weight is a matrix (out, in)")
        self.weight = weight
        self.bias = bias
        self.out_features, self.in_features = weight.shape

    def forward(self, a: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
                use_bias: bool = True, partials_ok: bool = False) -> torch.Tensor:
        """[M, out] in `out_dtype` (default: the operands' type).  A caller whose
        consumer adds partial sums (`partials_ok`) may get float32 [S, M, out]."""
        if a.shape[-1] != self.in_features or a.dtype != self.weight.dtype:
            raise ValueError(
                f"projection takes [{self.in_features}] rows of {self.weight.dtype}, "
                f"got {list(a.shape)} of {a.dtype}")
        bias = self.bias if use_bias else None
        out_dtype = out_dtype or a.dtype
        if a.shape[0] == 0:
            return torch.empty((0, self.out_features), dtype=out_dtype, device=a.device)
        if a.dtype == torch.float32:
            out = torch.empty((a.shape[0], self.out_features), dtype=out_dtype, device=a.device)
            ops.gemm_f32(a, self.weight, bias, out)
            return out
        return gemm_bf16.linear_bf16(a, self.weight, bias, out_dtype, partials_ok)
