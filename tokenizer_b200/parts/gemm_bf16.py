"""bfloat16 matrix products, 32-bit accumulation: chooses the kernel by the
number of rows.  Few rows (decoding) are bound by reading the weights once and
go to the framework's streaming kernel; many rows go to the tensor cores."""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops


def linear_bf16(a: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
                out: torch.Tensor) -> None:
    """out[M,N] = a[M,K] weight[N,K]^T (+ bias float32); out is bfloat16 or float32."""
    if out.dtype == torch.bfloat16:
        torch.mm(a, weight.t(), out=out)
    else:
        out.copy_(torch.mm(a, weight.t(), out_dtype=torch.float32))
    if bias is not None:
        out.add_(bias.to(out.dtype) if out.dtype != torch.float32 else bias)
