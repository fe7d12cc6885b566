"""The one place that picks a contraction kernel: out (+)= a @ w.T (+ bias).

The reference has one matmul driver for every weight matrix, with an `accumulate` flag that
folds the residual add into the store (src/model.zig:903-1026, 918-920).  Here the float32 path
always takes the CUDA-core FMA kernel (true 32-bit); the bfloat16 path takes a tensor-core
kernel when the shape allows one and the same FMA kernel otherwise.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels


def linear(a: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, out_dtype=None,
           accumulate: bool = False, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """a [M, K] and w [N, K] in the run dtype; result [M, N] in `out_dtype` (default: run dtype),
    or added into `out` when `accumulate`."""
    if a.dtype == torch.bfloat16:
        from . import linear_bf16
        y = linear_bf16.try_linear(a, w, out, out_dtype, accumulate, bias)
        if y is not None:
            return y
    return kernels.gemm_simt(a, w, out=out, out_dtype=out_dtype, accumulate=accumulate, bias=bias)
