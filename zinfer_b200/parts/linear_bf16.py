"""Tensor-core contractions of the bfloat16 path.  `try_linear` returns None for a shape no
tensor-core kernel takes; the caller then uses the CUDA-core kernel.

Few rows (single-token steps): the weight-streaming mma.sync kernel, which can also apply a
pending RMSNorm itself.  More rows (prompt steps): the TMA-fed tcgen05 kernel with its
accumulator in tensor memory."""
from __future__ import annotations

from .. import kernels


def try_linear(a, w, out, out_dtype, accumulate, bias):
    from .linear import as_tensor, fused_input

    x = fused_input(a, w)
    if x is not None:
        return kernels.gemm_skinny(x, w, out=out, out_dtype=out_dtype, accumulate=accumulate, bias=bias)
    a = as_tensor(a)
    if kernels.gemm_tc_takes(a, w, out):
        return kernels.gemm_tc(a, w, out=out, out_dtype=out_dtype, accumulate=accumulate, bias=bias)
    return None
