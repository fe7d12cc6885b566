"""Tensor-core contractions of the bfloat16 path.  `try_linear` returns None for a shape no
tensor-core kernel takes; the caller then uses the CUDA-core kernel."""
from __future__ import annotations

from .. import kernels


def try_linear(a, w, out, out_dtype, accumulate, bias):
    if kernels.gemm_skinny_takes(a, w):
        return kernels.gemm_skinny(a, w, out=out, out_dtype=out_dtype, accumulate=accumulate, bias=bias)
    return None
