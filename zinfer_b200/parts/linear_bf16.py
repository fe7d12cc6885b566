"""Tensor-core contractions of the bfloat16 path.  `try_linear` returns None for a shape no
tensor-core kernel takes; the caller then uses the CUDA-core kernel.

Few rows (single-token steps): the weight-streaming mma.sync kernel, which can also apply a
pending RMSNorm itself.  More rows (prompt steps): the TMA-fed tcgen05 kernel with its
accumulator in tensor memory."""
from __future__ import annotations

from .. import kernels


# Between 17 and 64 rows the tcgen05 kernel with the weights on its 128-row side beats the mma.sync
# kernel once the weight matrix gives it enough blocks (measured at 64 rows: 18 us against 44 us
# for N = 16384, 15 us against 22 us for N = 6144, 15 us against 12 us for N = 2048).
TC_SWAPPED_MIN_ROWS = 17
TC_SWAPPED_MIN_N = 4096


def try_linear(a, w, out, out_dtype, accumulate, bias):
    from .linear import as_tensor, fused_input

    if TC_SWAPPED_MIN_ROWS <= a.shape[0] <= kernels.gemm_skinny_max_m() and w.shape[0] >= TC_SWAPPED_MIN_N:
        t = as_tensor(a)
        if kernels.gemm_tc_takes(t, w, out):
            return kernels.gemm_tc(t, w, out=out, out_dtype=out_dtype, accumulate=accumulate, bias=bias)
    x = fused_input(a, w)
    if x is not None:
        return kernels.gemm_skinny(x, w, out=out, out_dtype=out_dtype, accumulate=accumulate, bias=bias)
    a = as_tensor(a)
    if kernels.gemm_tc_takes(a, w, out):
        return kernels.gemm_tc(a, w, out=out, out_dtype=out_dtype, accumulate=accumulate, bias=bias)
    return None
