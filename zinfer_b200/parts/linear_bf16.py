"""Tensor-core contractions of the bfloat16 path.  `try_linear` returns None for a shape no
tensor-core kernel takes; the caller then uses the CUDA-core kernel.

Few rows (single-token steps): the weight-streaming mma.sync kernel, which can also apply a
pending RMSNorm itself.  More rows (prompt steps): the TMA-fed tcgen05 kernel with its
accumulator in tensor memory."""
from __future__ import annotations

from .. import kernels


# Between 9 and 64 rows the tcgen05 kernel with the weights on its 128-row side beats the mma.sync
# kernel (measured at 64 rows on the LFM2-1.2B shapes: 18 us against 44 us for N = 16384, 13 against
# 22 for N = 6144, 9 against 12 for N = 2048, 14 against 38 for N = 2048 with K = 8192; a whole step
# of 9 sequences 0.97 against 1.13 ms, of 16 sequences 1.15 against 1.31 ms); up to 8 rows the
# mma.sync kernel is as fast or faster.  K is split over a cluster when the weight matrix alone
# gives fewer 128-row tiles than there are SMs.
TC_SWAPPED_MIN_ROWS = 9


def swapped_splits(n_weight_rows: int) -> int:
    tiles = -(-n_weight_rows // 128)
    want = max(1, min(8, 192 // tiles))
    return 1 << (want.bit_length() - 1)


def try_linear(a, w, out, out_dtype, accumulate, bias, sink=None):
    from .linear import as_tensor, fused_input

    if TC_SWAPPED_MIN_ROWS <= a.shape[0] <= kernels.gemm_skinny_max_m():
        t = as_tensor(a)
        if kernels.gemm_tc_takes(t, w, out):
            return kernels.gemm_tc(t, w, out=out, out_dtype=out_dtype, accumulate=accumulate, bias=bias,
                                   splits=swapped_splits(w.shape[0]))
    x = fused_input(a, w)
    if x is not None:
        emit = None
        if sink is not None and kernels.gemm_skinny_emits(x, out):
            emit = kernels.NormEmit(sink.norm_weight)
        y = kernels.gemm_skinny(x, w, out=out, out_dtype=out_dtype, accumulate=accumulate, bias=bias, emit=emit)
        if emit is not None:
            sink.emit = emit
        return y
    a = as_tensor(a)
    if kernels.gemm_tc_takes(a, w, out):
        return kernels.gemm_tc(a, w, out=out, out_dtype=out_dtype, accumulate=accumulate, bias=bias)
    return None
