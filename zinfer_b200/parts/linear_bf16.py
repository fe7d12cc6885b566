"""Tensor-core contractions of the bfloat16 path.  `try_linear` returns None for a shape no
tensor-core kernel takes; the caller then uses the CUDA-core kernel.

Few rows (single-token steps): the weight-streaming mma.sync kernel, which can also apply a
pending RMSNorm itself.  More rows (prompt steps): the TMA-fed tcgen05 kernel with its
accumulator in tensor memory."""
from __future__ import annotations

from .. import kernels


# From 17 to 64 rows the tcgen05 kernel with the weights on its 128-row side beats the mma.sync
# kernel (measured at 64 rows on the LFM2-1.2B shapes: 17 us against 44 us for N = 16384, 10 against
# 22 for N = 6144, 7 against 12 for N = 2048, 12 against 38 for N = 2048 with K = 8192).  Up to 16
# rows the mma.sync kernel is as fast or faster (16 rows: 3.1 against 5.0 us for out_proj, 9.0
# against 10.3 for w2, 5.9 against 6.1 for qkv, 9.3 against 8.6 for in_proj, 16.4 against 15.7 for
# w1|w3), fuses the short convolution and needs no cluster: whole steps of 9 / 12 / 16 sequences
# 0.83 / 0.84 / 0.88 ms against 0.90 / 0.91 / 0.97.
TC_SWAPPED_MIN_ROWS = 17


def swapped_splits(n_weight_rows: int, sm_count: int) -> int:
    """In how many parts K is cut (one per block of a cluster): the fewest that give every SM a block.
    Measured at 64 rows, microseconds for 1 / 2 / 4 / 8 parts: N = 2048 (16 tiles of 128 weight rows)
    13 / 9 / 7 / 7, with K = 8192 41 / 23 / 15 / 12; N = 3072 14 / 9 / 7.5 / 8; N = 6144 15 / 11 / 10 / 15;
    N = 16384 18 / 17 / 21 / 34."""
    tiles = -(-n_weight_rows // 128)
    s = 1
    while s < 8 and tiles * s < sm_count:
        s *= 2
    return s


def try_linear(a, w, out, out_dtype, accumulate, bias, sink=None):
    from .linear import as_tensor, fused_input, scaled_or_tensor

    if TC_SWAPPED_MIN_ROWS <= a.shape[0] <= kernels.gemm_skinny_max_m():
        t = scaled_or_tensor(a)
        if not kernels.gemm_tc_takes(t, w, out):
            t = as_tensor(a)
        if kernels.gemm_tc_takes(t, w, out):
            emit = None
            if sink is not None and kernels.gemm_tc_emits(t, out):
                emit = kernels.NormEmit(sink.norm_weight)
            y = kernels.gemm_tc(t, w, out=out, out_dtype=out_dtype, accumulate=accumulate, bias=bias,
                                splits=swapped_splits(w.shape[0], kernels.sm_count(w.device)), emit=emit)
            if emit is not None:
                sink.emit = emit
            return y
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
