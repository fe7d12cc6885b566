"""The one place that picks a contraction kernel: out (+)= a @ w.T (+ bias).

The reference has one matmul driver for every weight matrix, with an `accumulate` flag that
folds the residual add into the store (src/model.zig:903-1026, 918-920).  Here the float32 path
always takes the CUDA-core FMA kernel (true 32-bit); the bfloat16 path takes a tensor-core
kernel when the shape allows one and the same FMA kernel otherwise.

`a` may be a `NormedRows`: rows of the residual stream whose RMSNorm is still to be applied.
A kernel that can normalise its input itself takes it as it is; for any other kernel the norm
runs first, once, however many contractions read it.

`out` may be a `ResidualSink`: the residual rows together with the norm that reads them next.
A kernel that can then writes, beside the sum, what that norm needs (the rows times the norm's
weight in bfloat16 and partial sums of their squares), and the contraction behind the norm
scales its own sums by the rows' 1/rms: the norm costs neither a launch nor a pass over the rows.
"""
from __future__ import annotations

from typing import Optional, Union

import torch

from .. import kernels


class NormedRows:
    """RMSNorm(x) * weight that is computed when somebody needs it as a tensor."""

    def __init__(self, x: torch.Tensor, weight: torch.Tensor, eps: float, dtype: torch.dtype,
                 scaled: Optional["kernels.NormEmit"] = None):
        self.x, self.weight, self.eps, self.dtype = x, weight, eps, dtype
        self.scaled = scaled          # what the kernel that summed x wrote for this norm, if it did
        self._tensor: Optional[torch.Tensor] = None

    @property
    def shape(self):
        return self.x.shape

    def tensor(self) -> torch.Tensor:
        if self._tensor is None:
            self._tensor = kernels.rmsnorm(self.x, self.weight, self.eps, self.dtype)
        return self._tensor

    def kernel_input(self) -> "kernels.NormInput":
        return kernels.NormInput(self.x, self.weight, self.eps)


class ResidualSink:
    """The float32 residual rows as the target of an accumulating contraction (`linear(...,
    out=sink, accumulate=True)`), with the weight of the RMSNorm that reads them next.  `emit`
    is set once a kernel has written that norm's inputs beside the sum; it stays None when the
    kernel that ran cannot, and the norm then works from the rows as ever."""

    def __init__(self, rows: torch.Tensor, norm_weight: torch.Tensor):
        self.rows, self.norm_weight = rows, norm_weight
        self.emit: Optional["kernels.NormEmit"] = None


FUSION_GROUP = 16     # rows per part and group in the interleaved weight layouts of the fused kernels


def interleave_rows(parts, group: int = FUSION_GROUP) -> torch.Tensor:
    """Rows of equally shaped matrices (or vectors) regrouped as `group` rows of the first, the
    same `group` rows of the second, ...: a block of a fused kernel then finds all parts of its
    outputs in adjacent rows.  The row count must be a multiple of `group`."""
    n = parts[0].shape[0]
    if n % group or any(p.shape != parts[0].shape for p in parts):
        raise ValueError(f"cannot interleave {[tuple(p.shape) for p in parts]} in groups of {group}")
    stacked = torch.stack([p.reshape(n // group, group, *p.shape[1:]) for p in parts], dim=1)
    return stacked.reshape(len(parts) * n, *parts[0].shape[1:]).contiguous()


def as_tensor(a: Union[torch.Tensor, NormedRows]) -> torch.Tensor:
    return a.tensor() if isinstance(a, NormedRows) else a


def scaled_or_tensor(a: Union[torch.Tensor, NormedRows]):
    """For a kernel that takes a `kernels.ScaledInput`: that, if the rows came prepared and nobody
    has asked for the normalised tensor yet; else the tensor."""
    if isinstance(a, NormedRows) and a.scaled is not None and a._tensor is None and a.dtype == torch.bfloat16:
        return kernels.ScaledInput(a.scaled.xw, a.scaled.ssq, a.eps)
    return as_tensor(a)


# A block that applies the norm itself reads all M rows again, so fusing the norm pays only while
# few blocks do so (about one per SM) or the rows are very few; measured on the LFM2-1.2B shapes:
# fused 12.5 us against 14.5 us for the short convolution's in_proj (128 blocks, 8 rows), but
# 75 us against 50 us for the head (2048 blocks).  A whole step with every norm fused against the
# rule below: 0.673 against 0.680 ms at 4 rows, 0.723 against 0.714 ms at 8 rows.
NORM_FUSION_MAX_BLOCKS = 160
NORM_FUSION_ANY_BLOCKS_ROWS = 4


def fused_input(a: Union[torch.Tensor, NormedRows], w: torch.Tensor, need_fused_rows: bool = False,
                blocks: Optional[int] = None):
    """What a skinny kernel should be given for `a`, or None if it does not take it: the pending
    norm itself when the kernel can apply it and that is the faster way (`blocks` = thread blocks
    the kernel will run, default one per 16 weight rows), else the (materialised) bfloat16 tensor."""
    takes = kernels.gemm_skinny_fused_takes if need_fused_rows else kernels.gemm_skinny_takes
    if isinstance(a, NormedRows):
        if a.dtype != torch.bfloat16:
            return None
        if a._tensor is None:
            if a.scaled is not None:
                si = kernels.ScaledInput(a.scaled.xw, a.scaled.ssq, a.eps)
                if takes(si, w):
                    return si
            ki = a.kernel_input()
            n_blocks = blocks if blocks is not None else -(-w.shape[0] // 16)
            worth = n_blocks <= NORM_FUSION_MAX_BLOCKS or a.shape[0] <= NORM_FUSION_ANY_BLOCKS_ROWS
            if worth and takes(ki, w):
                return ki
            max_rows = kernels.gemm_skinny_fused_max_m() if need_fused_rows else kernels.gemm_skinny_max_m()
            if a.shape[0] > max_rows:
                return None             # too many rows for these kernels: the norm stays pending for another
        a = a.tensor()
    return a if takes(a, w) else None


def linear(a: Union[torch.Tensor, NormedRows], w: torch.Tensor,
           out: Union[torch.Tensor, ResidualSink, None] = None, out_dtype=None,
           accumulate: bool = False, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """a [M, K] and w [N, K] in the run dtype; result [M, N] in `out_dtype` (default: run dtype),
    or added into `out` when `accumulate`."""
    sink = None
    if isinstance(out, ResidualSink):
        sink, out = out, out.rows
    if w.dtype == torch.bfloat16:
        from . import linear_bf16
        y = linear_bf16.try_linear(a, w, out, out_dtype, accumulate, bias, sink)
        if y is not None:
            return y
    return kernels.gemm_simt(as_tensor(a), w, out=out, out_dtype=out_dtype, accumulate=accumulate, bias=bias)
