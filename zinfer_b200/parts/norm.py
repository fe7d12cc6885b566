"""RMSNorm: y = x * 1/sqrt(mean(x^2) + eps) * w, sum and scale in float32
(src/model.zig:1166-1181; plain weight, no 1 + w)."""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from .base import NORMS, Norm, WeightSpec
from .linear import NormedRows, ResidualSink


class RMSNorm(Norm):
    def __init__(self, dim: int, eps: float, weight_name: str):
        self.dim, self.eps, self.weight_name = dim, float(eps), weight_name
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self):
        return [WeightSpec(self.weight_name, (self.dim,), role="vector", init="norm")]

    def load(self, weights, dtype, device):
        self.weight = weights[self.weight_name]

    def forward(self, ctx, x, rows=None):
        return kernels.rmsnorm(x, self.weight, self.eps, ctx.dtype, rows)

    def pending(self, ctx, x, prepared=None):
        """All rows, not yet normalised: `linear` and the fused kernels resolve a `NormedRows`.
        `prepared` is what `ahead` returned for these rows, after the contraction that got it ran."""
        emit = None
        if (isinstance(prepared, ResidualSink) and prepared.emit is not None and prepared.rows is x
                and prepared.norm_weight is self.weight):
            emit = prepared.emit
        return NormedRows(x, self.weight, self.eps, ctx.dtype, scaled=emit)

    def ahead(self, ctx, x):
        """For the few rows of a single-token step in bfloat16: the contraction that sums into `x`
        can write this norm's inputs along (see `linear`)."""
        if ctx.dtype != torch.bfloat16 or x.shape[0] > kernels.GEMM_TC_SWAPPED_MAX_M:
            return None
        return ResidualSink(x, self.weight)


NORMS.register("rmsnorm", RMSNorm)
