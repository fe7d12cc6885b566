"""RMSNorm: y = x * 1/sqrt(mean(x^2) + eps) * w, sum and scale in float32
(src/model.zig:1166-1181; plain weight, no 1 + w)."""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from .base import NORMS, Norm, WeightSpec
from .linear import NormedRows


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

    def pending(self, ctx, x):
        """All rows, not yet normalised: `linear` and the fused kernels resolve a `NormedRows`."""
        return NormedRows(x, self.weight, self.eps, ctx.dtype)


NORMS.register("rmsnorm", RMSNorm)
