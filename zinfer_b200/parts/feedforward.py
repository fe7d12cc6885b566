"""SwiGLU feed-forward: h = silu(xn W1^T) * (xn W3^T), out (+)= h W2^T
(src/model.zig:2411-2422, 1085-1117; silu(g) = g / (1 + exp(-g)), src/ffn.zig:31-33).
W1 and W3 are stacked at load into one [2F, D] matrix so that gate and up are one contraction,
as the reference computes both in one worker; where a kernel can, the activation is its epilogue."""
from __future__ import annotations

import torch

from .. import kernels
from .base import FEED_FORWARDS, FeedForward, WeightSpec
from .linear import FUSION_GROUP, as_tensor, fused_input, interleave_rows, linear, scaled_or_tensor
from .linear_bf16 import TC_SWAPPED_MIN_ROWS, swapped_splits


class SwiGLU(FeedForward):
    takes_pending_norm = True
    sums_through_linear = True

    def __init__(self, hidden: int, ffn_dim: int, gate_name: str, up_name: str, down_name: str):
        self.hidden, self.ffn_dim = hidden, ffn_dim
        self.gate_name, self.up_name, self.down_name = gate_name, up_name, down_name
        self.w_gate_up = self.w_down = None
        # With F a multiple of 16 the stacked matrix is stored as groups of 16 gate rows followed by
        # their 16 up rows, which lets a contraction kernel apply the activation in its epilogue.
        self.interleave = FUSION_GROUP if ffn_dim % FUSION_GROUP == 0 else 0

    def weight_specs(self):
        return [WeightSpec(self.gate_name, (self.ffn_dim, self.hidden)),
                WeightSpec(self.up_name, (self.ffn_dim, self.hidden)),
                WeightSpec(self.down_name, (self.hidden, self.ffn_dim))]

    def load(self, weights, dtype, device):
        g, u = weights[self.gate_name], weights[self.up_name]
        self.w_gate_up = interleave_rows([g, u]) if self.interleave else torch.cat([g, u], dim=0).contiguous()
        self.w_down = weights[self.down_name]

    def forward(self, ctx, xn, out, accumulate):
        w, h = self.w_gate_up, None
        if self.interleave and w.dtype == torch.bfloat16:
            from . import linear_bf16
            rows_in = xn.shape[0]
            tc_rows = linear_bf16.TC_SWAPPED_MIN_ROWS <= rows_in <= kernels.gemm_skinny_max_m()
            x = None if tc_rows else fused_input(xn, w, need_fused_rows=True, blocks=self.ffn_dim // 16)
            if x is not None:                       # few rows: gate, up and the activation in one kernel
                h = kernels.gemm_skinny_swiglu(x, w)
            else:
                x = scaled_or_tensor(xn) if tc_rows else as_tensor(xn)
                if not kernels.gemm_tc_takes(x, w):
                    x = as_tensor(xn)
                rows = x.shape[0]
                # prompt steps, and steps of 17..64 rows: activation in the epilogue
                if (rows > kernels.gemm_skinny_max_m() or tc_rows) and kernels.gemm_tc_takes(x, w):
                    splits = swapped_splits(w.shape[0], kernels.sm_count(w.device)) if tc_rows else 1
                    h = kernels.gemm_tc(x, w, swiglu=True, splits=splits)
        if h is None:
            h = kernels.silu_mul(linear(xn, w), self.interleave)
        linear(h, self.w_down, out=out, accumulate=accumulate)


FEED_FORWARDS.register("swiglu", SwiGLU)
