"""SwiGLU feed-forward: h = silu(xn W1^T) * (xn W3^T), out (+)= h W2^T
(src/model.zig:2411-2422, 1085-1117; silu(g) = g / (1 + exp(-g)), src/ffn.zig:31-33).
W1 and W3 are stacked at load into one [2F, D] matrix so that gate and up are one contraction,
as the reference computes both in one worker."""
from __future__ import annotations

import torch

from .. import kernels
from .base import FEED_FORWARDS, FeedForward, WeightSpec
from .linear import fused_input, linear


FUSED_SWIGLU_MAX_ROWS = 2


class SwiGLU(FeedForward):
    def __init__(self, hidden: int, ffn_dim: int, gate_name: str, up_name: str, down_name: str):
        self.hidden, self.ffn_dim = hidden, ffn_dim
        self.gate_name, self.up_name, self.down_name = gate_name, up_name, down_name
        self.w_gate_up = self.w_down = None

    def weight_specs(self):
        return [WeightSpec(self.gate_name, (self.ffn_dim, self.hidden)),
                WeightSpec(self.up_name, (self.ffn_dim, self.hidden)),
                WeightSpec(self.down_name, (self.hidden, self.ffn_dim))]

    def load(self, weights, dtype, device):
        self.w_gate_up = torch.cat([weights[self.gate_name], weights[self.up_name]], dim=0).contiguous()
        self.w_down = weights[self.down_name]

    takes_pending_norm = True

    def forward(self, ctx, xn, out, accumulate):
        # One kernel for gate, up and the activation pays only for one or two rows: its two row
        # groups lie F rows apart in memory and stream slower than 32 adjacent rows (measured at 8
        # rows: 19.1 us fused against 13.7 + 3 us for the plain contraction and the activation).
        x = fused_input(xn, self.w_gate_up, need_fused_rows=True, blocks=-(-self.ffn_dim // 16)) \
            if xn.shape[0] <= FUSED_SWIGLU_MAX_ROWS else None
        if x is not None:
            h = kernels.gemm_skinny_swiglu(x, self.w_gate_up)
        else:
            h = kernels.silu_mul(linear(xn, self.w_gate_up))
        linear(h, self.w_down, out=out, accumulate=accumulate)


FEED_FORWARDS.register("swiglu", SwiGLU)
