"""Gated short-convolution mixer (src/model.zig:1994-2028).

[B, C, X] = xn W_in^T in that order along the 3D outputs; u = B * X; a causal depthwise
convolution of K taps over u, whose inputs before the step come from the sequence's state (the
last K-1 values of u, zero at a sequence's start); y = C * conv; out (+)= y W_out^T; the state
becomes the last K-1 values of u.  The taps are stored [K, D] (tap, channel), transposed from
the file's [D, 1, K] at load as the reference does (src/model.zig:788-802).

The reference has no bias tensors for this mixer (src/model.zig:729-734).  With `conv_bias` a
bias [D] is added to the convolution before the C gate, and biases of the two projections are
used when the file carries them.
"""
from __future__ import annotations

import torch

from .. import kernels
from .base import MIXERS, Mixer, StateRequest, WeightSpec
from .linear import FUSION_GROUP, fused_input, interleave_rows, linear


class ShortConv(Mixer):
    capture_safe = True        # kernels on the current stream only; launches depend on the batch size alone

    def __init__(self, hidden: int, kernel_size: int, in_name: str, conv_name: str, out_name: str,
                 conv_bias_name: str | None = None, in_bias_name: str | None = None,
                 out_bias_name: str | None = None):
        if kernel_size < 2:
            raise ValueError(f"a short convolution needs >= 2 taps, got {kernel_size}")       # src/model.zig:486
        self.hidden, self.K = hidden, kernel_size
        self.in_name, self.conv_name, self.out_name = in_name, conv_name, out_name
        self.conv_bias_name, self.in_bias_name, self.out_bias_name = conv_bias_name, in_bias_name, out_bias_name
        self.w_in = self.w_out = self.taps = self.conv_bias = self.in_bias = self.out_bias = None
        # With D a multiple of 16 in_proj is stored as groups of 16 B rows, 16 C rows, 16 X rows, so
        # that a block of the fused single-token kernel reads 48 adjacent rows.
        self.interleave = FUSION_GROUP if hidden % FUSION_GROUP == 0 else 0

    def weight_specs(self):
        D, K = self.hidden, self.K
        specs = [WeightSpec(self.in_name, (3 * D, D)),
                 WeightSpec(self.conv_name, (D, K), role="vector", alt_shapes=((D, 1, K),)),
                 WeightSpec(self.out_name, (D, D))]
        if self.conv_bias_name:
            specs.append(WeightSpec(self.conv_bias_name, (D,), role="vector"))
        if self.in_bias_name:
            specs.append(WeightSpec(self.in_bias_name, (3 * D,), role="vector", optional=True, init="skip"))
        if self.out_bias_name:
            specs.append(WeightSpec(self.out_bias_name, (D,), role="vector", optional=True, init="skip"))
        return specs

    def load(self, weights, dtype, device):
        self.w_in, self.w_out = weights[self.in_name], weights[self.out_name]
        if self.interleave:
            D = self.hidden
            self.w_in = interleave_rows([self.w_in[:D], self.w_in[D:2 * D], self.w_in[2 * D:]])
        self.taps = weights[self.conv_name].reshape(self.hidden, self.K).t().contiguous()
        self.conv_bias = weights.get(self.conv_bias_name) if self.conv_bias_name else None
        self.in_bias = weights.get(self.in_bias_name) if self.in_bias_name else None
        if self.in_bias is not None and self.interleave:
            D = self.hidden
            self.in_bias = interleave_rows([self.in_bias[:D], self.in_bias[D:2 * D], self.in_bias[2 * D:]])
        self.out_bias = weights.get(self.out_bias_name) if self.out_bias_name else None

    def state_request(self):
        return StateRequest((self.K - 1, self.hidden), torch.float32)

    takes_pending_norm = True
    sums_through_linear = True

    def forward(self, ctx, call, xn, out, accumulate):
        state = call.state
        x = fused_input(xn, self.w_in, need_fused_rows=True, blocks=self.hidden // 16) \
            if ctx.is_decode and self.interleave else None
        if x is not None:                       # single tokens, few rows: in_proj and convolution in one kernel
            y = kernels.gemm_skinny_conv(x, self.w_in, self.in_bias, state, self.taps, self.conv_bias, ctx.seq_slot)
            linear(y, self.w_out, out=out, accumulate=accumulate, bias=self.out_bias)
            return
        bcx = linear(xn, self.w_in, bias=self.in_bias)
        if ctx.is_decode:
            y = kernels.conv_decode(bcx, state, self.taps, self.conv_bias, ctx.seq_slot, self.interleave)
        else:
            y = kernels.conv_forward(bcx, state, self.taps, self.conv_bias, ctx.tok_seq, ctx.cu_q, ctx.seq_slot,
                                     self.interleave)
            kernels.conv_state_update(bcx, state, ctx.cu_q, ctx.seq_slot, ctx.n_seqs, self.K, self.interleave)
        linear(y, self.w_out, out=out, accumulate=accumulate, bias=self.out_bias)


MIXERS.register("short_conv", ShortConv)
