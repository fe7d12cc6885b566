"""Pre-norm decoder block with two residual sums: x += Mixer(norm(x)); x += FFN(norm(x))
(src/model.zig:2395-2422).  The residual stream x is float32; each sum is the `accumulate`
store of the part's last contraction (src/model.zig:918-920).

A part that sets `takes_pending_norm = True` receives its input as a `NormedRows` (the norm not
yet applied) and passes it to `linear` or a fused kernel; any other part receives a tensor."""
from __future__ import annotations

from .base import BLOCKS, Block, FeedForward, Mixer, Norm


class PreNormBlock(Block):
    def __init__(self, mixer_norm: Norm, mixer: Mixer, ffn_norm: Norm, ffn: FeedForward):
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = mixer_norm, mixer, ffn_norm, ffn

    def parts(self):
        return [self.mixer_norm, self.mixer, self.ffn_norm, self.ffn]

    def forward(self, ctx, call, x):
        xn = self.mixer_norm.forward(ctx, x, lazy=getattr(self.mixer, "takes_pending_norm", False))
        self.mixer.forward(ctx, call, xn, x, True)
        xn = self.ffn_norm.forward(ctx, x, lazy=getattr(self.ffn, "takes_pending_norm", False))
        self.ffn.forward(ctx, xn, x, True)


BLOCKS.register("prenorm", PreNormBlock)
