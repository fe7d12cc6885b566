"""Pre-norm decoder block with two residual sums: x += Mixer(norm(x)); x += FFN(norm(x))
(src/model.zig:2395-2422).  The residual stream x is float32; each sum is the `accumulate`
store of the part's last contraction (src/model.zig:918-920).

A part that sets `takes_pending_norm = True` receives its input as the norm's `pending` form (a
`NormedRows`: the norm not yet applied) when the norm has one, and passes it to `linear` or a
fused kernel; any other part, and any part behind a norm without that form, receives a tensor."""
from __future__ import annotations

from .base import BLOCKS, Block, FeedForward, Mixer, Norm


class PreNormBlock(Block):
    def __init__(self, mixer_norm: Norm, mixer: Mixer, ffn_norm: Norm, ffn: FeedForward):
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = mixer_norm, mixer, ffn_norm, ffn

    def parts(self):
        return [self.mixer_norm, self.mixer, self.ffn_norm, self.ffn]

    def forward(self, ctx, call, x):
        self.mixer.forward(ctx, call, normed_for(self.mixer, self.mixer_norm, ctx, x), x, True)
        self.ffn.forward(ctx, normed_for(self.ffn, self.ffn_norm, ctx, x), x, True)


def normed_for(consumer, norm: Norm, ctx, x):
    """norm(x) for `consumer`: still pending if the consumer takes that and the norm offers it."""
    if getattr(consumer, "takes_pending_norm", False):
        p = norm.pending(ctx, x)
        if p is not None:
            return p
    return norm.forward(ctx, x)


BLOCKS.register("prenorm", PreNormBlock)
