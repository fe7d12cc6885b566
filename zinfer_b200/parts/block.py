"""Pre-norm decoder block with two residual sums: x += Mixer(norm(x)); x += FFN(norm(x))
(src/model.zig:2395-2422).  The residual stream x is float32; each sum is the `accumulate`
store of the part's last contraction (src/model.zig:918-920).

A part that sets `takes_pending_norm = True` receives its input as the norm's `pending` form (a
`NormedRows`: the norm not yet applied) when the norm has one, and passes it to `linear` or a
fused kernel; any other part, and any part behind a norm without that form, receives a tensor.

A part that sets `sums_through_linear = True` uses `out` only as the `out=` of its last `linear`
call.  It may then be handed, in place of the residual rows, what the NEXT norm's `ahead`
returned (a `ResidualSink`), so that the kernel of that contraction writes the next norm's inputs
beside the sum.  The next norm is the block's own second norm for the mixer, and for the
feed-forward whatever the model says runs next (`forward_chained`)."""
from __future__ import annotations

from .base import BLOCKS, Block, FeedForward, Mixer, Norm


class PreNormBlock(Block):
    def __init__(self, mixer_norm: Norm, mixer: Mixer, ffn_norm: Norm, ffn: FeedForward):
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = mixer_norm, mixer, ffn_norm, ffn

    def parts(self):
        return [self.mixer_norm, self.mixer, self.ffn_norm, self.ffn]

    def entry_norm(self):
        return self.mixer_norm

    def forward(self, ctx, call, x):
        self.forward_chained(ctx, call, x)

    def forward_chained(self, ctx, call, x, entry=None, next_norm=None):
        mid = ahead_for(self.mixer, self.ffn_norm, ctx, x)
        self.mixer.forward(ctx, call, normed_for(self.mixer, self.mixer_norm, ctx, x, entry),
                           x if mid is None else mid, True)
        last = ahead_for(self.ffn, next_norm, ctx, x)
        self.ffn.forward(ctx, normed_for(self.ffn, self.ffn_norm, ctx, x, mid), x if last is None else last, True)
        return last


def normed_for(consumer, norm: Norm, ctx, x, prepared=None):
    """norm(x) for `consumer`: still pending if the consumer takes that and the norm offers it.
    `prepared`: what `ahead_for` returned for this norm before the rows were last summed into."""
    if getattr(consumer, "takes_pending_norm", False):
        p = norm.pending(ctx, x) if prepared is None else norm.pending(ctx, x, prepared)
        if p is not None:
            return p
    return norm.forward(ctx, x)


def ahead_for(producer, norm, ctx, x):
    """What `producer` gets as `out` in place of `x` so that its last contraction prepares `norm`,
    or None: the producer must sum through `linear`, and the norm must offer `ahead`."""
    if norm is None or not getattr(producer, "sums_through_linear", False):
        return None
    ahead = getattr(norm, "ahead", None)
    return ahead(ctx, x) if ahead is not None else None


BLOCKS.register("prenorm", PreNormBlock)
