"""Token embedding and output head.  x_t = E[token_t] (times a scale, 1 here:
src/model.zig:2352-2358, 466); logits = xn W_out^T in float32 with W_out the head tensor or
the embedding itself when tied (src/model.zig:595-598, 2490)."""
from __future__ import annotations

import torch

from .. import kernels
from .base import Part, WeightSpec
from .linear import linear


class TokenEmbedding(Part):
    def __init__(self, vocab: int, dim: int, weight_name: str, scale: float = 1.0):
        self.vocab, self.dim, self.weight_name, self.scale = vocab, dim, weight_name, float(scale)
        self.weight = None

    def weight_specs(self):
        return [WeightSpec(self.weight_name, (self.vocab, self.dim))]

    def load(self, weights, dtype, device):
        self.weight = weights[self.weight_name]

    def forward(self, ctx, tokens: torch.Tensor) -> torch.Tensor:
        return kernels.embed(tokens, self.weight, ctx.status, self.scale)


class LMHead(Part):
    """`weight_name` None ties the head to `embedding`."""

    def __init__(self, vocab: int, dim: int, weight_name: str | None, embedding: TokenEmbedding | None = None):
        if weight_name is None and embedding is None:
            raise ValueError("a tied head needs the embedding it is tied to")
        self.vocab, self.dim, self.weight_name, self.embedding = vocab, dim, weight_name, embedding
        self.weight = None

    def weight_specs(self):
        return [] if self.weight_name is None else [WeightSpec(self.weight_name, (self.vocab, self.dim))]

    def load(self, weights, dtype, device):
        self.weight = None if self.weight_name is None else weights[self.weight_name]

    takes_pending_norm = True

    def forward(self, ctx, xn, out: torch.Tensor | None = None) -> torch.Tensor:
        """float32 logits of the rows of xn (a tensor, or a norm still pending), into `out` if given."""
        w = self.weight if self.weight is not None else self.embedding.weight
        return linear(xn, w, out=out, out_dtype=torch.float32)
