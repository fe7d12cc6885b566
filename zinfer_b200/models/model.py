"""A model as data: an embedding, a list of layers, the order in which they run, a final norm
and an output head.  The reference's forward pass is this loop over its layer array
(src/model.zig:2347-2516); here the order is a list of its own (`schedule`), so a layer may be
named twice or read the cache of another entry."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from ..cache.manager import CallCacheSpec
from ..config.base import ModelConfig
from ..parts.base import Block, Norm, Part, WeightSpec, walk_parts
from ..parts.block import normed_for
from ..parts.embedding import LMHead, TokenEmbedding


@dataclass(frozen=True)
class LayerCall:
    """One entry of the schedule: run `layer`; `cache_of` names the earlier entry (by its index
    in the schedule) whose keys and values this entry reads instead of writing its own."""

    layer: int
    cache_of: Optional[int] = None


class Model:
    def __init__(self, config: ModelConfig, embedding: TokenEmbedding, layers: Sequence[Block],
                 final_norm: Norm, head: LMHead, schedule: Optional[Sequence[LayerCall]] = None,
                 ignorable_weights: Sequence[str] = ()):
        self.config = config
        self.embedding, self.layers, self.final_norm, self.head = embedding, list(layers), final_norm, head
        self.schedule = list(schedule) if schedule is not None else [LayerCall(i) for i in range(len(self.layers))]
        self.ignorable_weights = tuple(ignorable_weights)
        self.dtype: Optional[torch.dtype] = None
        self.device = None
        for c, call in enumerate(self.schedule):
            if not 0 <= call.layer < len(self.layers):
                raise ValueError(f"schedule[{c}] names layer {call.layer}, the model has {len(self.layers)}")
            if call.cache_of is not None and not 0 <= call.cache_of < c:
                raise ValueError(f"schedule[{c}] reads the cache of entry {call.cache_of}, which does not run before it")

    # ------------------------------------------------------------------ weights
    def all_parts(self) -> list[Part]:
        out: list[Part] = []
        seen: set[int] = set()
        for top in (self.embedding, *self.layers, self.final_norm, self.head):
            for p in walk_parts(top):
                if id(p) not in seen:
                    seen.add(id(p))
                    out.append(p)
        return out

    def weight_specs(self) -> dict[str, WeightSpec]:
        specs: dict[str, WeightSpec] = {}
        for p in self.all_parts():
            for s in p.weight_specs():
                if s.name in specs and specs[s.name] != s:
                    raise ValueError(f"tensor '{s.name}' is wanted twice with different shapes or roles")
                specs[s.name] = s
        return specs

    def load_weights(self, weights: dict[str, torch.Tensor], dtype: torch.dtype, device) -> None:
        """`weights`: name -> tensor already on `device` in the dtype its role asks for."""
        self.dtype, self.device = dtype, device
        for p in self.all_parts():
            p.load(weights, dtype, device)

    # ------------------------------------------------------------------ cache needs
    def cache_specs(self) -> list[CallCacheSpec]:
        specs = []
        for call in self.schedule:
            mixer = self.layers[call.layer].mixer
            specs.append(CallCacheSpec(kv=mixer.kv_request(), kv_owner=call.cache_of, state=mixer.state_request()))
        return specs

    # ------------------------------------------------------------------ forward
    def forward(self, ctx, calls, want_rows: Optional[torch.Tensor], want_all: bool = False,
                out: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Runs the step's tokens through every schedule entry; returns float32 logits of the rows
        listed in `want_rows` (row indices into the packed tokens), of every row with `want_all`
        (written into `out` if given), or None when none is wanted.  Only wanted rows meet the
        final norm and the head (src/model.zig:2482-2490)."""
        x = self.embedding.forward(ctx, ctx.tokens)
        carried = None      # what a block's last contraction prepared for the norm that reads x next
        for i, call_ctx in enumerate(calls):
            if i + 1 < len(calls):
                next_norm = self.layers[calls[i + 1].layer].entry_norm()
            else:
                next_norm = self.final_norm if want_all else None
            carried = self.layers[call_ctx.layer].forward_chained(ctx, call_ctx, x, carried, next_norm)
        if want_all:
            return self.head.forward(ctx, normed_for(self.head, self.final_norm, ctx, x, carried), out=out)
        if want_rows is None or want_rows.numel() == 0:
            return None
        xn = self.final_norm.forward(ctx, x, rows=want_rows)
        return self.head.forward(ctx, xn)
