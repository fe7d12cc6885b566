"""Interfaces of the parts a decoder layer is put together from, and their registries.

A layer of the reference is a struct of norms plus a tagged union `mixer` in {attention,
shortconv} and a tagged union `ffn` in {dense, moe} (src/model.zig:189-215).  Here every part is
a class with its sizes and constants as constructor parameters; an architecture's builder
picks parts layer by layer from its configuration.  No part knows which model it is in: it sees
its own weights (by the names it was given), the step's batch (`StepContext`) and, for a
mixer, the cache view and state of the call it runs in (`CallContext`).

Interfaces
----------
Part            weight_specs() -> [WeightSpec]; load(weights: dict name -> tensor, dtype, device)
Norm            forward(ctx, x_f32, rows=None) -> tensor in the run dtype
PositionEncoding  rotary() -> RotaryParams | None (lets the mixer fuse it), or
                  apply(ctx, q, k) -> None to rotate / shift in place on its own
Mixer           kv_request() -> KVRequest | None      growing cache it needs
                state_request() -> StateRequest | None  fixed-size per-sequence state it needs
                forward(ctx, call, xn, out, accumulate)  out (+)= mixer(xn); out is float32
FeedForward     forward(ctx, xn, out, accumulate)
Block           forward(ctx, call, x)  updates the float32 residual stream x in place
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Optional

import torch


@dataclass(frozen=True)
class WeightSpec:
    """One tensor a part wants from the weight file.

    role: "matrix" is kept in the run dtype (bfloat16, or float32 in the 32-bit path);
    "vector" (norm weights, conv taps, biases) is kept in float32, which holds a stored
    bfloat16 or float32 value exactly; "table" is an integer table kept as int32.
    init: how the random-weights mode fills it ("normal", "one_plus_normal", "zeros").
    alt_shapes: other stored shapes with the same element order (e.g. [D, 1, K] for [D, K]);
    the random-weights mode stores the first of them if there is one.
    """

    name: str
    shape: tuple[int, ...]
    role: str = "matrix"
    optional: bool = False
    init: str = "normal"
    alt_shapes: tuple[tuple[int, ...], ...] = ()


@dataclass(frozen=True)
class KVRequest:
    """A growing per-token cache: keys and values of `n_kv_heads` x `head_dim` per token.
    window = 0 keeps every token; window = W lets the cache drop tokens more than W behind."""

    n_kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateRequest:
    """Fixed-size per-sequence state, zero when a sequence starts."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass(frozen=True)
class RotaryParams:
    inv_freq: torch.Tensor          # [n_rot / 2] float32 on the device
    n_rot: int
    interleaved: bool = False


class Part:
    def weight_specs(self) -> list[WeightSpec]:
        return []

    def load(self, weights: dict[str, torch.Tensor], dtype: torch.dtype, device) -> None:
        """Takes its tensors (already in the dtype their role asks for, on `device`)."""

    def parts(self) -> list["Part"]:
        """Nested parts, so that a block's weights are found through it."""
        return []


class Norm(Part):
    def forward(self, ctx, x: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    def rotary(self) -> Optional[RotaryParams]:
        return None

    def apply(self, ctx, q: torch.Tensor, k: torch.Tensor) -> None:
        raise NotImplementedError


class Mixer(Part):
    def kv_request(self) -> Optional[KVRequest]:
        return None

    def state_request(self) -> Optional[StateRequest]:
        return None

    def forward(self, ctx, call, xn: torch.Tensor, out: torch.Tensor, accumulate: bool) -> None:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx, xn: torch.Tensor, out: torch.Tensor, accumulate: bool) -> None:
        raise NotImplementedError


class Block(Part):
    mixer: Mixer

    def forward(self, ctx, call, x: torch.Tensor) -> None:
        raise NotImplementedError


# ------------------------------------------------------------------------------- registries

class Registry:
    """Name -> factory.  `register` refuses to overwrite silently; `get` lists what exists."""

    def __init__(self, what: str):
        self.what = what
        self._items: dict[str, Callable] = {}

    def register(self, name: str, factory: Callable | None = None, *, replace: bool = False):
        def put(f):
            if name in self._items and not replace:
                raise KeyError(f"{self.what} '{name}' is already registered")
            self._items[name] = f
            return f

        return put if factory is None else put(factory)

    def unregister(self, name: str) -> None:
        self._items.pop(name, None)

    def get(self, name: str) -> Callable:
        try:
            return self._items[name]
        except KeyError:
            raise KeyError(f"unknown {self.what} '{name}'; registered: {sorted(self._items)}") from None

    def names(self) -> list[str]:
        return sorted(self._items)

    def __contains__(self, name: str) -> bool:
        return name in self._items


MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
BLOCKS = Registry("block")


def walk_parts(part: Part):
    """The part and everything nested in it, depth first."""
    yield part
    for p in part.parts():
        yield from walk_parts(p)
