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
                pending(ctx, x_f32) -> object | None   optional: the norm not yet applied, for a
                                                       consumer that can apply it itself
                ahead(ctx, x_f32) -> object | None     optional: a stand-in for x as the `out` of the
                                                       contraction that sums into x before this norm
PositionEncoding  rotary() -> RotaryParams | None (lets the mixer fuse it), or
                  apply(ctx, q, k) -> None to rotate / shift in place on its own
Mixer           kv_request() -> KVRequest | None      growing cache it needs
                state_request() -> StateRequest | None  fixed-size per-sequence state it needs
                forward(ctx, call, xn, out, accumulate)  out (+)= mixer(xn); out is float32
                check(dtype, page_size)               refuse sizes no kernel takes, at engine set-up
                capture_safe                          whether forward may be recorded in a CUDA graph
                launch_key(n_seqs, longest)           what a recorded single-token step bakes in
FeedForward     forward(ctx, xn, out, accumulate)
Block           forward(ctx, call, x)  updates the float32 residual stream x in place
                entry_norm() / forward_chained(...)   optional: lets the kernel that writes x last in
                                                       one block prepare the first norm of the next

Optional flags of a mixer or feed-forward, read by the block (parts.block):
takes_pending_norm     its input may be the norm's pending form
sums_through_linear    `out` is used only as `out=` of its last `linear` call and may be a ResidualSink
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
    """A growing per-token cache.  Per token and layer it holds `n_kv_heads` rows of `head_dim`
    values in a first tensor ("k") and `n_kv_heads` rows of `value_dim` values in a second ("v").
    value_dim None = as wide as head_dim (keys and values of attention); value_dim 0 = no
    second tensor (a mixer that keeps one vector per token, e.g. a latent).
    window = 0 keeps every token; window = W lets the cache drop tokens more than W behind."""

    n_kv_heads: int
    head_dim: int
    window: int = 0
    value_dim: Optional[int] = None

    @property
    def v_dim(self) -> int:
        return self.head_dim if self.value_dim is None else self.value_dim


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
        """The normalised rows of float32 `x` (all, or those listed in `rows`) in the run dtype."""
        raise NotImplementedError

    def pending(self, ctx, x: torch.Tensor):
        """The norm of all rows of `x` as an object that a consumer with `takes_pending_norm`
        resolves itself (parts.linear.NormedRows), or None if this norm has no such form; the
        caller then uses `forward`.  A norm that also has `ahead(ctx, x)` takes what that returned
        as a third argument."""
        return None


class PositionEncoding(Part):
    def rotary(self) -> Optional[RotaryParams]:
        return None

    def apply(self, ctx, q: torch.Tensor, k: torch.Tensor) -> None:
        raise NotImplementedError


class Mixer(Part):
    # Whether `forward` may be recorded into a CUDA graph: it launches kernels on the current
    # stream only, reads nothing back to the host, and its launches depend on the batch only
    # through (number of sequences, launch_key).  The engine replays single-token steps from
    # graphs only if every mixer of the model says so; otherwise it runs them one by one.
    capture_safe = False

    def kv_request(self) -> Optional[KVRequest]:
        return None

    def state_request(self) -> Optional[StateRequest]:
        return None

    def check(self, dtype: torch.dtype, page_size: int) -> None:
        """Raises ValueError if no kernel of this mixer takes its sizes with this run dtype and
        page size.  Called once when an engine is built, before anything runs."""

    def launch_key(self, n_seqs: int, longest: int):
        """What a recorded single-token step of `n_seqs` sequences, the longest of which then has
        `longest` tokens, bakes into its launches besides `n_seqs` (any hashable; None = nothing).
        A recorded step is replayed only for batches that give the same key."""
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

    def entry_norm(self) -> Optional[Norm]:
        """The norm this block applies to `x` before anything else, if the block before may
        prepare it (see forward_chained); None = nothing to prepare."""
        return None

    def forward_chained(self, ctx, call, x: torch.Tensor, entry=None, next_norm: Optional[Norm] = None):
        """As `forward`.  `entry`: what the block before returned, prepared for this block's
        entry_norm().  `next_norm`: the norm that reads `x` after this block.  Returns what this
        block's last contraction prepared for `next_norm` (to be handed on as `entry`), or None."""
        self.forward(ctx, call, x)
        return None


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
