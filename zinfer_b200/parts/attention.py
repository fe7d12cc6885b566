"""Grouped-query attention mixer over the paged cache (src/model.zig:1715-1991).

q, k, v come from one contraction against the stacked [Q + 2KV, D] weight (the reference fuses
them in one dispatch, src/model.zig:1720-1734); then per-head RMSNorm of q and k with the
layer's eps, before the rotation (src/model.zig:1741-1744, 1760-1763); keys and values are
written to the cache at the tokens' absolute positions; every query then attends to the cache
(its own token included) under the causal mask and an optional window
(src/model.zig:1362-1363); the output projection adds into the residual stream
(src/model.zig:1988-1990).  Scores are scaled by 1/sqrt(head_dim) (src/model.zig:465).

A call that reads another call's cache (`call.writes_kv` False) computes only its queries.

How the kernels are launched is decided here, not by the engine: the table of query tiles of a
step, and for single-token steps the cut of a sequence's keys into chunks that separate blocks
walk (the reference cuts single-token attention into up to 16 chunks for its threads,
src/model.zig:1941-1955).
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import numpy as np
import torch

from .. import kernels
from .base import MIXERS, KVRequest, Mixer, PositionEncoding, WeightSpec
from .linear import linear


def query_tiles(q_lens: Sequence[int], bq: int) -> np.ndarray:
    """Query tiles of `bq` tokens: rows [tile_seq; tile_q0] as one int32 array [2, n_tiles]."""
    seq, q0 = [], []
    for b, l in enumerate(q_lens):
        for s in range(0, l, bq):
            seq.append(b)
            q0.append(s)
    return np.asarray([seq, q0], dtype=np.int32).reshape(2, len(seq))


def key_capacity(longest: int) -> int:
    """The smallest of 512, 768, 1024, 1536, 2048, 3072, ... that holds `longest` keys.  The chunks of a
    single-token step are laid out for this capacity, not for the longest sequence itself, so
    that the layout (which a recorded step bakes in) changes a few times in a sequence's life
    instead of every few hundred tokens; chunks beyond a sequence's end cost a block that exits."""
    cap = 512
    while cap < longest:
        cap = cap * 3 // 2 if cap & (cap - 1) == 0 else cap // 3 * 4
    return cap


CHUNK_ALIGN = 64            # chunk boundaries the single-token kernels take (their key tile)


def key_chunks(n_seqs: int, n_kv_heads: int, longest: int, sm_count: int, split_keys: int = 0) -> tuple[int, int]:
    """(number of key chunks, keys per chunk) for single-token attention of `n_seqs` sequences up to
    `longest` tokens long.  The cuts lie at multiples of the chunk size, whatever the batch, and
    the chunks are added in order by the merge kernel, so a sequence's result does not depend on its
    neighbours.  split_keys > 0 fixes the chunk size; otherwise it is chosen so that about four
    blocks per SM have work, between 128 and 4096 keys: with unequal sequences a longer chunk
    leaves the SMs that drew a short sequence idle (64 sequences of 1K to 32K tokens on a B200:
    3.90 ms a step with chunks of 16K keys, 3.27 ms with 4K)."""
    if longest <= 0:
        return 1, 0
    cap = key_capacity(longest)
    keys = split_keys
    if keys <= 0:
        blocks = max(1, n_seqs * n_kv_heads)
        want = max(1, -(-4 * max(sm_count, 1) // blocks))
        keys = min(4096, max(128, -(-cap // want)))
        keys = -(-keys // CHUNK_ALIGN) * CHUNK_ALIGN
    n = -(-cap // keys)
    return (n, keys) if n > 1 else (1, 0)


class GqaAttention(Mixer):
    capture_safe = True

    def __init__(self, hidden: int, n_heads: int, n_kv_heads: int, head_dim: int, q_name: str, k_name: str,
                 v_name: str, out_name: str, q_norm_name: Optional[str] = None, k_norm_name: Optional[str] = None,
                 norm_eps: float = 1e-5, position: Optional[PositionEncoding] = None, window: int = 0,
                 scale: Optional[float] = None, split_keys: int = 0):
        """split_keys: keys per chunk of single-token attention, a multiple of 64 (0 = chosen per
        step from the batch and the GPU's size)."""
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads are not a multiple of {n_kv_heads} KV heads")    # src/model.zig:487
        self.split_keys = int(split_keys)
        self._sm_count = 0
        self.hidden, self.n_heads, self.n_kv, self.head_dim = hidden, n_heads, n_kv_heads, head_dim
        self.q_name, self.k_name, self.v_name, self.out_name = q_name, k_name, v_name, out_name
        self.q_norm_name, self.k_norm_name = q_norm_name, k_norm_name
        self.eps, self.position, self.window = float(norm_eps), position, int(window)
        self.scale = 1.0 / math.sqrt(head_dim) if scale is None else float(scale)
        self.w_qkv = self.w_out = self.q_norm = self.k_norm = None

    @property
    def q_dim(self):
        return self.n_heads * self.head_dim

    @property
    def kv_dim(self):
        return self.n_kv * self.head_dim

    def parts(self):
        return [self.position] if self.position is not None else []

    def weight_specs(self):
        specs = [WeightSpec(self.q_name, (self.q_dim, self.hidden)),
                 WeightSpec(self.k_name, (self.kv_dim, self.hidden)),
                 WeightSpec(self.v_name, (self.kv_dim, self.hidden)),
                 WeightSpec(self.out_name, (self.hidden, self.q_dim))]
        for n in (self.q_norm_name, self.k_norm_name):
            if n is not None:
                specs.append(WeightSpec(n, (self.head_dim,), role="vector", init="norm"))
        return specs

    def load(self, weights, dtype, device):
        self.w_qkv = torch.cat([weights[self.q_name], weights[self.k_name], weights[self.v_name]], dim=0).contiguous()
        self.w_out = weights[self.out_name]
        self.q_norm = weights[self.q_norm_name] if self.q_norm_name else None
        self.k_norm = weights[self.k_norm_name] if self.k_norm_name else None
        self._sm_count = kernels.sm_count(device) if torch.device(device).type == "cuda" else 0

    def kv_request(self):
        return KVRequest(self.n_kv, self.head_dim, self.window)

    def check(self, dtype, page_size):
        most = kernels.attn_max_head_dim()
        if self.head_dim % 2 or self.head_dim > most:        # the reference: a multiple of 8, at most 512 (src/model.zig:1469)
            raise ValueError(f"attention: head_dim {self.head_dim} must be even and at most {most}")
        if self.split_keys < 0 or self.split_keys % CHUNK_ALIGN:
            raise ValueError(f"attention: split_keys {self.split_keys} must be a multiple of {CHUNK_ALIGN}")

    def launch_key(self, n_seqs, longest):
        return key_chunks(n_seqs, self.n_kv, longest, self._sm_count, self.split_keys)

    takes_pending_norm = True
    sums_through_linear = True

    def forward(self, ctx, call, xn, out, accumulate):
        kv = call.kv
        qkv = linear(xn, self.w_qkv)
        rot = self.position.rotary() if self.position is not None else None
        fused = self.position is None or rot is not None
        common = dict(tok_seq=ctx.tok_seq, tok_pos=ctx.tok_pos, seq_slot=ctx.seq_slot, page_table=kv.page_table,
                      n_heads=self.n_heads, n_kv=self.n_kv, head_dim=self.head_dim, eps=self.eps, status=ctx.status)
        if fused:
            q = kernels.qk_prepare(qkv, kv.k, kv.v, self.q_norm, self.k_norm, rot.inv_freq if rot else None,
                                   n_rot=rot.n_rot if rot else 0, interleaved=rot.interleaved if rot else False,
                                   write_kv=call.writes_kv, **common)
        else:
            # A position encoding that is not a rotation table runs between the norm and the
            # cache write: norm in place of a copy of qkv, the encoding's own step, then the write.
            normed = kernels.qk_normed(qkv, self.q_norm, self.k_norm, self.n_heads, self.n_kv, self.head_dim, self.eps,
                                       ctx.tok_pos, ctx.status)
            self.position.apply(ctx, normed[:, :self.q_dim], normed[:, self.q_dim:self.q_dim + self.kv_dim])
            q = kernels.qk_prepare(normed, kv.k, kv.v, None, None, None, n_rot=0, interleaved=False,
                                   write_kv=call.writes_kv, **common)
        kind, tile_tokens = kernels.attention_plan(q.dtype, self.n_heads, self.n_kv, self.head_dim, kv.page_size,
                                                   ctx.is_decode, self.window)
        tile_seq, tile_q0 = ctx.memo(("query tiles", tile_tokens), lambda: self._tiles_on_device(ctx, tile_tokens))
        num_splits, split_keys = (key_chunks(ctx.n_seqs, self.n_kv, ctx.max_kv_len, self._sm_count, self.split_keys)
                                  if ctx.is_decode else (1, 0))
        att = kernels.attention(q, kv.k, kv.v, tile_seq, tile_q0, ctx.cu_q, ctx.seq_start, ctx.seq_slot,
                                kv.page_table, self.n_heads, self.n_kv, self.head_dim, self.scale, self.window,
                                num_splits, split_keys, single_token=ctx.is_decode, kind=kind)
        linear(att, self.w_out, out=out, accumulate=accumulate)


    @staticmethod
    def _tiles_on_device(ctx, tile_tokens: int):
        dev = torch.from_numpy(query_tiles(ctx.q_lens, tile_tokens)).to(ctx.device, non_blocking=True)
        return dev[0].contiguous(), dev[1].contiguous()


MIXERS.register("gqa_attention", GqaAttention)
