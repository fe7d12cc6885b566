"""Grouped-query attention mixer over the paged cache (src/model.zig:1715-1991).

q, k, v come from one contraction against the stacked [Q + 2KV, D] weight (the reference fuses
them in one dispatch, src/model.zig:1720-1734); then per-head RMSNorm of q and k with the
layer's eps, before the rotation (src/model.zig:1741-1744, 1760-1763); keys and values are
written to the cache at the tokens' absolute positions; every query then attends to the cache
(its own token included) under the causal mask and an optional window
(src/model.zig:1362-1363); the output projection adds into the residual stream
(src/model.zig:1988-1990).  Scores are scaled by 1/sqrt(head_dim) (src/model.zig:465).

A call that reads another call's cache (`call.writes_kv` False) computes only its queries.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import kernels
from .base import MIXERS, KVRequest, Mixer, PositionEncoding, WeightSpec
from .linear import linear


class GqaAttention(Mixer):
    def __init__(self, hidden: int, n_heads: int, n_kv_heads: int, head_dim: int, q_name: str, k_name: str,
                 v_name: str, out_name: str, q_norm_name: Optional[str] = None, k_norm_name: Optional[str] = None,
                 norm_eps: float = 1e-5, position: Optional[PositionEncoding] = None, window: int = 0,
                 scale: Optional[float] = None):
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads are not a multiple of {n_kv_heads} KV heads")    # src/model.zig:487
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

    def kv_request(self):
        return KVRequest(self.n_kv, self.head_dim, self.window)

    takes_pending_norm = True

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
        tile_seq, tile_q0 = ctx.attn_tiles(tile_tokens)
        num_splits, split_keys = ctx.kv_splits(self.n_kv)
        att = kernels.attention(q, kv.k, kv.v, tile_seq, tile_q0, ctx.cu_q, ctx.seq_start, ctx.seq_slot,
                                kv.page_table, self.n_heads, self.n_kv, self.head_dim, self.scale, self.window,
                                num_splits, split_keys, single_token=ctx.is_decode, kind=kind)
        linear(att, self.w_out, out=out, accumulate=accumulate)


MIXERS.register("gqa_attention", GqaAttention)
