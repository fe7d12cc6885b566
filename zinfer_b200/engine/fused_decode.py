"""The single-token step as ONE kernel launch: a program of operations built from the model.

`csrc/fused_decode.cu` runs the whole chain of a single-token step (embedding, every layer's
contractions with their fused prologues and epilogues, attention, the head) in one persistent
grid with grid-wide barriers between dependent operations, and streams the weights through a
shared-memory ring that runs ahead of the barriers.  This module turns a `Model` into that
kernel's program.  It knows the library's parts (`PreNormBlock`, `RMSNorm`, `ShortConv`,
`GqaAttention` with a rotary encoding, `SwiGLU`, `TokenEmbedding`, `LMHead`); for a model with any
other part, a dtype other than bfloat16, or sizes the kernel does not take, `build` returns None
and the engine keeps launching the parts' own kernels.  The reference runs the same chain as one
loop over its layers (src/model.zig:2395-2422, 2484-2490).

The engine uses it only when asked (`Engine(fused_decode=True)`): on a B200 a step of 8 sequences
of an LFM2-1.2B-shaped model takes 1.40 ms this way and 1.04 ms as a graph of separate kernels.
`FusedDecodePlan.trace` shows where the time goes: per operation about 2 us at the barrier and
2 to 3.5 us staging the input (each a chain of L2 round trips), the contraction loops at some
35 GB/s per SM, and attention without a split of a sequence's keys over blocks.
"""
from __future__ import annotations

from typing import Optional

import numpy
import torch

from .. import kernels
from ..parts import GqaAttention, PreNormBlock, RMSNorm, ShortConv, SwiGLU
from ..parts.embedding import LMHead, TokenEmbedding

K = kernels


class FusedDecodePlan:
    """Program and activation buffers of the fused step for a fixed number of sequences."""

    def __init__(self, n_rows: int, ops: list, buffers: dict, logits: torch.Tensor, device):
        self.n_rows, self.n_ops = n_rows, len(ops)
        self.names = [{K.FUSED_OP_EMBED: "embed", K.FUSED_OP_ATTN: "attention"}.get(
            o.kind, f"gemm {o.N}x{o.K}" + (" norm" if o.xin == K.FUSED_XIN_NORM else "")
            + {K.FUSED_EPI_SWIGLU: " swiglu", K.FUSED_EPI_CONV: " conv", K.FUSED_EPI_ACC_F32: " +=x"}.get(o.epi, ""))
            for o in ops]
        raw = b"".join(bytes(o) for o in ops)
        self.ops = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(device)
        self.buffers, self.logits = buffers, logits
        self.barrier = torch.zeros(1, dtype=torch.int32, device=device)
        self.n_blocks = torch.cuda.get_device_properties(device).multi_processor_count

    def run(self, ctx, trace: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Launches the step for the batch in `ctx`; returns the float32 logits [n_rows, vocab]
        (the plan's own buffer, overwritten by the next run)."""
        self.barrier.zero_()
        kernels.fused_decode(self.ops, self.n_ops, self.n_rows, ctx.tokens, ctx.seq_start, ctx.seq_slot, self.barrier,
                             ctx.status, self.n_blocks, trace)
        return self.logits

    def trace(self, ctx, repeats: int = 5) -> list[dict]:
        """Runs the step `repeats` times with the kernel's time stamps on and returns, for each
        operation, its name and the microseconds block 0 spent staging its input, working and
        waiting at the barrier (the smallest of the repeats).  Each run is a real step: it writes
        the cache at the positions `ctx` names and moves the convolution states on."""
        stamps = torch.zeros(self.n_ops * 4, dtype=torch.int64, device=self.ops.device)
        best = None
        for _ in range(repeats):
            self.run(ctx, stamps)
            t = stamps.cpu().numpy().reshape(-1, 4).astype("float64")
            d = [t[:, 1] - t[:, 0], t[:, 2] - t[:, 1], t[:, 3] - t[:, 2], t[:, 2] - t[:, 0]]
            best = d if best is None else [numpy.minimum(a, b) for a, b in zip(best, d)]
        out = []
        for i, name in enumerate(self.names):
            staged = name.startswith("gemm")
            out.append({"op": name, "stage_us": best[0][i] / 1e3 if staged else 0.0,
                        "work_us": (best[1][i] if staged else best[3][i]) / 1e3,
                        "barrier_us": max(best[2][i], 0.0) / 1e3})
        return out


def _gemm(xin, x, w, out, epi, n_out, rg, ldx, ldc, norm=None, bias=None) -> "kernels.FusedOp":
    op = K.FusedOp()
    op.kind, op.xin, op.epi, op.rg = K.FUSED_OP_GEMM, xin, epi, rg
    op.N, op.K, op.ldw, op.ldx, op.ldc = n_out, w.shape[1], w.stride(0), ldx, ldc
    op.W, op.X, op.C = w.data_ptr(), x.data_ptr(), out.data_ptr()
    if norm is not None:
        op.norm_w, op.eps = norm.weight.data_ptr(), norm.eps
    if bias is not None:
        op.bias = bias.data_ptr()
    return op


def _plain_rg(n_rows_of_w: int, n_blocks: int) -> int:
    return 2 if n_rows_of_w >= 16 * n_blocks * 6 else 1


def build(engine, n_rows: int) -> Optional[FusedDecodePlan]:
    """The fused program of `engine.model` for `n_rows` sequences, or None if it cannot be fused."""
    model, dev = engine.model, engine.device
    if engine.dtype != torch.bfloat16 or torch.device(dev).type != "cuda":
        return None
    lim = kernels.fused_decode_limits(n_rows)
    if n_rows > lim["max_rows"]:
        return None
    emb, head, fnorm = model.embedding, model.head, model.final_norm
    if not (type(emb) is TokenEmbedding and type(head) is LMHead and type(fnorm) is RMSNorm):
        return None
    D = emb.dim
    if D % 32 or D > lim["max_staged_k"]:
        return None
    n_blocks = torch.cuda.get_device_properties(dev).multi_processor_count
    bf, f32 = torch.bfloat16, torch.float32
    buf = {"x": torch.zeros((n_rows, D), dtype=f32, device=dev)}
    ops: list = []

    def tensor(name, cols, dtype=bf):
        t = buf.get(name)
        if t is None or t.shape[1] < cols:
            t = buf[name] = torch.zeros((n_rows, cols), dtype=dtype, device=dev)
        return t

    def usable(w):
        return (w is not None and w.dtype == bf and w.is_contiguous() and w.shape[1] % 32 == 0
                and w.data_ptr() % 16 == 0)

    op = K.FusedOp()
    op.kind, op.K, op.vocab, op.scale = K.FUSED_OP_EMBED, D, emb.vocab, emb.scale
    op.table, op.C = emb.weight.data_ptr(), buf["x"].data_ptr()
    if emb.weight.dtype != bf:
        return None
    ops.append(op)

    for call in engine.calls:
        block = model.layers[call.layer]
        if type(block) is not PreNormBlock or type(block.mixer_norm) is not RMSNorm or type(block.ffn_norm) is not RMSNorm:
            return None
        mixer, ffn = block.mixer, block.ffn
        if type(mixer) is ShortConv:
            if not (mixer.interleave == 16 and usable(mixer.w_in) and usable(mixer.w_out) and call.state is not None):
                return None
            y = tensor("y", D)
            op = _gemm(K.FUSED_XIN_NORM, buf["x"], mixer.w_in, y, K.FUSED_EPI_CONV, D, 3, D, y.stride(0),
                       norm=block.mixer_norm, bias=mixer.in_bias)
            op.conv_state, op.state_stride = call.state.data_ptr(), call.state.stride(0)
            op.conv_taps, op.taps = mixer.taps.data_ptr(), mixer.K
            if mixer.conv_bias is not None:
                op.conv_bias = mixer.conv_bias.data_ptr()
            ops.append(op)
            ops.append(_gemm(K.FUSED_XIN_BF16, y, mixer.w_out, buf["x"], K.FUSED_EPI_ACC_F32, D,
                             _plain_rg(D, n_blocks), y.stride(0), D, bias=mixer.out_bias))
        elif type(mixer) is GqaAttention:
            rot = mixer.position.rotary() if mixer.position is not None else None
            kv = call.kv
            if not (call.writes_kv and kv is not None and (mixer.position is None or rot is not None)
                    and usable(mixer.w_qkv) and usable(mixer.w_out)
                    and kernels.fused_decode_attn_takes(mixer.n_heads, mixer.n_kv, mixer.head_dim, kv.page_size)):
                return None
            width = mixer.q_dim + 2 * mixer.kv_dim
            qkv, att = tensor("qkv", width), tensor("att", mixer.q_dim)
            ops.append(_gemm(K.FUSED_XIN_NORM, buf["x"], mixer.w_qkv, qkv, K.FUSED_EPI_BF16, width,
                             _plain_rg(width, n_blocks), D, qkv.stride(0), norm=block.mixer_norm))
            op = K.FusedOp()
            op.kind = K.FUSED_OP_ATTN
            op.H, op.Hkv, op.hd, op.page_size, op.window = mixer.n_heads, mixer.n_kv, mixer.head_dim, kv.page_size, mixer.window
            op.pt_stride, op.eps, op.scale = kv.page_table.stride(0), mixer.eps, mixer.scale
            op.X, op.C = qkv.data_ptr(), att.data_ptr()
            op.k_cache, op.v_cache, op.page_table = kv.k.data_ptr(), kv.v.data_ptr(), kv.page_table.data_ptr()
            if mixer.q_norm is not None:
                op.q_norm = mixer.q_norm.data_ptr()
            if mixer.k_norm is not None:
                op.k_norm = mixer.k_norm.data_ptr()
            if rot is not None:
                op.inv_freq, op.n_rot, op.rope_interleaved = rot.inv_freq.data_ptr(), rot.n_rot, int(rot.interleaved)
            if qkv.stride(0) != width or att.stride(0) != mixer.q_dim:
                return None
            ops.append(op)
            ops.append(_gemm(K.FUSED_XIN_BF16, att, mixer.w_out, buf["x"], K.FUSED_EPI_ACC_F32, D,
                             _plain_rg(D, n_blocks), att.stride(0), D))
        else:
            return None
        if type(ffn) is not SwiGLU or ffn.interleave != 16 or not (usable(ffn.w_gate_up) and usable(ffn.w_down)):
            return None
        F = ffn.ffn_dim
        h = tensor("h", F)
        ops.append(_gemm(K.FUSED_XIN_NORM, buf["x"], ffn.w_gate_up, h, K.FUSED_EPI_SWIGLU, F, 2, D, h.stride(0),
                         norm=block.ffn_norm))
        ops.append(_gemm(K.FUSED_XIN_BF16, h, ffn.w_down, buf["x"], K.FUSED_EPI_ACC_F32, D, _plain_rg(D, n_blocks),
                         h.stride(0), D))

    w_head = head.weight if head.weight is not None else head.embedding.weight
    if not usable(w_head):
        return None
    logits = torch.zeros((n_rows, head.vocab), dtype=f32, device=dev)
    ops.append(_gemm(K.FUSED_XIN_NORM, buf["x"], w_head, logits, K.FUSED_EPI_F32, head.vocab,
                     _plain_rg(head.vocab, n_blocks), D, logits.stride(0), norm=fnorm))
    return FusedDecodePlan(n_rows, ops, buf, logits, dev)
