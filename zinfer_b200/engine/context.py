"""What a step's kernels see of the batch: packed tokens and per-token / per-sequence index arrays.

The reference runs one sequence, so `pos0` and `nt` are all it needs (src/model.zig:2347-2359).
A batch of sequences with unequal lengths is packed here: the tokens of sequence b occupy rows
cu_q[b] .. cu_q[b+1] of every activation matrix, and stand at positions
seq_start[b] .. seq_start[b] + len_b of the sequence.  All arrays are int32 and live in ONE
device buffer that a step fills with a single host-to-device copy.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch


def batch_layout(n_tokens: int, n_seqs: int) -> dict[str, tuple[int, int]]:
    """Offsets (in int32 elements) of each array inside the step buffer."""
    out, off = {}, 0
    for name, size in (("tokens", n_tokens), ("tok_seq", n_tokens), ("tok_pos", n_tokens), ("cu_q", n_seqs + 1),
                       ("seq_start", n_seqs), ("seq_slot", n_seqs)):
        out[name] = (off, size)
        off += -(-size // 4) * 4            # keep every array 16-byte aligned
    out["_total"] = (off, 0)
    return out


def pack_batch(slots: Sequence[int], starts: Sequence[int], token_lists: Sequence[Sequence[int]]) -> np.ndarray:
    """The step buffer on the host for sequences `slots[b]` continuing at `starts[b]`."""
    lens = [len(t) for t in token_lists]
    n, B = sum(lens), len(slots)
    lay = batch_layout(n, B)
    buf = np.zeros(lay["_total"][0], dtype=np.int32)
    cu = np.zeros(B + 1, dtype=np.int64)
    np.cumsum(lens, out=cu[1:])
    o = lay["tokens"][0]
    buf[o:o + n] = np.concatenate([np.asarray(t, dtype=np.int64) for t in token_lists]) if n else []
    o = lay["tok_seq"][0]
    buf[o:o + n] = np.repeat(np.arange(B), lens)
    o = lay["tok_pos"][0]
    buf[o:o + n] = np.concatenate([np.arange(s, s + l) for s, l in zip(starts, lens)]) if n else []
    o = lay["cu_q"][0]
    buf[o:o + B + 1] = cu
    o = lay["seq_start"][0]
    buf[o:o + B] = starts
    o = lay["seq_slot"][0]
    buf[o:o + B] = slots
    return buf


def attn_tiles_host(q_lens: Sequence[int], bq: int) -> np.ndarray:
    """Query tiles of `bq` tokens: rows [tile_seq; tile_q0] as one int32 array [2, n_tiles]."""
    seq, q0 = [], []
    for b, l in enumerate(q_lens):
        for s in range(0, l, bq):
            seq.append(b)
            q0.append(s)
    return np.asarray([seq, q0], dtype=np.int32).reshape(2, len(seq))


@dataclass
class CallContext:
    """What a mixer sees of the schedule entry it runs in."""

    index: int                       # position in the schedule
    layer: int                       # which layer's weights
    kv: Optional[object]             # cache.KVView or None
    writes_kv: bool
    state: Optional[torch.Tensor]    # [slots, *state shape] or None


class StepContext:
    """One step's batch on the device.  Built by the engine; parts only read it."""

    def __init__(self, dtype: torch.dtype, device, status: torch.Tensor, buf: torch.Tensor, n_tokens: int,
                 n_seqs: int, q_lens: Sequence[int], max_kv_len: int, split_keys: int = 0,
                 tiles: Optional[dict] = None):
        self.dtype, self.device, self.status = dtype, device, status
        self.n_tokens, self.n_seqs = n_tokens, n_seqs
        self.q_lens = list(q_lens)
        self.max_q_len = max(self.q_lens) if self.q_lens else 0
        self.max_kv_len = max_kv_len
        self.is_decode = self.max_q_len == 1 and n_tokens == n_seqs
        self._split_keys = split_keys
        self._buf = buf
        lay = batch_layout(n_tokens, n_seqs)
        for name in ("tokens", "tok_seq", "tok_pos", "cu_q", "seq_start", "seq_slot"):
            o, size = lay[name]
            setattr(self, name, buf[o:o + size])
        # query-tile tables by tile size; a caller that reuses the same batch shape may share them
        self._tiles: dict[int, tuple[torch.Tensor, torch.Tensor]] = {} if tiles is None else tiles

    def attn_tiles(self, bq: int):
        """(tile_seq, tile_q0) device arrays for query tiles of `bq` tokens."""
        t = self._tiles.get(bq)
        if t is None:
            host = attn_tiles_host(self.q_lens, bq)
            dev = torch.from_numpy(host).to(self.device, non_blocking=True)
            t = (dev[0].contiguous(), dev[1].contiguous())
            self._tiles[bq] = t
        return t

    def set_tiles(self, bq: int, tile_seq: torch.Tensor, tile_q0: torch.Tensor) -> None:
        self._tiles[bq] = (tile_seq, tile_q0)

    def kv_splits(self, n_kv_heads: int) -> tuple[int, int]:
        """(number of key chunks, keys per chunk) for the attention of this step.  Single-token
        steps cut the keys so that the GPU's 148 SMs have work (the reference splits single-token
        attention into up to 16 chunks for its threads, src/model.zig:1941-1955); the cuts lie at
        multiples of `split_keys`, independent of the batch."""
        if not self.is_decode or self.max_kv_len <= 0:
            return 1, 0
        keys = self._split_keys
        if keys <= 0:
            # about four blocks per SM, chunks of 128 to 4096 keys: with unequal sequences a longer
            # chunk leaves the SMs that drew a short sequence idle (64 sequences of 1K to 32K tokens:
            # 3.90 ms a step with chunks of 16K keys, 3.27 ms with 4K)
            blocks = max(1, self.n_seqs * n_kv_heads)
            want = max(1, -(-592 // blocks))
            keys = min(4096, max(128, -(-self.max_kv_len // want)))
            keys = -(-keys // 64) * 64
        n = -(-self.max_kv_len // keys)
        return (n, keys) if n > 1 else (1, 0)
