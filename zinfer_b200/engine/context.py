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


@dataclass
class CallContext:
    """What a mixer sees of the schedule entry it runs in."""

    index: int                       # position in the schedule
    layer: int                       # which layer's weights
    kv: Optional[object]             # cache.KVView or None
    writes_kv: bool
    state: Optional[torch.Tensor]    # [slots, *state shape] or None


class StepContext:
    """One step's batch on the device.  Built by the engine; parts only read it.

    n_tokens, n_seqs; q_lens (host list: tokens each sequence brings), max_q_len, max_kv_len
    (longest sequence after the step), is_decode (one token for every sequence); the device
    arrays tokens, tok_seq, tok_pos [n_tokens], cu_q [n_seqs + 1], seq_start, seq_slot [n_seqs];
    `status` (the device's status word) and `sm_count`.  `memo` keeps what parts derive from the
    batch's shape alone (tile tables and the like), so that equal parts derive it once a step; a
    step that is recorded and replayed keeps its memo with the recording."""

    def __init__(self, dtype: torch.dtype, device, status: torch.Tensor, buf: torch.Tensor, n_tokens: int,
                 n_seqs: int, q_lens: Sequence[int], max_kv_len: int, memo: Optional[dict] = None,
                 sm_count: int = 0):
        self.dtype, self.device, self.status = dtype, device, status
        self.n_tokens, self.n_seqs = n_tokens, n_seqs
        self.q_lens = list(q_lens)
        self.max_q_len = max(self.q_lens) if self.q_lens else 0
        self.max_kv_len = max_kv_len
        self.is_decode = self.max_q_len == 1 and n_tokens == n_seqs
        self.sm_count = sm_count
        self._buf = buf
        lay = batch_layout(n_tokens, n_seqs)
        for name in ("tokens", "tok_seq", "tok_pos", "cu_q", "seq_start", "seq_slot"):
            o, size = lay[name]
            setattr(self, name, buf[o:o + size])
        self._memo: dict = {} if memo is None else memo

    def memo(self, key, make):
        """`make()` once per step (or recording) and key."""
        v = self._memo.get(key)
        if v is None:
            v = self._memo[key] = make()
        return v
