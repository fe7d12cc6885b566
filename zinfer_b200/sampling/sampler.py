"""Sampling parameters, per-request history and the host side of the device sampler.

Names, meanings and defaults of the options are the reference's `Params`
(src/sampler.zig:3-27): temp (<= 0 is greedy), top_k (0 = off), top_p, min_p, repeat_penalty
over the last 64 tokens (1 = off), DRY and XTC options, seed.  The filter chain and the draw run
on the device (csrc/sampling.cu); the host decides WHICH tokens the DRY penalty touches (the continuation
tokens with their penalties, found with the Z-algorithm on the reversed history,
src/sampler.zig:104-187), and with DRY on also lists the distinct tokens among the last 64 for
the repetition penalty (src/sampler.zig:91-100).  The repetition penalty alone works from a window
of each request's last 64 tokens kept on the device: the prompt's end is sent once, every sampled
token is appended by a kernel, and the host has nothing to send or to wait for in a step.

Random numbers are counter based: the uniforms of a draw depend only on (seed, request index,
number of tokens the request has sampled so far), never on which other requests share the batch.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch

from .. import kernels

REPEAT_LAST_N = 64          # src/sampler.zig:30
MAX_HISTORY = 4096          # src/sampler.zig:31
MAX_PENALIZED = 128         # src/sampler.zig:159


@dataclass
class SamplingParams:
    temp: float = 0.8
    top_k: int = 40
    top_p: float = 0.95
    min_p: float = 0.05
    repeat_penalty: float = 1.0
    seed: int = 0
    dry_multiplier: float = 0.0
    dry_base: float = 1.75
    dry_allowed_length: int = 2
    dry_range: int = 1024
    xtc_probability: float = 0.0
    xtc_threshold: float = 0.1
    xtc_min_keep: int = 1

    def validate(self) -> None:
        if self.top_k < 0:
            raise ValueError(f"top_k {self.top_k} must be >= 0")
        if not 0.0 < self.top_p:
            raise ValueError(f"top_p {self.top_p} must be positive")
        if not 0.0 <= self.min_p <= 1.0:
            raise ValueError(f"min_p {self.min_p} must lie in [0, 1]")
        if self.repeat_penalty <= 0:
            raise ValueError(f"repeat_penalty {self.repeat_penalty} must be positive")

    @property
    def greedy(self) -> bool:
        return self.temp <= 0                                        # src/sampler.zig:193


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & 0xFFFFFFFFFFFFFFFF
    return x ^ (x >> 31)


def uniform(seed: int, request: int, draw: int, stream: int) -> float:
    """A float32 in [0, 1) that depends only on its four arguments."""
    h = _splitmix64(seed & 0xFFFFFFFFFFFFFFFF)
    h = _splitmix64(h ^ (request & 0xFFFFFFFF))
    h = _splitmix64(h ^ (draw & 0xFFFFFFFF))
    h = _splitmix64(h ^ stream)
    return float(np.float32((h >> 40) / float(1 << 24)))


def dry_penalties(history: Sequence[int], p: SamplingParams, breakers: Sequence[int] = ()) -> dict[int, float]:
    """token -> penalty of the DRY sampler for the next token after `history`
    (src/sampler.zig:104-187): for every earlier place where the text's ending repeats for at
    least `dry_allowed_length` tokens, the token that followed there is penalised by
    multiplier * base^(repeat length - allowed length)."""
    if p.dry_multiplier == 0.0 or p.dry_base < 1.0 or p.dry_range == 0:
        return {}
    hist = list(history)[-MAX_HISTORY:]
    L = min(len(hist), p.dry_range, MAX_HISTORY)
    if L <= p.dry_allowed_length:
        return {}
    R = hist[::-1][:L]                                   # R[k] = k-th token from the end
    bset = set(breakers)
    rep_limit = L
    for k in range(L):
        if R[k] in bset:
            rep_limit = k
            break
    if rep_limit < p.dry_allowed_length:
        return {}
    z = [0] * L
    l = r = 0
    for i in range(1, L):
        z[i] = min(r - i + 1, z[i - l]) if i <= r else 0
        max_z = min(L - i, rep_limit)
        while z[i] < max_z and R[z[i]] == R[i + z[i]]:
            z[i] += 1
        if i + z[i] > 0 and i + z[i] - 1 > r:
            l, r = i, i + z[i] - 1
    lens: dict[int, int] = {}
    for k in range(1, L):
        if z[k] >= p.dry_allowed_length:
            tok = R[k - 1]
            if tok in bset:
                continue
            if tok in lens:
                lens[tok] = max(lens[tok], z[k])
            elif len(lens) < MAX_PENALIZED:
                lens[tok] = z[k]
    max_exp = 88.0 / math.log(p.dry_base) if p.dry_base > 1.0001 else 100.0
    return {t: p.dry_multiplier * p.dry_base ** min(float(n - p.dry_allowed_length), max_exp) for t, n in lens.items()}


def recent_distinct(history: Sequence[int]) -> list[int]:
    """The distinct tokens among the last 64, each once (src/sampler.zig:91-100)."""
    return list(dict.fromkeys(list(history)[-REPEAT_LAST_N:]))


class Sampler:
    """One sampler for the requests of a generation call; request `r` has its own history and
    its own stream of random numbers."""

    def __init__(self, params: SamplingParams, vocab_size: int, n_requests: int, device="cuda",
                 breakers: Sequence[int] = ()):
        params.validate()
        self.p, self.vocab, self.device = params, vocab_size, device
        self.history: list[list[int]] = [[] for _ in range(n_requests)]
        self.draws = [0] * n_requests
        self.breakers = tuple(breakers)
        # the device's copy of `draws`, advanced by the sampling kernel itself, and the rows' request
        # numbers as last sent: a step sends nothing unless the batch has changed
        self._draws_dev: Optional[torch.Tensor] = None
        self._rows: Optional[tuple] = None
        self._rows_dev: Optional[torch.Tensor] = None
        self._rows_pinned: Optional[torch.Tensor] = None
        # the device's window of each request's last tokens (a ring) for the repetition penalty, how
        # many tokens each request has had, and which requests' prompts have been sent
        self._recent: Optional[torch.Tensor] = None
        self._seen: Optional[torch.Tensor] = None
        self._sent = [False] * n_requests

    @property
    def needs_history(self) -> bool:
        """Whether sampling a request's next token needs its earlier tokens on the host (the DRY
        penalty does); if not, a step may be launched before the host has read the previous
        step's tokens."""
        return self.p.dry_multiplier != 0.0

    @property
    def plain_greedy(self) -> bool:
        """Greedy with no penalty: the token is the arg-max of the logits as the model left them."""
        return self.p.greedy and self.p.repeat_penalty == 1.0 and self.p.dry_multiplier == 0.0

    @property
    def _window_on_device(self) -> bool:
        return self.p.repeat_penalty != 1.0 and self.p.dry_multiplier == 0.0

    def accept(self, request: int, tokens: Sequence[int]) -> None:
        """Records tokens that entered the context, prompt or generated (src/sampler.zig:84-89)."""
        h = self.history[request]
        h.extend(int(t) for t in tokens)
        if len(h) > 2 * MAX_HISTORY:
            del h[:-MAX_HISTORY]

    def _penalties(self, logits: torch.Tensor, requests: Sequence[int]) -> None:
        p = self.p
        use_rep = p.repeat_penalty != 1.0
        use_dry = p.dry_multiplier != 0.0
        if not (use_rep or use_dry):
            return
        n = len(requests)
        rep = dry_t = dry_p = None
        if use_rep:
            a = np.full((n, REPEAT_LAST_N), -1, dtype=np.int32)
            for i, r in enumerate(requests):
                d = recent_distinct(self.history[r])
                a[i, :len(d)] = d
            rep = torch.from_numpy(a).to(self.device)
        if use_dry:
            t = np.full((n, MAX_PENALIZED), -1, dtype=np.int32)
            v = np.zeros((n, MAX_PENALIZED), dtype=np.float32)
            for i, r in enumerate(requests):
                pen = dry_penalties(self.history[r], p, self.breakers)
                for j, (tok, val) in enumerate(pen.items()):
                    t[i, j], v[i, j] = tok, val
            dry_t, dry_p = torch.from_numpy(t).to(self.device), torch.from_numpy(v).to(self.device)
        kernels.apply_penalties(logits, rep, p.repeat_penalty, dry_t, dry_p)

    def _rows_on_device(self, requests: Sequence[int]) -> torch.Tensor:
        """The rows' request numbers as an int32 tensor; sent only when the batch has changed."""
        rows = tuple(int(r) for r in requests)
        if len(set(rows)) != len(rows):
            raise ValueError("a request appears in two rows of one sampling step")
        if rows != self._rows:
            self._rows_pinned = torch.tensor(rows, dtype=torch.int32).pin_memory()
            self._rows_dev = self._rows_pinned.to(self.device, non_blocking=True)
            self._rows = rows
        return self._rows_dev

    def _send_windows(self, requests: Sequence[int]) -> None:
        """The end of the history (the prompt) of every request that samples for the first time."""
        n_win = kernels.recent_window()
        if self._recent is None:
            self._recent = torch.full((len(self.history), n_win), -1, dtype=torch.int32, device=self.device)
            self._seen = torch.zeros(len(self.history), dtype=torch.int32, device=self.device)
        new = [r for r in requests if not self._sent[r]]
        if not new:
            return
        win = np.full((len(new), n_win), -1, dtype=np.int32)
        cnt = np.zeros(len(new), dtype=np.int32)
        for i, r in enumerate(new):
            tail = self.history[r][-n_win:]
            win[i, :len(tail)] = tail
            cnt[i] = len(tail)
            self._sent[r] = True
        where = torch.tensor(new, dtype=torch.int64).pin_memory().to(self.device, non_blocking=True)
        self._recent.index_copy_(0, where, torch.from_numpy(win).pin_memory().to(self.device, non_blocking=True))
        self._seen.index_copy_(0, where, torch.from_numpy(cnt).pin_memory().to(self.device, non_blocking=True))

    def sample(self, logits: torch.Tensor, requests: Sequence[int]) -> torch.Tensor:
        """One token per row of float32 logits [n, V] (row i belongs to requests[i]); int32 on the
        device.  `logits` is edited in place by the penalties, as in the reference."""
        rows_dev = None
        if self._window_on_device:
            rows_dev = self._rows_on_device(requests)
            self._send_windows(requests)
            kernels.penalize_recent(logits, self._recent, self._seen, rows_dev, self.p.repeat_penalty)
        else:
            self._penalties(logits, requests)
        if self.p.greedy:
            tokens = kernels.argmax(logits)
        else:
            # The draw's uniforms are uniform(seed, request, draws[request], 0 and 1), computed by the
            # kernel from its own count of the request's draws: nothing is copied to the device in a
            # step whose rows are those of the step before, so the step can be queued behind the one
            # that runs.
            if self._draws_dev is None:
                self._draws_dev = torch.zeros(len(self.draws), dtype=torch.int32, device=self.device)
            rows_dev = self._rows_on_device(requests)
            for r in requests:
                self.draws[r] += 1
            tokens = kernels.sample(logits, None, self.p.temp, self.p.top_k, self.p.top_p, self.p.min_p,
                                    self.p.xtc_probability, self.p.xtc_threshold, self.p.xtc_min_keep, seed=self.p.seed,
                                    req_ids=rows_dev, draws=self._draws_dev)
        if self._window_on_device:
            kernels.recent_append(tokens, self._recent, self._seen, rows_dev)
        return tokens
