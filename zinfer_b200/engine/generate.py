"""The generation loop above the step function.

The reference's loop (src/gen.zig:434-537): feed the prompt whole, sample, then forward one
token and sample again until an end-of-generation token, `n` tokens or a full context; the
end token is returned but neither emitted nor fed (src/gen.zig:461-464, 532-535).  Here the
same loop runs for batches of requests with unequal prompts: a batch starts together (every
prompt in one step), then each live request goes on by one token a step; a request that stops
leaves the batch, the others go on; when the batch has ended its slots go back to the cache and
the next batch starts, until every request is served.

The reference polls an atomic `interrupted` flag once per token and ends the generation there,
keeping what it has (src/gen.zig:476-479; the command line sets it on Ctrl-C, src/main.zig:297-299).
Here `interrupt` is a `threading.Event`: once it is set the loop ends every running request with
the reason "interrupted" and the tokens it has so far, starts no further batch (requests that
never ran come back empty with the same reason), and gives the slots back.

The loop talks to a backend with five methods (`start`, `finish`, `prefill`, `decode`,
`read_tokens`), so its decisions can be tested without a GPU.
"""
from __future__ import annotations

import threading
import time

import torch
from dataclasses import dataclass, field
from typing import Callable, Optional, Sequence


@dataclass
class GenerationResult:
    tokens: list[int]
    # "stop" (a stop token was sampled), "length" (max_new_tokens), "context" (cache full),
    # "interrupted" (the caller asked the loop to end: what was generated so far is returned)
    finish_reason: str
    prompt_tokens: int
    stop_token: Optional[int] = None


@dataclass
class Stats:
    """Counters of a generation call (src/gen.zig:33-42)."""

    n_prompt: int = 0
    n_gen: int = 0
    t_prompt_s: float = 0.0
    t_gen_s: float = 0.0
    n_batches: int = 0
    n_decode_steps: int = 0

    def report(self) -> str:
        """One line in the manner of the reference's report (src/gen.zig:632-656)."""
        pp = self.n_prompt / self.t_prompt_s if self.t_prompt_s > 0 else 0.0
        tg = self.n_gen / self.t_gen_s if self.t_gen_s > 0 else 0.0
        return (f"prompt: {self.n_prompt} tokens, {pp:.1f} tok/s | gen: {self.n_gen} tokens, {tg:.1f} tok/s | "
                f"{self.n_batches} batches, {self.n_decode_steps} decode steps")


def round_up(n: int, m: int) -> int:
    return -(-n // m) * m


def token_budget(prompt_len: int, max_new_tokens: int, max_seq_len: int) -> tuple[int, str]:
    """How many tokens a request may generate and why it ends there.  A sampled token is fed only
    if another one is to follow, so a context of C tokens allows C - P + 1 new ones
    (src/gen.zig:475: `while n_run < max_new and pos < ctx`)."""
    by_context = max_seq_len - prompt_len + 1
    if max_new_tokens <= 0 or by_context < max_new_tokens:       # <= 0 means unlimited, src/main.zig:157-163
        return by_context, "context"
    return max_new_tokens, "length"


def plan_batch(pending: Sequence[int], prompt_lens: Sequence[int], budgets: Sequence[int], max_batch: int,
               max_tokens: int, page_size: int) -> list[int]:
    """The requests of the next batch: in order, as many as there are slots and as the cache holds
    when every one of them runs to its budget (each rounded up to whole pages).  At least one."""
    batch, used = [], 0
    for r in pending:
        if len(batch) == max_batch:
            break
        need = round_up(prompt_lens[r] + max(budgets[r] - 1, 0), page_size)
        if batch and used + need > max_tokens:
            break
        batch.append(r)
        used += need
    return batch


class GenerationLoop:
    def __init__(self, backend, max_batch: int, max_tokens: int, max_seq_len: int, page_size: int,
                 interrupt: Optional[threading.Event] = None):
        self.backend = backend
        self.max_batch, self.max_tokens, self.max_seq_len, self.page_size = max_batch, max_tokens, max_seq_len, page_size
        self.interrupt = interrupt if interrupt is not None else threading.Event()
        self.stats = Stats()

    def _interrupted(self, active, out, results, lens) -> bool:
        """Polled once per step: ends the running requests with what they have."""
        if not self.interrupt.is_set():
            return False
        for r in active:
            if results[r] is None:
                results[r] = GenerationResult(out[r], "interrupted", lens[r])
        return True

    def run(self, prompts: Sequence[Sequence[int]], sampler, max_new_tokens: int = 256,
            stop_ids: Sequence[int] = (), on_step: Optional[Callable[[dict[int, int]], None]] = None
            ) -> list[GenerationResult]:
        stop = set(int(s) for s in stop_ids)
        n = len(prompts)
        for r, p in enumerate(prompts):
            if len(p) == 0:
                raise ValueError(f"request {r}: an empty prompt")
            if len(p) > self.max_seq_len:
                raise ValueError(f"request {r}: prompt of {len(p)} tokens exceeds the context of {self.max_seq_len}")
            if round_up(len(p), self.page_size) > self.max_tokens:
                raise ValueError(f"request {r}: prompt of {len(p)} tokens does not fit a cache of {self.max_tokens}")
        lens = [len(p) for p in prompts]
        budgets, reasons = [], []
        for l in lens:
            b, why = token_budget(l, max_new_tokens, self.max_seq_len)
            by_cache = self.max_tokens - l + 1                     # alone in the cache
            if by_cache < b:
                b, why = by_cache, "context"
            budgets.append(b)
            reasons.append(why)
        results: list[Optional[GenerationResult]] = [None] * n
        pending = list(range(n))
        be = self.backend
        while pending:
            if self.interrupt.is_set():
                for r in pending:
                    results[r] = GenerationResult([], "interrupted", lens[r])
                break
            batch = plan_batch(pending, lens, budgets, self.max_batch, self.max_tokens, self.page_size)
            pending = pending[len(batch):]
            self.stats.n_batches += 1
            slots = be.start(len(batch))
            try:
                slot_of = dict(zip(batch, slots))
                out = {r: [] for r in batch}
                for r in batch:
                    sampler.accept(r, prompts[r])
                t0 = time.perf_counter()
                logits = be.prefill([slot_of[r] for r in batch], [list(prompts[r]) for r in batch])
                toks_dev = sampler.sample(logits, batch)
                toks = be.read_tokens(toks_dev)
                self.stats.t_prompt_s += time.perf_counter() - t0
                self.stats.n_prompt += sum(lens[r] for r in batch)
                active = list(batch)
                t0 = time.perf_counter()
                if (getattr(be, "supports_device_tokens", False) and not getattr(sampler, "needs_history", True)
                        and isinstance(toks_dev, torch.Tensor)):
                    self._run_ahead(be, sampler, active, toks, toks_dev, slot_of, out, results, lens, budgets, reasons,
                                    stop, on_step)
                    self.stats.t_gen_s += time.perf_counter() - t0
                    continue
                while True:
                    live, feed, emitted = [], [], {}
                    for r, tok in zip(active, toks):
                        tok = int(tok)
                        if tok in stop:                      # returned, not emitted, not fed
                            results[r] = GenerationResult(out[r], "stop", lens[r], stop_token=tok)
                            continue
                        out[r].append(tok)
                        emitted[r] = tok
                        sampler.accept(r, [tok])
                        self.stats.n_gen += 1
                        if len(out[r]) >= budgets[r]:
                            results[r] = GenerationResult(out[r], reasons[r], lens[r])
                            continue
                        live.append(r)
                        feed.append(tok)
                    if on_step is not None and emitted:
                        on_step(emitted)
                    if not live or self._interrupted(live, out, results, lens):
                        break
                    logits = be.decode([slot_of[r] for r in live], feed)
                    toks = be.read_tokens(sampler.sample(logits, live))
                    self.stats.n_decode_steps += 1
                    active = live
                self.stats.t_gen_s += time.perf_counter() - t0
            finally:
                be.finish(slots)
        return results  # type: ignore[return-value]

    def _run_ahead(self, be, sampler, active, toks, toks_dev, slot_of, out, results, lens, budgets, reasons, stop,
                   on_step) -> None:
        """The decode loop with one step of lookahead: step n+1 is launched on the tokens that step
        n sampled while they are still on the device; the host reads them meanwhile and learns one
        step late that a request has stopped.  Such a request has then been fed one token too
        many, which nobody sees: its result ends at the stop token and its slot is freed with the
        batch.  The tokens, their order and the reasons are those of the plain loop; the sampler
        must not need the host's history of a request."""
        pending, keep = None, None       # the copy of `toks_dev` under way, and which of its rows are `active`
        # a backend whose steps end with the arg-max of their logits spares a greedy sampler its kernel
        greedy = getattr(be, "greedy_tokens", None) if getattr(sampler, "plain_greedy", False) else None
        while True:
            # Requests that go on unless the token they are about to receive is a stop token.
            # Their step is launched now, on the device's copy of those tokens; the host reads
            # the tokens while that step runs.
            rows = [i for i, r in enumerate(active) if len(out[r]) + 1 < budgets[r]]
            ahead = [active[i] for i in rows]
            nxt_pending = nxt_dev = None
            if ahead:
                feed = toks_dev if len(rows) == len(active) else toks_dev[torch.tensor(rows, device=toks_dev.device)]
                logits = be.decode([slot_of[r] for r in ahead], feed)
                packed = greedy(logits) if greedy is not None else None
                if packed is not None:      # the step computed its own arg-max; the status word lies behind it
                    nxt_dev = packed[:len(ahead)]
                    direct = getattr(be, "read_greedy_async", None)      # ... and may have written both to the host
                    nxt_pending = direct(logits) if direct is not None else None
                    if nxt_pending is None:
                        nxt_pending = be.read_tokens_async(packed, with_status=True)
                else:
                    nxt_dev = sampler.sample(logits, ahead)
                    nxt_pending = be.read_tokens_async(nxt_dev)
                self.stats.n_decode_steps += 1
            if pending is not None:
                got = pending.wait()
                toks = got if keep is None else [got[i] for i in keep]
            live, emitted = [], {}
            for r, tok in zip(active, toks):
                tok = int(tok)
                if tok in stop:
                    results[r] = GenerationResult(out[r], "stop", lens[r], stop_token=tok)
                    continue
                out[r].append(tok)
                emitted[r] = tok
                sampler.accept(r, [tok])
                self.stats.n_gen += 1
                if len(out[r]) >= budgets[r]:
                    results[r] = GenerationResult(out[r], reasons[r], lens[r])
                    continue
                live.append(r)
            if on_step is not None and emitted:
                on_step(emitted)
            if not live or self._interrupted(live, out, results, lens):
                if nxt_pending is not None:
                    nxt_pending.wait()      # nothing of the step that ran ahead is used
                return
            keep = None
            if live != ahead:                # some request stopped: its row of the step that ran ahead is dropped
                keep = [ahead.index(r) for r in live]
                nxt_dev = nxt_dev[torch.tensor(keep, device=nxt_dev.device)]
            active, toks_dev, pending = live, nxt_dev, nxt_pending
