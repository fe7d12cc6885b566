"""The step function and the engine that owns a model's cache.

The reference's step is `State.forwardN(tokens, n_logits)`: embed, run every layer over the
given tokens from the cache, advance the position, and return logits of the last `n_logits`
rows; long prompts are cut into chunks (src/model.zig:2519-2542, 2347-2516).  `Engine.step` is
that function for a batch: for each sequence its next tokens (whole prompts in a batch's first
step, one token each afterwards), run as one packed batch from the cache, logits returned at
the wanted places only.  Nothing but the given tokens is computed, and padding does not exist:
sequences of unequal length are packed, not padded.
"""
from __future__ import annotations

import threading
from collections import OrderedDict
from typing import Optional, Sequence

import numpy as np
import torch

from .. import kernels
from ..cache.manager import CacheManager
from ..models.model import Model
from .context import CallContext, StepContext, batch_layout, pack_batch


class StepError(RuntimeError):
    """The device reported a fault of the step's inputs (a token id outside the vocabulary, a
    position without a page)."""


_STATUS_TEXT = {1: "a token id lies outside the vocabulary", 2: "a token's position has no cache page",
                11: "a tensor-core contraction gave up waiting for a free pipeline stage",
                12: "a tensor-core contraction gave up waiting for its operand tiles",
                13: "a tensor-core contraction gave up waiting for its accumulator",
                14: "the tcgen05 prompt attention gave up waiting for a free K/V stage",
                15: "the tcgen05 prompt attention gave up waiting for its query or K/V tiles",
                16: "the tcgen05 prompt attention gave up waiting for the probabilities",
                17: "the tcgen05 prompt attention gave up waiting for the scores",
                18: "the tcgen05 prompt attention gave up waiting for P V"}


class _DecodeBatch:
    """What the recorded single-token steps of one batch size share: the static buffer that holds
    the batch's description, the static logits they write, and what the parts memoised about a
    batch of this shape.

    The description reaches the static device buffer through a small ring of pinned host
    buffers: a buffer is rewritten only after the copy that last read it has run, so a host
    that runs several steps ahead of the device cannot change a step's input under it."""

    RING = 4
    OUT_RING = 4        # results the host may still have to read while later steps run (it reads one step late)

    def __init__(self, n_seqs: int, vocab: int, device):
        words = batch_layout(n_seqs, n_seqs)["_total"][0]
        self.meta_dev = torch.zeros(words, dtype=torch.int32, device=device)
        self.logits = torch.empty((n_seqs, vocab), dtype=torch.float32, device=device)
        # every step ends with the arg-max of its logits: the n tokens and, behind them, the status word
        self.greedy = torch.zeros(n_seqs + 1, dtype=torch.int32, device=device)
        # ... and writes both into slot (step % OUT_RING) of a ring as well, the device counting the steps in
        # `ring_pos` as the host does in `steps`: the host fetches a step's slot on a stream of its own
        # while the next step runs.  The same copy queued between two recorded steps cost 40 us a step.
        self.ring = torch.zeros((self.OUT_RING, n_seqs + 1), dtype=torch.int32, device=device)
        self.host_ring = torch.zeros((self.OUT_RING, n_seqs + 1), dtype=torch.int32).pin_memory()
        self.ring_pos = torch.zeros(1, dtype=torch.int32, device=device)
        self.steps = 0
        self.n_seqs = n_seqs
        self._tail = batch_layout(n_seqs, n_seqs)["tok_seq"][0]      # where the description goes on behind the token ids
        self._hosts = [torch.zeros(words, dtype=torch.int32).pin_memory() for _ in range(self.RING)]
        self._copied = [None] * self.RING
        self._next = 0
        self.memo: dict = {}
        self.warmed = False         # one step of this batch size has run outside a recording (it loads the kernels)

    def upload(self, words, dev_tokens: Optional[torch.Tensor] = None) -> None:
        """Copies the packed batch description to the static device buffer; `dev_tokens`, if
        given, then replaces its token ids (the first array of the description) on the device.
        If `dev_tokens` are this batch's own greedy tokens of the step before, they already lie in
        the token slots (the step's last kernel put them there): only the rest is copied."""
        i = self._next
        self._next = (i + 1) % self.RING
        if self._copied[i] is not None:
            self._copied[i].synchronize()
        self._hosts[i].numpy()[:] = words
        in_place = (dev_tokens is not None and dev_tokens.data_ptr() == self.greedy.data_ptr()
                    and dev_tokens.numel() == self.n_seqs)
        if in_place:
            self.meta_dev[self._tail:].copy_(self._hosts[i][self._tail:], non_blocking=True)
        else:
            self.meta_dev.copy_(self._hosts[i], non_blocking=True)
        if self._copied[i] is None:
            self._copied[i] = torch.cuda.Event()
        self._copied[i].record()
        if dev_tokens is not None and not in_place:
            self.meta_dev[:dev_tokens.numel()].copy_(dev_tokens)


class _PendingTokens:
    def __init__(self, engine, host, done):
        self.engine, self.host, self.done = engine, host, done

    def wait(self) -> list[int]:
        self.done.synchronize()
        both = self.host.tolist()
        if both[-1]:
            self.engine.status.zero_()
            raise StepError(_STATUS_TEXT.get(both[-1], f"device status {both[-1]}"))
        return both[:-1]


class Engine:
    MAX_GRAPHS = 48         # recorded single-token steps kept; the least recently used one goes first

    def __init__(self, model: Model, max_batch: int = 64, max_seq_len: Optional[int] = None,
                 max_tokens: Optional[int] = None, page_size: int = 64, max_step_tokens: int = 8192,
                 use_graphs: bool = True, lookahead: bool = True):
        """max_batch: slots (sequences alive at once).  max_seq_len: longest sequence, default
        the model's max_position_embeddings.  max_tokens: tokens the cache holds in total, each
        sequence rounded up to whole pages; default max_batch * max_seq_len.  max_step_tokens:
        a step with more tokens runs as several packed chunks.  use_graphs: replay single-token
        steps of `decode` from CUDA graphs (only if every mixer of the model is `capture_safe`).
        lookahead: `generate` launches a step before the host has read the previous step's tokens
        whenever the sampler allows it."""
        kernels.require_cuda()
        if model.device is None:
            raise ValueError("the model has no weights loaded")
        self.model = model
        self.dtype, self.device = model.dtype, model.device
        cfg = model.config
        self.max_seq_len = int(max_seq_len or cfg.max_position_embeddings)
        if max_tokens is None:
            max_tokens = max_batch * (-(-self.max_seq_len // page_size) * page_size)
        self.max_step_tokens = max(1, int(max_step_tokens))
        mixers = [layer.mixer for layer in model.layers]
        for m in mixers:
            m.check(self.dtype, page_size)       # sizes no kernel takes are refused here, not in the first step
        self.cache = CacheManager(model.cache_specs(), max_batch, int(max_tokens), self.max_seq_len, page_size,
                                  self.dtype, self.device)
        self.calls = [CallContext(c, call.layer, self.cache.kv_view(c), self.cache.writes_kv(c),
                                  self.cache.state_view(c)) for c, call in enumerate(model.schedule)]
        self.status = kernels.status_word(self.device)      # one status word per device, shared by all kernels
        self.sm_count = kernels.sm_count(self.device)
        self.vocab_size = cfg.vocab_size
        self.use_graphs = bool(use_graphs) and all(getattr(m, "capture_safe", False) for m in mixers)
        self.supports_device_tokens = bool(lookahead)    # GenerationLoop asks this before running ahead
        self._key_mixers = list({id(m): m for m in mixers}.values())
        self._decode_batches: dict[int, _DecodeBatch] = {}
        self._graphs: "OrderedDict[tuple, torch.cuda.CUDAGraph]" = OrderedDict()
        self._graph_pool = torch.cuda.graph_pool_handle() if self.use_graphs else None
        self.graph_captures = 0         # steps that were recorded instead of replayed, since the engine was built
        self._host_ring, self._host_next = None, 0      # pinned buffers the sampled tokens are read into
        self._copy_stream = None                        # the stream on which recorded steps' tokens are fetched
        self.interrupt = threading.Event()   # set it (from a signal handler, another thread, a callback) to end `generate`
        self.stats = None

    # ------------------------------------------------------------------ sequences
    def start(self, n: int) -> list[int]:
        """Slots for `n` new sequences that start together."""
        return self.cache.alloc_slots(n)

    def finish(self, slots: Sequence[int]) -> None:
        """Gives the slots and all they hold back to the cache."""
        self.cache.free_slots(slots)

    def length(self, slot: int) -> int:
        return int(self.cache.lengths[slot])

    # ------------------------------------------------------------------ the step
    def step(self, slots: Sequence[int], token_lists: Sequence[Sequence[int]],
             want: Optional[Sequence[Sequence[int]]] = None, check: bool = True) -> Optional[torch.Tensor]:
        """Feeds `token_lists[i]` to the sequence in `slots[i]` and returns float32 logits
        [wanted, vocab] on the device, in the order of the sequences and of `want[i]` (indices
        into token_lists[i]; default: the last token of each sequence).  Returns None if nothing
        is wanted.  Raises ContextFull / OutOfPages before anything is changed."""
        if len(slots) != len(token_lists):
            raise ValueError("one token list per slot")
        if len(set(slots)) != len(slots):
            raise ValueError("a slot is named twice in one step")
        lens = [len(t) for t in token_lists]
        if any(l == 0 for l in lens):
            raise ValueError("every sequence of a step brings at least one token")
        if want is None:
            want = [[l - 1] for l in lens]
        for w, l in zip(want, lens):
            if any(not 0 <= i < l for i in w):
                raise ValueError(f"wanted position outside the {l} tokens of its sequence")
        self.cache.reserve(slots, lens)
        self.cache.sync()

        pieces = []
        total = sum(lens)
        if total <= self.max_step_tokens:
            out = self._run(slots, [int(self.cache.lengths[s]) for s in slots], token_lists, want)
            if out is not None:
                pieces.append((None, out))
            order = None
        else:
            order = self._run_chunked(slots, token_lists, want, pieces)
        self.cache.advance(slots, lens)
        if check:
            self.check_status()
        if not pieces:
            return None
        if order is None:
            return pieces[0][1]
        logits = torch.cat([p[1] for p in pieces], dim=0)
        # chunks produce wanted rows chunk by chunk; put them into request order
        keys = [k for p in pieces for k in p[0]]
        perm = sorted(range(len(keys)), key=lambda i: keys[i])
        return logits[torch.tensor(perm, device=logits.device)]

    def _run_chunked(self, slots, token_lists, want, pieces):
        """Runs a large step as packed chunks of at most max_step_tokens tokens.  Every chunk is
        itself a step that continues each sequence where the previous chunk left it, so the cut
        shows only as rounding."""
        done = [0] * len(slots)
        base = [int(self.cache.lengths[s]) for s in slots]
        lens = [len(t) for t in token_lists]
        while any(d < l for d, l in zip(done, lens)):
            room = self.max_step_tokens
            sub_idx, sub_tokens, sub_want, sub_keys = [], [], [], []
            for i, (d, l) in enumerate(zip(done, lens)):
                if d >= l or room == 0:
                    continue
                take = min(l - d, room)
                room -= take
                sub_idx.append(i)
                sub_tokens.append(token_lists[i][d:d + take])
                w = [(j, p) for j, p in enumerate(want[i]) if d <= p < d + take]
                sub_want.append([p - d for _, p in w])
                sub_keys.extend((i, j) for j, _ in w)
            out = self._run([slots[i] for i in sub_idx], [base[i] + done[i] for i in sub_idx], sub_tokens, sub_want)
            if out is not None:
                pieces.append((sub_keys, out))
            for i, t in zip(sub_idx, sub_tokens):
                done[i] += len(t)
        return True

    def _run(self, slots, starts, token_lists, want) -> Optional[torch.Tensor]:
        lens = [len(t) for t in token_lists]
        n, B = sum(lens), len(slots)
        host = pack_batch(slots, starts, token_lists)
        buf = torch.from_numpy(host).pin_memory().to(self.device, non_blocking=True)
        max_kv = max(s + l for s, l in zip(starts, lens))
        ctx = StepContext(self.dtype, self.device, self.status, buf, n, B, lens, max_kv, sm_count=self.sm_count)
        cu = np.concatenate([[0], np.cumsum(lens)])
        rows = [int(cu[b]) + int(i) for b, w in enumerate(want) for i in w]
        if rows == list(range(n)):      # every row in order (a step of single tokens): no gather before the head
            return self.model.forward(ctx, self.calls, None, want_all=True)
        want_rows = torch.tensor(rows, dtype=torch.int32).pin_memory().to(self.device, non_blocking=True) if rows else None
        return self.model.forward(ctx, self.calls, want_rows)

    # ------------------------------------------------------------------ single-token steps

    def decode(self, slots: Sequence[int], tokens, check: bool = False) -> torch.Tensor:
        """One token for each sequence, logits [len(slots), vocab] for all of them.  The same
        computation as `step(slots, [[t] for t in tokens])`, replayed from a CUDA graph: a step of
        single tokens is some hundred small kernels, and launching them one by one costs more than
        running them.  A recording serves a batch size and whatever else the mixers bake into
        their launches (`Mixer.launch_key`: for attention the layout of key chunks, which changes
        when the longest sequence outgrows 512, 768, 1024, 1536, ... tokens).  The first step of a
        batch size runs unrecorded (which also loads every kernel); later ones are recorded at
        their first use and replayed from then on.  The returned tensor is a static buffer of
        the batch size: use it before the next call.  `tokens` is a sequence of ints, or an int32
        tensor [len(slots)] on the device (a sampler's output): the step then starts without the
        host having seen them."""
        on_device = isinstance(tokens, torch.Tensor)
        if not self.use_graphs:
            host = tokens.cpu().tolist() if on_device else tokens
            return self.step(slots, [[int(t)] for t in host], check=check)
        B = len(slots)
        if B != len(tokens) or len(set(slots)) != B:
            raise ValueError("one token per distinct slot")
        dev_tokens = None
        if on_device:
            if tokens.dtype != torch.int32 or not tokens.is_cuda or tokens.dim() != 1:
                raise ValueError("device tokens must be a one-dimensional int32 CUDA tensor")
            dev_tokens, tokens = tokens, [0] * B
        ones = [1] * B
        self.cache.reserve(slots, ones)
        self.cache.sync()
        starts = [int(self.cache.lengths[s]) for s in slots]
        words = pack_batch(slots, starts, [[int(t)] for t in tokens])
        batch = self._decode_batch(B)
        batch.upload(words, dev_tokens)
        logits = self._decode_graph(batch, B, max(starts) + 1)
        self.cache.advance(slots, ones)
        if check:
            self.check_status()
        return logits

    def _decode_batch(self, B: int) -> _DecodeBatch:
        batch = self._decode_batches.get(B)
        if batch is None:
            batch = self._decode_batches[B] = _DecodeBatch(B, self.vocab_size, self.device)
        return batch

    def decode_key(self, n_seqs: int, longest: int) -> tuple:
        """What a recorded single-token step is good for: the batch size and every mixer's launch key."""
        return (n_seqs, *(m.launch_key(n_seqs, longest) for m in self._key_mixers))

    def _forward_single_tokens(self, ctx, batch: _DecodeBatch) -> None:
        """The step's kernels: the model, then the arg-max of every row of logits.  The arg-max goes to
        `batch.greedy` (with the status word behind it: one small copy brings both to the host) and into
        the token slots of the batch description, where the next step of the same batch finds it."""
        self.model.forward(ctx, self.calls, None, want_all=True, out=batch.logits)
        kernels.argmax(batch.logits, out=batch.greedy, feed=batch.meta_dev[:batch.n_seqs], status=self.status,
                       ring=batch.ring, ring_pos=batch.ring_pos)

    def greedy_tokens(self, logits: torch.Tensor) -> Optional[torch.Tensor]:
        """If `logits` are what the last `decode` returned from a recorded (or warm-up) step: the int32
        tensor [n + 1] with the arg-max token of every row and the status word behind them, computed by
        the step itself.  Feeding its first n elements to the next `decode` of the same slots costs no
        copy on the device.  None for logits of any other origin."""
        for batch in self._decode_batches.values():
            if batch.logits is logits:
                return batch.greedy
        return None

    def read_greedy_async(self, logits: torch.Tensor):
        """For logits that the last `decode` returned: an object whose `wait()` gives the arg-max tokens
        of that step on the host (and raises on a device status).  The step's last kernel left them in a
        slot of the batch's ring; they are copied from there on a stream of their own, so the steps that
        follow on the main stream do not wait for the copy.  None for logits of any other origin."""
        for batch in self._decode_batches.values():
            if batch.logits is logits:
                slot = (batch.steps - 1) % batch.OUT_RING
                ran = torch.cuda.Event()
                ran.record()
                if self._copy_stream is None:
                    self._copy_stream = torch.cuda.Stream(device=self.device)
                done = torch.cuda.Event()
                with torch.cuda.stream(self._copy_stream):
                    self._copy_stream.wait_event(ran)
                    batch.host_ring[slot].copy_(batch.ring[slot], non_blocking=True)
                    done.record()
                return _PendingTokens(self, batch.host_ring[slot], done)
        return None

    def _decode_graph(self, batch: _DecodeBatch, B: int, longest: int) -> torch.Tensor:
        ctx = StepContext(self.dtype, self.device, self.status, batch.meta_dev, B, B, [1] * B, longest,
                          memo=batch.memo, sm_count=self.sm_count)
        batch.steps += 1            # the kernels run once below (a recording in between runs nothing)
        if not batch.warmed:
            batch.warmed = True
            self._forward_single_tokens(ctx, batch)
            return batch.logits
        key = self.decode_key(B, longest)
        graph = self._graphs.get(key)
        if graph is None:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, pool=self._graph_pool):
                self._forward_single_tokens(ctx, batch)
            self._graphs[key] = graph
            self.graph_captures += 1
            while len(self._graphs) > self.MAX_GRAPHS:
                self._graphs.popitem(last=False)
        else:
            self._graphs.move_to_end(key)
        graph.replay()
        return batch.logits

    def prepare_decode(self, n_seqs: int, first: int, last: int) -> None:
        """Records, ahead of time, the single-token steps that `n_seqs` sequences need while their
        longest grows from `first` to `last` tokens (one per launch key on the way), so that none of
        those steps pays for a recording.  Needs one unrecorded step of that batch size to have run."""
        if not self.use_graphs:
            return
        batch = self._decode_batch(n_seqs)
        if not batch.warmed:
            raise RuntimeError(f"no single-token step of {n_seqs} sequences has run yet")
        longest = max(first, last)
        length = max(1, first)
        while True:
            key = self.decode_key(n_seqs, length)
            if key not in self._graphs:
                ctx = StepContext(self.dtype, self.device, self.status, batch.meta_dev, n_seqs, n_seqs, [1] * n_seqs,
                                  length, memo=batch.memo, sm_count=self.sm_count)
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, pool=self._graph_pool):
                    self._forward_single_tokens(ctx, batch)
                self._graphs[key] = graph
                self.graph_captures += 1
            if length >= longest:
                break
            # the next length at which some mixer's key may change: keys are functions of coarse
            # buckets, so doubling steps with a linear probe in between find every one of them
            nxt = length + 1
            while nxt < longest and self.decode_key(n_seqs, nxt) == key:
                nxt = min(longest, nxt + max(1, nxt // 8))
            length = nxt
        while len(self._graphs) > self.MAX_GRAPHS:
            self._graphs.popitem(last=False)

    # ------------------------------------------------------------------ generation
    def prefill(self, slots, prompts) -> torch.Tensor:
        return self.step(slots, prompts, check=False)

    def read_tokens(self, tokens: torch.Tensor) -> list[int]:
        """Sampled tokens on the host; this is the step's synchronisation point, so the device's
        status word is read with them."""
        both = torch.cat([tokens.to(torch.int32), self.status]).cpu().tolist()
        if both[-1]:
            self.status.zero_()
            raise StepError(_STATUS_TEXT.get(both[-1], f"device status {both[-1]}"))
        return both[:-1]

    def read_tokens_async(self, tokens: torch.Tensor, with_status: bool = False):
        """Starts copying sampled tokens (and the status word) to the host; the returned object's
        `wait()` gives them once the copy has run, whatever was launched after it.  `with_status`: the
        tensor's last element already is the status word (`greedy_tokens`).  The copy runs on a stream of
        its own behind what has been launched so far: queued on the main stream it would stand between
        two steps and cost them 40 us.  `tokens` must not be written again before `wait()` returns."""
        ring = self._host_ring
        n = tokens.numel() + (0 if with_status else 1)
        if ring is None or ring[0].numel() < n:
            ring = self._host_ring = [torch.empty(max(n, self.cache.max_slots + 1), dtype=torch.int32,
                                                  pin_memory=True) for _ in range(8)]
        self._host_next = (self._host_next + 1) % len(ring)
        host = ring[self._host_next][:n]     # at most two reads are under way at a time
        ran = torch.cuda.Event()
        ran.record()
        if self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream(device=self.device)
        done = torch.cuda.Event()
        with torch.cuda.stream(self._copy_stream):
            self._copy_stream.wait_event(ran)
            m = tokens.numel()
            host[:m].copy_(tokens if tokens.dtype == torch.int32 else tokens.to(torch.int32), non_blocking=True)
            if not with_status:
                host[m:].copy_(self.status, non_blocking=True)
            done.record()
        pending = _PendingTokens(self, host, done)
        pending.source = tokens          # alive until the copy has run
        return pending

    def generate(self, prompts, max_new_tokens: int = 256, sampling=None, stop_ids=None, on_step=None,
                 **sampling_options):
        """Generates for every prompt (a list of token ids each); returns a GenerationResult per
        prompt, in order.  `sampling` is a SamplingParams, or give its fields as keyword
        arguments (temp, top_k, top_p, min_p, repeat_penalty, seed, ...; `temperature` is
        accepted for `temp`).  stop_ids default to the configuration's eos token ids.
        Setting `self.interrupt` while it runs ends it at the next step: requests come back with
        the tokens they have and the reason "interrupted" (the flag is cleared when a call starts)."""
        from ..sampling.sampler import Sampler, SamplingParams
        from .generate import GenerationLoop

        if sampling is None:
            if "temperature" in sampling_options:
                sampling_options["temp"] = sampling_options.pop("temperature")
            sampling = SamplingParams(**sampling_options)
        elif sampling_options:
            raise ValueError("give either `sampling` or its fields, not both")
        if stop_ids is None:
            stop_ids = self.model.config.eos_token_ids
        sampler = Sampler(sampling, self.vocab_size, len(prompts), self.device)
        self.interrupt.clear()
        loop = GenerationLoop(self, self.cache.max_slots, self.cache.num_pages * self.cache.page_size,
                              self.max_seq_len, self.cache.page_size, interrupt=self.interrupt)
        results = loop.run(prompts, sampler, max_new_tokens, stop_ids, on_step)
        self.stats = loop.stats
        return results

    def check_status(self) -> None:
        """Synchronises and raises StepError if a kernel flagged its inputs."""
        code = int(self.status.item())
        if code:
            self.status.zero_()
            raise StepError(_STATUS_TEXT.get(code, f"device status {code}"))
