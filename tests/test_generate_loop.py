"""The generation loop's decisions, with a scripted backend instead of a model: batches one
after another, unequal prompts, stop tokens neither emitted nor fed, requests that end earlier
leave the batch, budgets by length and by context, slots given back even on errors."""
import pytest

from zinfer_b200.engine.generate import GenerationLoop, plan_batch, token_budget


class Script:
    """Backend whose 'model' continues request r with script[r][k] as its k-th new token.  It
    identifies a request by its prompt's first token and checks everything the loop feeds."""

    def __init__(self, prompts, scripts, max_slots):
        self.prompts, self.scripts, self.max_slots = prompts, scripts, max_slots
        self.free = list(range(max_slots))
        self.seq = {}            # slot -> (request, tokens fed so far)
        self.log = []

    def start(self, n):
        assert n <= len(self.free), "more sequences started than slots"
        slots = [self.free.pop(0) for _ in range(n)]
        self.log.append(("start", tuple(slots)))
        return slots

    def finish(self, slots):
        for s in slots:
            assert s not in self.free
            self.seq.pop(s, None)
            self.free.append(s)
        self.log.append(("finish", tuple(slots)))

    def prefill(self, slots, prompts):
        for s, p in zip(slots, prompts):
            r = p[0]
            assert p == self.prompts[r] and s not in self.seq
            self.seq[s] = (r, list(p))
        self.log.append(("prefill", tuple(slots)))
        return [self._next(s) for s in slots]

    def decode(self, slots, tokens):
        for s, t in zip(slots, tokens):
            r, fed = self.seq[s]
            k = len(fed) - len(self.prompts[r])
            assert t == self.scripts[r][k], "the loop must feed exactly what was sampled"
            fed.append(t)
        self.log.append(("decode", tuple(slots)))
        return [self._next(s) for s in slots]

    def _next(self, s):
        r, fed = self.seq[s]
        return self.scripts[r][len(fed) - len(self.prompts[r])]

    def read_tokens(self, toks):
        return list(toks)


class PassThrough:
    def __init__(self):
        self.accepted = {}

    def accept(self, r, toks):
        self.accepted.setdefault(r, []).extend(toks)

    def sample(self, logits, requests):
        return logits


def run(prompts, scripts, max_batch=2, max_tokens=10_000, max_seq_len=1000, page=16, **kw):
    be = Script(prompts, scripts, max_batch)
    loop = GenerationLoop(be, max_batch, max_tokens, max_seq_len, page)
    smp = PassThrough()
    res = loop.run(prompts, smp, **kw)
    assert sorted(be.free) == list(range(max_batch)), "every slot is given back"
    return res, be, smp, loop


STOP = 99
PROMPTS = [[0, 5, 5], [1], [2, 7, 7, 7, 7], [3, 8], [4, 9, 9]]
SCRIPTS = [[10, 11, STOP, 12], [20, 21, 22, 23, 24, 25], [STOP], [30, 31, 32, 33, 34, 35], [40, STOP]]


def test_batches_stop_tokens_and_early_finishers():
    res, be, smp, loop = run(PROMPTS, SCRIPTS, max_batch=2, max_new_tokens=4, stop_ids=[STOP])
    assert [r.tokens for r in res] == [[10, 11], [20, 21, 22, 23], [], [30, 31, 32, 33], [40]]
    assert [r.finish_reason for r in res] == ["stop", "length", "stop", "length", "stop"]
    assert res[0].stop_token == STOP and res[1].stop_token is None
    assert [r.prompt_tokens for r in res] == [3, 1, 5, 2, 3]
    # three batches one after another: (0,1), (2,3), (4); the stopped request leaves its batch
    starts = [e for e in be.log if e[0] == "start"]
    assert len(starts) == 3 and loop.stats.n_batches == 3
    first = be.log[: be.log.index(("finish", starts[0][1])) + 1]
    decodes = [e[1] for e in first if e[0] == "decode"]
    assert decodes == [starts[0][1], starts[0][1], (starts[0][1][1],)]
    # the stop token never reaches the sampler's history, everything else does
    assert smp.accepted[0] == PROMPTS[0] + [10, 11] and smp.accepted[2] == PROMPTS[2]
    assert loop.stats.n_prompt == 14 and loop.stats.n_gen == 11


def test_last_token_is_sampled_but_not_fed():
    res, be, _, _ = run([[0]], [[10, 11, 12, 13]], max_batch=1, max_new_tokens=3, stop_ids=[])
    assert res[0].tokens == [10, 11, 12] and res[0].finish_reason == "length"
    assert [e[0] for e in be.log] == ["start", "prefill", "decode", "decode", "finish"]


def test_context_budget():
    assert token_budget(10, 5, 100) == (5, "length")
    assert token_budget(98, 5, 100) == (3, "context")        # 100 - 98 + 1
    assert token_budget(10, 0, 100) == (91, "context") and token_budget(10, -1, 100) == (91, "context")
    res, be, _, _ = run([[0, 1, 1, 1, 1, 1]], [[10] * 20], max_batch=1, max_seq_len=8, max_new_tokens=10, stop_ids=[])
    assert len(res[0].tokens) == 3 and res[0].finish_reason == "context"
    assert sum(1 for e in be.log if e[0] == "decode") == 2       # 6 + 2 fed tokens = the context of 8
    with pytest.raises(ValueError, match="exceeds the context"):
        run([[0] * 9], [[1]], max_seq_len=8)
    with pytest.raises(ValueError, match="empty prompt"):
        run([[]], [[1]])


def test_batches_are_planned_by_slots_and_by_cache_room():
    lens, budgets = [10, 10, 10, 10, 10], [7, 7, 7, 7, 7]
    assert plan_batch([0, 1, 2, 3, 4], lens, budgets, max_batch=3, max_tokens=10_000, page_size=16) == [0, 1, 2]
    assert plan_batch([0, 1, 2, 3, 4], lens, budgets, max_batch=8, max_tokens=40, page_size=16) == [0, 1]
    assert plan_batch([3, 4], lens, budgets, max_batch=8, max_tokens=8, page_size=16) == [3]      # at least one
    assert plan_batch([0, 1], [16, 1], [1, 17], 8, 48, 16) == [0, 1]                               # 16 + 32
    assert plan_batch([0, 1], [16, 1], [2, 17], 8, 48, 16) == [0]                                  # 32 + 32


def test_slots_are_given_back_when_a_step_fails():
    class Failing(Script):
        def decode(self, slots, tokens):
            raise RuntimeError("boom")

    be = Failing([[0]], [[1, 2, 3]], 1)
    loop = GenerationLoop(be, 1, 1000, 100, 16)
    with pytest.raises(RuntimeError, match="boom"):
        loop.run([[0]], PassThrough(), max_new_tokens=3)
    assert be.free == [0]


def test_streaming_callback_sees_every_emitted_token():
    seen = []
    res, *_ = run(PROMPTS[:2], SCRIPTS[:2], max_batch=2, max_new_tokens=3, stop_ids=[STOP], on_step=lambda d: seen.append(dict(d)))
    assert seen == [{0: 10, 1: 20}, {0: 11, 1: 21}, {1: 22}]


def test_interruption_returns_what_was_generated_so_far():
    """The flag is polled once per step (src/gen.zig:476-479): running requests end with their
    tokens and the reason "interrupted", requests of later batches come back empty, every slot is
    given back, and a request that ended before the flag keeps its own reason."""
    be = Script(PROMPTS, SCRIPTS, 2)
    loop = GenerationLoop(be, 2, 10_000, 1000, 16)
    seen = []

    def on_step(d):
        seen.append(dict(d))
        if len(seen) == 2:
            loop.interrupt.set()

    res = loop.run(PROMPTS, PassThrough(), max_new_tokens=5, stop_ids=[STOP], on_step=on_step)
    assert sorted(be.free) == [0, 1]
    assert [r.tokens for r in res] == [[10, 11], [20, 21], [], [], []]
    assert [r.finish_reason for r in res] == ["interrupted"] * 5
    assert sum(1 for e in be.log if e[0] == "start") == 1 and sum(1 for e in be.log if e[0] == "decode") == 1

    # a request that stopped before the flag was set keeps "stop"
    prompts, scripts = [[0, 7], [1, 8]], [[STOP], [30, 31, 32, 33, 34]]
    be = Script(prompts, scripts, 2)
    loop = GenerationLoop(be, 2, 10_000, 1000, 16)
    res = loop.run(prompts, PassThrough(), max_new_tokens=5, stop_ids=[STOP], on_step=lambda d: loop.interrupt.set())
    assert [(r.tokens, r.finish_reason) for r in res] == [([], "stop"), ([30], "interrupted")]
