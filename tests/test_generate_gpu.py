"""Generation through the Python entry point against the plain implementation: greedy tokens,
stop tokens, more requests than slots (slots used again), seeded temperature sampling that
does not depend on the batch, single-token steps from CUDA graphs, long decoding, the first
tokens of a sequence, and a toy mixer with state of its own."""
import numpy as np
import pytest
import torch

import helpers
from plain_lfm2 import PlainLfm2

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def check_greedy(plain, prompt, result, dtype, stop_ids, max_new, name="tiny"):
    """Every generated token is the plain implementation's argmax given the same prefix (in
    bfloat16: within the rounding tolerance of the best logit); the end is the plain one's too."""
    toks = list(prompt) + result.tokens
    ref = plain.logits(toks + ([result.stop_token] if result.stop_token is not None else []))
    tol = helpers.tol(name, dtype) * np.abs(ref).max()
    sampled = result.tokens + ([result.stop_token] if result.stop_token is not None else [])
    for i, t in enumerate(sampled):
        row = ref[len(prompt) - 1 + i]
        assert row[t] >= row.max() - 2 * tol, f"token {i} = {t} is not the best (best {row.argmax()})"
        if dtype == "float32":
            assert t == int(row.argmax())
    if result.finish_reason == "stop":
        assert result.stop_token in stop_ids
    else:
        assert len(result.tokens) == max_new and not (set(result.tokens) & set(stop_ids))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(helpers.TINY))
def test_greedy_generation_matches_plain(model_folders, name, dtype):
    import zinfer_b200 as z
    folder = model_folders[name]
    plain = PlainLfm2(folder, dtype=np.float64)
    vocab = plain.cfg["vocab_size"]
    prompts = [helpers.random_tokens(50 + i, n, vocab) for i, n in enumerate([3, 1, 20, 70, 9, 2, 33])]
    model = z.load(folder, dtype=dtype)
    engine = z.Engine(model, max_batch=3, max_seq_len=128, page_size=16)
    # stop ids: the tokens that greedy decoding of two of the prompts produces at step 4 and 2
    probe = engine.generate(prompts, max_new_tokens=8, temp=0.0, stop_ids=[])
    stop_ids = [probe[2].tokens[4], probe[4].tokens[2]]
    results = engine.generate(prompts, max_new_tokens=12, temp=0.0, stop_ids=stop_ids)
    assert any(r.finish_reason == "stop" for r in results) and any(r.finish_reason == "length" for r in results)
    for p, r in zip(prompts, results):
        check_greedy(plain, p, r, dtype, stop_ids, 12, name)
    assert engine.stats.n_batches == 3 and engine.cache.free_slot_count() == 3
    assert engine.cache.free_page_count() == [g.num_pages for g in engine.cache.groups]
    engine.cache.check_consistency()


def test_seeded_sampling_is_reproducible_and_independent_of_the_batch(model_folders):
    import zinfer_b200 as z
    model = z.load(model_folders["tiny_b"], dtype="fp32")
    vocab = model.config.vocab_size
    prompts = [helpers.random_tokens(70 + i, n, vocab) for i, n in enumerate([1, 2, 9, 33, 64])]
    opts = dict(max_new_tokens=16, temp=0.8, top_k=0, top_p=1.0, min_p=0.0, seed=123, stop_ids=[])
    eng = z.Engine(model, max_batch=5, max_seq_len=128, page_size=32)
    a = [r.tokens for r in eng.generate(prompts, **opts)]
    b = [r.tokens for r in eng.generate(prompts, **opts)]
    assert a == b and all(len(t) == 16 for t in a)
    small = z.Engine(model, max_batch=2, max_seq_len=128, page_size=16, use_graphs=False)
    c = [r.tokens for r in small.generate(prompts, **opts)]
    assert a == c, "a request's tokens changed with the batch it ran in"
    d = [r.tokens for r in eng.generate(prompts, **dict(opts, seed=124))]
    assert a != d
    assert len({tuple(t) for t in a}) == 5


def test_sampled_tokens_follow_the_plain_distribution(model_folders):
    """Teacher-forced: at every step the sampled token equals the plain chain's pick from the plain
    logits with the same uniform number."""
    import zinfer_b200 as z
    import plain_lfm2 as P
    from zinfer_b200.sampling import uniform
    folder = model_folders["tiny_a"]
    plain = PlainLfm2(folder, dtype=np.float64)
    model = z.load(folder, dtype="fp32")
    prompt = helpers.random_tokens(90, 11, 256)
    eng = z.Engine(model, max_batch=1, max_seq_len=128)
    opts = dict(temp=0.8, top_k=40, top_p=0.95, min_p=0.05, seed=5)
    out = eng.generate([prompt], max_new_tokens=20, stop_ids=[], **opts)[0].tokens
    ref = plain.logits(prompt + out)
    same = 0
    for i, t in enumerate(out):
        p = P.filtered_probs(ref[len(prompt) - 1 + i], 0.8, 40, 0.95, 0.05)
        c = np.cumsum(p)
        assert p[t] > 0
        same += int(t == int(np.searchsorted(c, uniform(5, 0, i, 0) * c[-1], side="left")))
    assert same >= 19


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_graph_decode_equals_plain_steps_and_long_decoding(model_folders, dtype):
    """300 single-token steps over page edges and far past the window, from CUDA graphs and as
    plain steps, both against whole-sequence logits."""
    import zinfer_b200 as z
    folder = model_folders["tiny_c"]
    plain = PlainLfm2(folder, dtype=np.float64)
    vocab = plain.cfg["vocab_size"]
    seqs = [helpers.random_tokens(200 + i, n, vocab) for i, n in enumerate([330, 301, 317])]
    heads = [30, 1, 17]
    ref = [plain.logits(s) for s in seqs]
    model = z.load(folder, dtype=dtype)
    worst = {}
    for graphs in (True, False):
        eng = z.Engine(model, max_batch=4, max_seq_len=512, page_size=16, use_graphs=graphs)
        slots = eng.start(3)
        eng.step(slots, [s[:h] for s, h in zip(seqs, heads)], want=[[] for _ in seqs])
        err = 0.0
        for p in range(300):
            logits = eng.decode(slots, [s[h + p] for s, h in zip(seqs, heads)]).cpu().numpy()
            for i in range(3):
                err = max(err, np.abs(logits[i] - ref[i][heads[i] + p]).max() / np.abs(ref[i]).max())
        eng.check_status()
        eng.finish(slots)
        worst[graphs] = err
        assert (eng.graph_captures > 0) == graphs, "single-token steps are recorded exactly when graphs are asked for"
    assert max(worst.values()) <= helpers.TOL[dtype], worst


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_first_tokens_of_a_sequence(model_folders, name):
    """Prompts of one token, shorter than the conv window, then the first decoded tokens."""
    import zinfer_b200 as z
    folder = model_folders[name]
    plain = PlainLfm2(folder, dtype=np.float64)
    vocab = plain.cfg["vocab_size"]
    seqs = [helpers.random_tokens(300 + i, 6, vocab) for i in range(4)]
    ref = [plain.logits(s) for s in seqs]
    eng = z.Engine(z.load(folder, dtype="fp32"), max_batch=4, max_seq_len=64, page_size=16)
    slots = eng.start(4)
    first = eng.step(slots, [s[:n] for s, n in zip(seqs, [1, 2, 3, 1])], want=[[0], [0, 1], [0, 1, 2], [0]]).cpu().numpy()
    rows = [(0, 0), (1, 0), (1, 1), (2, 0), (2, 1), (2, 2), (3, 0)]
    for r, (i, p) in enumerate(rows):
        assert np.abs(first[r] - ref[i][p]).max() <= helpers.TOL["float32"] * np.abs(ref[i]).max()
    fed = [1, 2, 3, 1]
    for step in range(3):
        live = [i for i in range(4) if fed[i] < 6]
        out = eng.step([slots[i] for i in live], [[seqs[i][fed[i]]] for i in live]).cpu().numpy()
        for r, i in enumerate(live):
            assert np.abs(out[r] - ref[i][fed[i]]).max() <= helpers.TOL["float32"] * np.abs(ref[i]).max()
            fed[i] += 1
    eng.finish(slots)


def test_chunked_prompt_step_equals_the_whole_step(model_folders):
    import zinfer_b200 as z
    folder = model_folders["tiny_c"]
    model = z.load(folder, dtype="fp32")
    vocab = model.config.vocab_size
    seqs = [helpers.random_tokens(400 + i, n, vocab) for i, n in enumerate([90, 7, 41])]
    want = [[0, 50, 89], [6], [0, 40]]
    outs = []
    for chunk in (8192, 32):
        eng = z.Engine(model, max_batch=3, max_seq_len=128, page_size=16, max_step_tokens=chunk)
        slots = eng.start(3)
        outs.append(eng.step(slots, seqs, want=want).cpu().numpy())
        eng.finish(slots)
    assert outs[0].shape == (6, vocab)
    assert np.abs(outs[0] - outs[1]).max() <= 1e-5 * np.abs(outs[0]).max()


def test_errors_leave_the_engine_usable(model_folders):
    import zinfer_b200 as z
    from zinfer_b200.cache import ContextFull, NoFreeSlot, OutOfPages
    model = z.load(model_folders["tiny_a"], dtype="fp32")
    eng = z.Engine(model, max_batch=2, max_seq_len=64, max_tokens=64, page_size=16)
    slots = eng.start(2)
    with pytest.raises(NoFreeSlot):
        eng.start(1)
    with pytest.raises(ContextFull):
        eng.step([slots[0]], [[1] * 65])
    with pytest.raises(OutOfPages):
        eng.step(slots, [[1] * 40, [2] * 40])
    with pytest.raises(z.StepError, match="vocabulary"):
        eng.step([slots[0]], [[1, 256]])
    eng.finish(slots)
    slots = eng.start(1)
    ok = eng.step(slots, [[1, 2, 3]])
    assert ok.shape == (1, 256) and torch.isfinite(ok).all()
    eng.finish(slots)
    eng.cache.check_consistency()


@pytest.mark.parametrize("temp", [0.0, 0.9])
def test_running_one_step_ahead_changes_no_token(model_folders, temp):
    """The loop that launches a step before the host has read the previous tokens gives the
    tokens, stop reasons and order of the plain loop: unequal prompts, budgets that end requests
    at different steps, and stop tokens that end some requests in mid-batch (learned one step
    late by the loop that runs ahead)."""
    import zinfer_b200 as z
    folder = model_folders["tiny_b"]
    model = z.load(folder, dtype="float32")
    vocab = model.config.vocab_size
    prompts = [helpers.random_tokens(700 + i, n, vocab) for i, n in enumerate([3, 17, 40, 9, 26, 1])]
    plain = z.Engine(model, max_batch=4, max_seq_len=256, page_size=16, lookahead=False)
    ahead = z.Engine(model, max_batch=4, max_seq_len=256, page_size=16)
    free = plain.generate(prompts, max_new_tokens=24, temp=temp, seed=5, stop_ids=[])
    # stop tokens: what some requests emit at their 5th and 11th place
    stops = sorted({free[1].tokens[4], free[4].tokens[10], free[2].tokens[0]})
    for stop_ids, budget in (([], 24), (stops, 24), (stops, 7)):
        seen = []
        a = plain.generate(prompts, max_new_tokens=budget, temp=temp, seed=5, stop_ids=stop_ids)
        b = ahead.generate(prompts, max_new_tokens=budget, temp=temp, seed=5, stop_ids=stop_ids,
                           on_step=lambda d: seen.append(dict(d)))
        assert [(r.tokens, r.finish_reason, r.stop_token) for r in a] == [(r.tokens, r.finish_reason, r.stop_token) for r in b]
        assert ahead.stats.n_gen == plain.stats.n_gen
        for i, r in enumerate(b):       # the callback saw every emitted token, in order
            assert [d[i] for d in seen if i in d] == r.tokens
    assert any(r.finish_reason == "stop" for r in b) and any(r.finish_reason != "stop" for r in b)
    plain.cache.check_consistency()
    ahead.cache.check_consistency()


@pytest.mark.parametrize("temp", [0.0, 0.8])
def test_repetition_penalty_through_the_entry_point(model_folders, temp):
    """With a repetition penalty the loop runs a step ahead too (the window of recent tokens lives on
    the device).  Greedy: every token is the arg-max of the plain logits after the plain penalty over
    the last 64 tokens of prompt and output, for prompts shorter and longer than the window.  Sampled:
    the tokens are those of the loop that does not run ahead."""
    import zinfer_b200 as z
    import plain_lfm2 as P
    folder = model_folders["tiny_b"]
    plain = PlainLfm2(folder, dtype=np.float64)
    vocab = plain.cfg["vocab_size"]
    prompts = [helpers.random_tokens(900 + i, n, vocab) for i, n in enumerate([3, 80, 17, 1, 64])]
    model = z.load(folder, dtype="float32")
    ahead = z.Engine(model, max_batch=3, max_seq_len=256, page_size=16)
    out = ahead.generate(prompts, max_new_tokens=20, temp=temp, top_k=0, top_p=1.0, min_p=0.0, seed=2,
                         repeat_penalty=1.7, stop_ids=[])
    if temp == 0.0:
        for p, r in zip(prompts, out):
            toks = list(p)
            for i, t in enumerate(r.tokens):
                row = P.repeat_penalty(plain.logits(toks)[-1], toks, 1.7)
                assert t == int(np.argmax(row)), f"token {i}: {t}, plain {int(np.argmax(row))}"
                toks.append(t)
        # the penalty changes what is generated (else the test would not see a missing one)
        free = ahead.generate(prompts, max_new_tokens=20, temp=0.0, stop_ids=[])
        assert any(a.tokens != b.tokens for a, b in zip(out, free))
    else:
        slow = z.Engine(model, max_batch=3, max_seq_len=256, page_size=16, lookahead=False)
        ref = slow.generate(prompts, max_new_tokens=20, temp=temp, top_k=0, top_p=1.0, min_p=0.0, seed=2,
                            repeat_penalty=1.7, stop_ids=[])
        assert [r.tokens for r in out] == [r.tokens for r in ref]
