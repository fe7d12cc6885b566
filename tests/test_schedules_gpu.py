"""Schedules of the engine that only large or long batches reach, against the plain implementation:
single-token steps of 12, 20, 40 and 100 sequences whose batch shrinks as requests end (the kernels
chosen for up to 8, up to 16, up to 64 and more than 64 rows, each recorded in a CUDA graph and replayed), a
second batch in the same engine; sequences that grow past 512, 768 and 1024 tokens, where the
layout of the key chunks of single-token attention (and with it the recorded step) changes;
and prompts cut into chunks of 64 and 128 tokens in bfloat16.  All on the loud configurations,
where a wrong row, slot or chunk moves the logits as a whole."""
import numpy as np
import pytest
import torch

import helpers
from plain_lfm2 import PlainLfm2

pytestmark = pytest.mark.gpu


def drive(engine, seqs, heads, ref, use_decode=True):
    """Feeds seqs[i][:heads[i]] in one step, then one token per live sequence and step until every
    sequence is through; compares the logits at every fed position from the heads' last on.
    Returns (worst error relative to max |logit| of the sequence, where, batch sizes seen)."""
    n = len(seqs)
    slots = engine.start(n)
    worst, where, sizes = 0.0, None, []

    def compare(rows, logits):
        nonlocal worst, where
        got = logits.float().cpu().numpy().astype(np.float64)
        for r, (i, p) in enumerate(rows):
            e = np.abs(got[r] - ref[i][p]).max() / np.abs(ref[i]).max()
            if not e <= worst:              # also catches NaN
                worst, where = e, (i, p, len(rows))

    try:
        out = engine.step(slots, [s[:h] for s, h in zip(seqs, heads)])
        compare([(i, heads[i] - 1) for i in range(n)], out)
        fed = list(heads)
        while True:
            live = [i for i in range(n) if fed[i] < len(seqs[i])]
            if not live:
                break
            sizes.append(len(live))
            toks = [seqs[i][fed[i]] for i in live]
            ls = [slots[i] for i in live]
            out = engine.decode(ls, toks) if use_decode else engine.step(ls, [[t] for t in toks])
            compare([(i, fed[i]) for i in live], out)
            for i in live:
                fed[i] += 1
        engine.check_status()
    finally:
        engine.finish(slots)
    return worst, where, sizes


@pytest.mark.parametrize("n_seqs,dtype", [(12, "bfloat16"), (20, "bfloat16"), (40, "bfloat16"), (20, "float32"), (100, "bfloat16")])
@pytest.mark.parametrize("name", ["loud_d", "loud_e"])
def test_many_sequences_shrinking_batches_then_a_second_batch(model_folders, name, n_seqs, dtype):
    import zinfer_b200 as z
    folder = model_folders[name]
    plain = PlainLfm2(folder, dtype=np.float64)
    vocab = plain.cfg["vocab_size"]
    rng = np.random.default_rng(n_seqs)
    engine = z.Engine(z.load(folder, dtype=dtype), max_batch=n_seqs, max_seq_len=192, page_size=64)
    for batch in range(2):
        heads = rng.integers(1, 100, size=n_seqs).tolist()
        tails = rng.choice([3, 7, 11, 16], size=n_seqs).tolist()          # requests end in four groups
        seqs = [helpers.random_tokens(5000 + 100 * batch + i, h + t, vocab) for i, (h, t) in enumerate(zip(heads, tails))]
        ref = [plain.logits(s) for s in seqs]
        worst, where, sizes = drive(engine, seqs, heads, ref)
        assert len(set(sizes)) >= 3 and sizes[0] == n_seqs, sizes
        print(f"{name} {dtype} {n_seqs} sequences, batch {batch}: worst error {worst:.3e}, batch sizes {sorted(set(sizes))}")
        assert worst <= helpers.tol(name, dtype), f"worst error {worst:.3e} at (sequence, position, batch size) {where}"
    if dtype == "bfloat16":
        assert engine.graph_captures >= 3, "the single-token steps were not replayed from graphs"
    engine.cache.check_consistency()
    assert engine.cache.free_slot_count() == n_seqs


LONG = dict(helpers.TINY["loud_d"]["config"], max_position_embeddings=2048)


@pytest.fixture(scope="module")
def long_folder(tmp_path_factory):
    import zinfer_b200 as z
    return z.write_random_model(tmp_path_factory.mktemp("long") / "m", z.config_from_dict(LONG), 77,
                                std=LONG["hidden_size"] ** -0.5)


@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_sequences_that_outgrow_the_key_chunk_layout(long_folder, dtype, graphs):
    """Three sequences decode across 512, 768 and 1024 tokens: the longest decides the layout of
    the key chunks, so every sequence sees its keys cut differently as the batch grows, with
    recorded steps (one per layout) and without."""
    import zinfer_b200 as z
    from zinfer_b200.parts.attention import key_chunks
    plain = PlainLfm2(long_folder, dtype=np.float64)
    vocab = plain.cfg["vocab_size"]
    heads = [500, 190, 3]
    lens = [1040, 760, 530]                                    # the batch shrinks on the way, too
    seqs = [helpers.random_tokens(900 + i, n, vocab) for i, n in enumerate(lens)]
    ref = [plain.logits(s) for s in seqs]
    model = z.load(long_folder, dtype=dtype)
    engine = z.Engine(model, max_batch=3, max_seq_len=1100, page_size=64, use_graphs=graphs)
    att = next(l.mixer for l in model.layers if l.mixer.kv_request() is not None)
    layouts = {key_chunks(3, att.n_kv, n, engine.sm_count) for n in (501, 600, 800, 1040)}
    assert len(layouts) == 4 and all(n > 1 for n, _ in layouts), layouts
    worst, where, sizes = drive(engine, seqs, heads, ref)
    print(f"long decode {dtype} graphs={graphs}: worst error {worst:.3e}")
    assert worst <= helpers.TOL_LOUD[dtype], f"worst error {worst:.3e} at (sequence, position, batch size) {where}"
    if graphs:
        assert engine.graph_captures >= 5, engine.graph_captures      # 3 layouts at 3 sequences, then 2 and 1 sequences
    else:
        assert engine.graph_captures == 0


@pytest.mark.parametrize("chunk", [64, 128])
@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
@pytest.mark.parametrize("name", ["loud_d", "loud_e", "loud_c"])
def test_chunked_prompts_against_plain(model_folders, name, dtype, chunk):
    """Prompts longer than a step may be are cut into packed chunks; a chunk continues every
    sequence from the cache and the state the chunk before it left."""
    import zinfer_b200 as z
    folder = model_folders[name]
    plain = PlainLfm2(folder, dtype=np.float64)
    vocab = plain.cfg["vocab_size"]
    lens = [200, 7, 65, 130, 129]
    seqs = [helpers.random_tokens(400 + i, n, vocab) for i, n in enumerate(lens)]
    want = [[0, 63, 64, 127, 128, 199], [6], [0, 64], [1, 129], [128]]
    ref = [plain.logits(s) for s in seqs]
    engine = z.Engine(z.load(folder, dtype=dtype), max_batch=5, max_seq_len=256, page_size=64, max_step_tokens=chunk)
    for round_ in range(2):
        slots = engine.start(5)
        out = engine.step(slots, seqs, want=want).float().cpu().numpy()
        # and one more token each, which reads what the last chunks left
        nxt = [helpers.random_tokens(450 + i, 1, vocab) for i in range(5)]
        more = engine.decode(slots, [t[0] for t in nxt]).float().cpu().numpy()
        engine.finish(slots)
        rows = [(i, p) for i, w in enumerate(want) for p in w]
        assert out.shape == (len(rows), vocab)
        for r, (i, p) in enumerate(rows):
            e = np.abs(out[r] - ref[i][p]).max() / np.abs(ref[i]).max()
            assert e <= helpers.tol(name, dtype), f"round {round_}: sequence {i} position {p}: error {e:.3e}"
        for i in range(5):
            full = plain.logits(seqs[i] + nxt[i])
            e = np.abs(more[i] - full[-1]).max() / np.abs(full).max()
            assert e <= helpers.tol(name, dtype), f"round {round_}: sequence {i}, the token after the prompt: error {e:.3e}"
    engine.cache.check_consistency()


@pytest.mark.parametrize("n_seqs", [5, 12, 40])
@pytest.mark.parametrize("name", ["loud_d", "loud_e"])
def test_single_token_steps_prepare_their_norms(model_folders, name, n_seqs, monkeypatch):
    """In bfloat16 steps of up to 64 rows the contraction that sums into the residual rows prepares the
    norm that follows, for every norm of the step but the first (behind the embedding), the final
    norm included: up to 8 rows in the mma.sync kernels, above in the tcgen05 kernel.  The same steps
    with that route closed agree with the plain model as well."""
    import zinfer_b200 as z
    from zinfer_b200 import kernels
    from zinfer_b200.parts.norm import RMSNorm
    folder = model_folders[name]
    plain = PlainLfm2(folder, dtype=np.float64)
    vocab, n_layers = plain.cfg["vocab_size"], plain.cfg["num_hidden_layers"]
    seqs = [helpers.random_tokens(900 + i, 9 + (3 * i) % 50 + 6, vocab) for i in range(n_seqs)]
    heads = [len(s) - 6 for s in seqs]
    ref = [plain.logits(s) for s in seqs]
    made = []      # contractions that were handed rows with their norm prepared

    def counting(fn):
        def call(a, *rest, **kw):
            if isinstance(a, kernels.ScaledInput):
                made.append(fn.__name__)
            return fn(a, *rest, **kw)
        return call

    for fn in ("gemm_skinny", "gemm_skinny_swiglu", "gemm_skinny_conv", "gemm_tc"):
        monkeypatch.setattr(kernels, fn, counting(getattr(kernels, fn)))
    counts = {}
    for route in ("prepared", "closed"):
        if route == "closed":
            monkeypatch.setattr(RMSNorm, "ahead", lambda self, ctx, x: None)
        engine = z.Engine(z.load(folder, dtype="bfloat16"), max_batch=n_seqs, max_seq_len=128, page_size=64,
                          use_graphs=False)
        made.clear()
        worst, where, sizes = drive(engine, seqs, heads, ref)
        counts[route] = len(made) / len(sizes)
        print(f"{name} {route}: {counts[route]:.1f} prepared norms a single-token step, worst error {worst:.3e}")
        assert worst <= helpers.tol(name, "bfloat16"), f"{route}: worst error {worst:.3e} at {where}"
    assert counts["prepared"] == 2 * n_layers and counts["closed"] == 0, counts
