"""The model that bench.py measures, checked: the LFM2-1.2B shape (all 16 layers, vocabulary
65,536) with seeded random weights written to a folder, loaded as a bfloat16 engine, a float32
engine and the plain implementation from the same file.

At this size the engine takes kernels that no tiny configuration reaches: pairs of thread blocks
on 256 x 256 tiles with the TMA reduce-add into the residual stream, the SwiGLU epilogue of the
tcgen05 product with the weights on its 128-row side (17 to 64 rows and 2F > 12,288 only), its
split-K over a cluster of 8 blocks, 32 heads on 8 KV heads in the tcgen05 prompt attention, a
head of 65,536 rows.

What one step must equal: src/model.zig:2347-2516.  (a) float32 engine = plain float64 on a short
prompt; (b) float32 engine under every cut = itself whole; (c) bfloat16 engine under every cut =
float32 engine whole: each request alone and whole, the last 32 tokens one by one, and unequal
batches whose shorter requests end earlier, one batch after another in the same engine.
Random weights N(0, 0.02) at width 2048 keep every contraction's output as large as its input,
so the logits depend on every layer (they are not the token's own embedding)."""
import numpy as np
import pytest
import torch

import helpers
from bench import LFM2_1_2B
import plain_lfm2 as P
from plain_lfm2 import PlainLfm2

pytestmark = pytest.mark.gpu

VOCAB = LFM2_1_2B["vocab_size"]
TAIL = 32
# requests: three of 40 / 129 / 300 tokens, and twenty short ones for batches of 9 to 64 rows (both kernels for few rows)
LENS = [40, 129, 300] + [5 + (7 * i) % 56 for i in range(20)]
BATCHES = [[0, 1, 2], list(range(3, 23)), [2, 0, 22, 1]]


class Shape:
    def __init__(self, folder):
        import zinfer_b200 as z
        self.folder = folder
        self.engines = {}
        for dtype in ("float32", "bfloat16"):
            model = z.load(folder, dtype=dtype)
            self.engines[dtype] = z.Engine(model, max_batch=24, max_seq_len=384, page_size=64)
        self.reqs = [helpers.random_tokens(8000 + i, n, VOCAB) for i, n in enumerate(LENS)]
        self.heads = [max(1, n - TAIL) for n in LENS]
        # the float32 engine, each request alone and whole: the reference of everything else
        self.whole = {}
        eng = self.engines["float32"]
        for i, toks in enumerate(self.reqs):
            slot = eng.start(1)
            self.whole[i] = eng.step(slot, [toks], want=[list(range(len(toks)))]).cpu().numpy().astype(np.float64)
            eng.finish(slot)
        eng.check_status()


@pytest.fixture(scope="module")
def shape(tmp_path_factory):
    import zinfer_b200 as z
    cfg = z.config_from_dict(dict(LFM2_1_2B))
    assert cfg.num_hidden_layers == 16 and cfg.ffn_dim == 8192
    folder = z.write_random_model(tmp_path_factory.mktemp("lfm2_1_2b") / "m", cfg, seed=5, fill_on_device=True)
    return Shape(folder)


def err(got, ref_rows, scale_of):
    return float(np.abs(got.astype(np.float64) - ref_rows).max() / np.abs(scale_of).max())


def test_float32_engine_equals_plain_on_a_short_prompt(shape):
    plain = PlainLfm2(shape.folder, dtype=np.float64)
    toks = shape.reqs[0][:12]
    ref = plain.logits(toks).astype(np.float64)
    e = err(shape.whole[0][:12], ref, ref)
    print(f"1.2B shape, float32 engine against plain float64, 12 tokens: error {e:.3e} of max |logit| {np.abs(ref).max():.2f}")
    assert e <= helpers.TOL_LOUD["float32"]
    # the logits are not the token's own embedding: the largest is rarely the input token's
    assert np.mean(ref.argmax(-1) == np.asarray(toks)) < 0.5
    eng = shape.engines["bfloat16"]
    slot = eng.start(1)
    got = eng.step(slot, [toks], want=[list(range(12))]).cpu().numpy()
    eng.finish(slot)
    e16 = err(got, ref, ref)
    plain.act = P.to_bf16              # what rounding the contractions' inputs, the cache and the probabilities alone costs
    floor = err(plain.logits(toks), ref, ref)
    print(f"1.2B shape, bfloat16 engine against plain float64, 12 tokens: error {e16:.3e} (floor of a bfloat16 pipeline {floor:.3e})")
    assert e16 <= helpers.TOL_LOUD["bfloat16"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_every_cut_equals_the_float32_engine_whole(shape, dtype):
    eng, reqs, heads, ref = shape.engines[dtype], shape.reqs, shape.heads, shape.whole
    tol = helpers.TOL_LOUD[dtype]
    worst = {"whole": 0.0, "tail": 0.0, "batches": 0.0}

    # each request alone and whole, logits at several positions
    for i in (0, 1, 2, 5, 17):
        n = len(reqs[i])
        want = sorted({0, 1, n // 3, n // 2, n - 2, n - 1} & set(range(n)))
        slot = eng.start(1)
        got = eng.step(slot, [reqs[i]], want=[want]).cpu().numpy()
        eng.finish(slot)
        worst["whole"] = max(worst["whole"], err(got, ref[i][want], ref[i]))

    # the prefix whole, then the last 32 tokens one by one
    for i in (0, 1, 2):
        slot = eng.start(1)
        got = eng.step(slot, [reqs[i][:heads[i]]]).cpu().numpy()
        worst["tail"] = max(worst["tail"], err(got, ref[i][heads[i] - 1:heads[i]], ref[i]))
        for p in range(heads[i], len(reqs[i])):
            got = eng.decode(slot, [reqs[i][p]]).cpu().numpy()
            worst["tail"] = max(worst["tail"], err(got, ref[i][p:p + 1], ref[i]))
        eng.finish(slot)

    # batches of unequal lengths, one after another in the same engine; shorter requests end earlier
    sizes = set()
    for batch in BATCHES:
        slots = eng.start(len(batch))
        got = eng.step(slots, [reqs[i][:heads[i]] for i in batch], want=[[0, heads[i] - 1] for i in batch]).cpu().numpy()
        for r, i in enumerate(batch):
            worst["batches"] = max(worst["batches"], err(got[2 * r:2 * r + 2], ref[i][[0, heads[i] - 1]], ref[i]))
        fed = {i: heads[i] for i in batch}
        while True:
            live = [i for i in batch if fed[i] < len(reqs[i])]
            if not live:
                break
            sizes.add(len(live))
            got = eng.decode([slots[batch.index(i)] for i in live], [reqs[i][fed[i]] for i in live]).cpu().numpy()
            for r, i in enumerate(live):
                worst["batches"] = max(worst["batches"], err(got[r:r + 1], ref[i][fed[i]:fed[i] + 1], ref[i]))
                fed[i] += 1
        eng.finish(slots)
    eng.check_status()
    eng.cache.check_consistency()
    assert {20, 3} <= sizes and any(9 <= s <= 16 for s in sizes) and any(s <= 8 for s in sizes), sizes
    print(f"1.2B shape {dtype} against the float32 engine whole: " + ", ".join(f"{k} {v:.3e}" for k, v in worst.items()))
    assert max(worst.values()) <= tol, worst
