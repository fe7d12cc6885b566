"""Replays requests through bin/trace_run in every way of cutting the work and compares the
logits with the plain implementation: each request alone and whole; the last 32 tokens one by
one; batches of unequal lengths whose shorter requests end earlier, one batch after another so
that slots and pages are used again.  Float32 and bfloat16."""
import numpy as np
import pytest

import helpers
from plain_lfm2 import PlainLfm2

pytestmark = pytest.mark.gpu

LENGTHS = {"tiny_a": [5, 11, 17, 40, 70], "tiny_b": [1, 2, 9, 33, 64, 100], "tiny_c": [3, 29, 66, 130, 47],
           "tiny_d": [200, 7, 65, 130, 33], "tiny_e": [90, 41, 3, 150, 64]}
DECODE_TAIL = 32


def _lengths(name):
    return LENGTHS[name.replace("loud_", "tiny_")]


def _requests(name):
    vocab = helpers.TINY[name]["config"]["vocab_size"]
    return {f"r{i}": helpers.random_tokens(1000 + i, n, vocab) for i, n in enumerate(_lengths(name))}


def _batches(reqs):
    """Groups of requests that start together: prompts whole (all but the last `tail` tokens),
    then one token each; shorter requests end earlier."""
    ids = list(reqs)
    return [ids[:3], ids[3:], ids[1:4]]


def build_steps(reqs):
    """One trace with all three cuts; returns (steps, expectations) where an expectation is
    (step, row, request id, position)."""
    steps, expect = [], []
    n = 0

    def emit(entries, end):
        nonlocal n
        row = 0
        for e in entries:
            for w in e["want"]:
                expect.append((n, row, e["id"].split("#")[0], e["_pos0"] + w))
                row += 1
        steps.append({"step": n, "entries": [{k: v for k, v in e.items() if not k.startswith("_")} for e in entries],
                      "end": end})
        n += 1

    # cut 1: each request alone and whole, logits at every position
    for rid, toks in reqs.items():
        emit([{"id": rid + "#whole", "tokens": toks, "want": list(range(len(toks))), "_pos0": 0}], [rid + "#whole"])
    # cut 2: prefix whole, then the last 32 tokens one by one
    for rid, toks in reqs.items():
        tail = min(DECODE_TAIL, len(toks) - 1)
        if tail <= 0:
            continue
        head = len(toks) - tail
        emit([{"id": rid + "#tail", "tokens": toks[:head], "want": [head - 1], "_pos0": 0}], [])
        for p in range(head, len(toks)):
            emit([{"id": rid + "#tail", "tokens": [toks[p]], "want": [0], "_pos0": p}],
                 [rid + "#tail"] if p == len(toks) - 1 else [])
    # cut 3: batches of unequal lengths, one after another
    for bi, batch in enumerate(_batches(reqs)):
        tag = f"#b{bi}"
        heads = {rid: max(1, len(reqs[rid]) - DECODE_TAIL) for rid in batch}
        entries, end = [], []
        for rid in batch:
            h = heads[rid]
            entries.append({"id": rid + tag, "tokens": reqs[rid][:h], "want": [0, h - 1] if h > 1 else [0], "_pos0": 0})
            if h == len(reqs[rid]):
                end.append(rid + tag)
        emit(entries, end)
        live = [rid for rid in batch if heads[rid] < len(reqs[rid])]
        p = 0
        while live:
            entries, end = [], []
            for rid in live:
                pos = heads[rid] + p
                entries.append({"id": rid + tag, "tokens": [reqs[rid][pos]], "want": [0], "_pos0": pos})
                if pos == len(reqs[rid]) - 1:
                    end.append(rid + tag)
            emit(entries, end)
            live = [rid for rid in live if heads[rid] + p < len(reqs[rid]) - 1]
            p += 1
    return steps, expect


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(helpers.TINY))
def test_replay_all_cuts(model_folders, tmp_path, name, dtype):
    folder = model_folders[name]
    reqs = _requests(name)
    plain = PlainLfm2(folder, dtype=np.float64)
    ref = {rid: plain.logits(toks) for rid, toks in reqs.items()}
    steps, expect = build_steps(reqs)
    live_max = 3 * 64 * (-(-max(_lengths(name)) // 64))
    got = helpers.run_trace(folder, dtype, steps, max_tokens=live_max, out_dir=tmp_path / "out")
    worst, where = 0.0, None
    for step, row, rid, pos in expect:
        e = np.max(np.abs(got[step][row].astype(np.float64) - ref[rid][pos])) / np.max(np.abs(ref[rid]))
        if e > worst:
            worst, where = e, (step, row, rid, pos, steps[step]["entries"][0]["id"])
    print(f"replay {name} {dtype}: worst error {worst:.3e} of max |logit| (tolerance {helpers.tol(name, dtype):.0e})")
    assert worst <= helpers.tol(name, dtype), f"{name} {dtype}: worst error {worst:.3e} at (step,row,req,pos,first id) {where}"
