"""The step's batch description on the host: how sequences of unequal lengths are packed into one
int32 buffer; and the attention part's launch plans: how query tiles are cut, and how a
single-token step cuts the keys into chunks."""
import numpy as np
import pytest
import torch

from zinfer_b200.engine.context import StepContext, batch_layout, pack_batch
from zinfer_b200.parts.attention import key_capacity, key_chunks, query_tiles


def unpack(buf, n_tokens, n_seqs):
    lay = batch_layout(n_tokens, n_seqs)
    return {name: buf[o:o + size] for name, (o, size) in lay.items() if name != "_total"}


@pytest.mark.parametrize("lens", [[3], [1, 1, 1], [5, 1, 9, 2], [64, 63, 65]])
def test_packed_batch_holds_every_sequence_at_its_place(lens):
    rng = np.random.default_rng(sum(lens))
    slots = list(rng.permutation(len(lens) + 3)[:len(lens)])
    starts = [int(rng.integers(0, 50)) for _ in lens]
    tokens = [list(rng.integers(0, 1000, size=n)) for n in lens]
    buf = pack_batch(slots, starts, tokens)
    n, B = sum(lens), len(lens)
    lay = batch_layout(n, B)
    assert buf.dtype == np.int32 and buf.shape[0] == lay["_total"][0]
    assert all(o % 4 == 0 for o, _ in lay.values()), "every array starts on a 16-byte boundary"
    a = unpack(buf, n, B)
    assert a["cu_q"].tolist() == np.concatenate([[0], np.cumsum(lens)]).tolist()
    assert a["seq_start"].tolist() == starts and a["seq_slot"].tolist() == [int(s) for s in slots]
    for b in range(B):
        rows = slice(a["cu_q"][b], a["cu_q"][b + 1])
        assert a["tokens"][rows].tolist() == [int(t) for t in tokens[b]]
        assert set(a["tok_seq"][rows].tolist()) == {b}
        assert a["tok_pos"][rows].tolist() == list(range(starts[b], starts[b] + lens[b]))


@pytest.mark.parametrize("lens,bq", [([5, 1, 9, 2], 4), ([128, 1, 200], 128), ([3], 16), ([64, 64], 32)])
def test_query_tiles_cover_every_token_once(lens, bq):
    tiles = query_tiles(lens, bq)
    assert tiles.dtype == np.int32 and tiles.shape[0] == 2
    seen = [np.zeros(n, dtype=int) for n in lens]
    for b, q0 in tiles.T:
        assert q0 % bq == 0 and q0 < lens[b]
        seen[b][q0:min(q0 + bq, lens[b])] += 1
    assert all((s == 1).all() for s in seen)
    order = [(int(b), int(q0)) for b, q0 in tiles.T]
    assert order == sorted(order), "tiles go sequence by sequence, front to back"


def context(lens, starts):
    buf = torch.from_numpy(pack_batch(list(range(len(lens))), starts, [[0] * n for n in lens]))
    status = torch.zeros(1, dtype=torch.int32)
    return StepContext(torch.float32, torch.device("cpu"), status, buf, sum(lens), len(lens), lens,
                       max(s + n for s, n in zip(starts, lens)))


def test_step_context_views_and_kind_of_step():
    ctx = context([4, 1, 2], [10, 0, 7])
    assert ctx.n_tokens == 7 and ctx.n_seqs == 3 and ctx.max_q_len == 4 and ctx.max_kv_len == 14
    assert not ctx.is_decode
    assert ctx.cu_q.tolist() == [0, 4, 5, 7] and ctx.tok_pos.tolist() == [10, 11, 12, 13, 0, 7, 8]
    made = []
    first = ctx.memo("k", lambda: made.append(1) or [1, 2])
    assert ctx.memo("k", lambda: made.append(1) or [3]) is first and made == [1], "a memo is made once per key"
    one = context([1, 1], [5, 900])
    assert one.is_decode
    mixed = context([1, 2], [5, 9])
    assert not mixed.is_decode, "one token each is what makes a single-token step"


def test_key_capacity_grows_in_few_coarse_steps():
    caps = sorted({key_capacity(n) for n in range(1, 40000, 7)})
    assert caps[:6] == [512, 768, 1024, 1536, 2048, 3072] and len(caps) <= 14
    for n in (1, 512, 513, 3000, 32768, 32769):
        c = key_capacity(n)
        assert c >= n and (n <= 512 or c < 1.5 * n + 1), "never less than the sequence, never 1.5 times more"


@pytest.mark.parametrize("sm_count", [148, 20])
@pytest.mark.parametrize("n_seqs,n_kv,longest", [(1, 8, 100), (1, 8, 4096), (8, 8, 4096), (64, 8, 32768), (3, 1, 70000)])
def test_key_chunks_of_a_single_token_step(n_seqs, n_kv, longest, sm_count):
    n, keys = key_chunks(n_seqs, n_kv, longest, sm_count)
    cap = key_capacity(longest)
    if n == 1:
        assert keys == 0
        return
    assert keys % 64 == 0 and 128 <= keys <= 4096
    assert (n - 1) * keys < cap <= n * keys, "the chunks cover the capacity that holds the longest sequence"
    # the plan is the same for every length that shares the capacity: a recorded step stays valid
    assert key_chunks(n_seqs, n_kv, cap, sm_count) == (n, keys)
    below = cap * 3 // 4 if cap & (cap - 1) == 0 else cap * 2 // 3      # the capacity before this one
    assert key_capacity(below + 1) == cap and key_chunks(n_seqs, n_kv, below + 1, sm_count) == (n, keys)


def test_given_chunk_size_is_kept_whatever_the_batch():
    for n_seqs in (1, 5, 40):
        assert key_chunks(n_seqs, 4, 1000, 148, split_keys=256) == (4, 256)
    assert key_chunks(1, 4, 100, 148, split_keys=512) == (1, 0)
