"""The device sampler against the plain implementation: greedy, temperature, top-k, top-p,
min-p with ties, the sparse penalties, XTC's support, and the distribution of many draws."""
import numpy as np
import pytest
import torch

import plain_lfm2 as P

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def k():
    from zinfer_b200 import kernels
    kernels.require_cuda()
    return kernels


def logits_rows(n, V, seed, scale=3.0):
    return (np.random.default_rng(seed).standard_normal((n, V)) * scale).astype(np.float32)


def expected_pick(probs, u):
    """First index, in index order, at which the running sum reaches u * total."""
    c = np.cumsum(probs)
    return int(np.searchsorted(c, u * c[-1], side="left"))


def test_argmax_first_maximum_wins_and_nan_never_does(k):
    x = logits_rows(6, 1000, 1)
    x[0, [700, 20, 333]] = 50.0
    x[1, :] = 0.0
    x[2, 5] = np.nan
    x[2, 900] = 60.0
    got = k.argmax(torch.from_numpy(x).cuda()).cpu().tolist()
    assert got[0] == 20 and got[1] == 0 and got[2] == 900
    assert got[3:] == np.argmax(x[3:], axis=1).tolist()
    big = logits_rows(3, 65536 + 7, 2)
    assert k.argmax(torch.from_numpy(big).cuda()).cpu().tolist() == np.argmax(big, axis=1).tolist()


@pytest.mark.parametrize("V", [331, 5000, 65536])
@pytest.mark.parametrize("opts", [dict(temp=1.0), dict(temp=0.8, top_k=40, top_p=0.95, min_p=0.05),
                                  dict(temp=0.5, top_k=7), dict(temp=1.3, top_p=0.5), dict(temp=1.0, min_p=0.3),
                                  dict(temp=2.0, top_k=5, top_p=0.7, min_p=0.1)])
def test_draw_matches_the_plain_chain(k, V, opts):
    n = 48
    x = logits_rows(n, V, 3 + V)
    u = np.random.default_rng(4).random((n, 2)).astype(np.float32)
    got = k.sample(torch.from_numpy(x).cuda(), torch.from_numpy(u).cuda(), **opts).cpu().numpy()
    exact = 0
    for i in range(n):
        p = P.filtered_probs(x[i], opts["temp"], opts.get("top_k", 0), opts.get("top_p", 1.0), opts.get("min_p", 0.0))
        assert p[got[i]] > 0, f"row {i}: token {got[i]} is outside the support {np.nonzero(p)[0][:10]}"
        exact += int(got[i] == expected_pick(p, float(u[i, 0])))
    assert exact >= n - 1, f"only {exact} of {n} draws equal the plain implementation's"


def test_ties_are_cut_in_index_order(k):
    V = 2000
    x = np.full((4, V), -5.0, dtype=np.float32)
    x[:, 100:110] = 2.0                       # ten tied candidates
    x[:, 50] = 3.0
    u = np.array([[0.999, 0], [0.5, 0], [0.0, 0], [0.9999, 0]], dtype=np.float32)
    xs, us = torch.from_numpy(x).cuda(), torch.from_numpy(u).cuda()
    for _ in range(3):
        got = k.sample(xs, us, temp=1.0, top_k=4).cpu().numpy()      # 50 and the first three of the tie
        assert set(got.tolist()) <= {50, 100, 101, 102} and got[0] == 102 and got[2] == 50
    p = P.filtered_probs(x[0], 1.0, top_p=0.55)
    got = k.sample(xs, us, temp=1.0, top_p=0.55).cpu().numpy()
    assert all(p[g] > 0 for g in got) and got[3] == int(np.nonzero(p)[0].max())


def test_top_p_cut_is_the_same_in_every_run(k):
    """The masses that decide the top-p cut are summed in an order-independent way: the same rows
    and uniforms give the same tokens run after run, also for rows made so that the cut lies at a
    bin boundary (many equal values, top-k off)."""
    V, n = 65536, 64
    x = logits_rows(n, V, 21)
    x[: n // 2] = np.round(x[: n // 2] * 4) / 4            # few distinct values: cuts fall between whole groups
    u = np.random.default_rng(22).random((n, 2)).astype(np.float32)
    xs, us = torch.from_numpy(x).cuda(), torch.from_numpy(u).cuda()
    for top_p in (0.3, 0.9):
        first = k.sample(xs, us, temp=1.0, top_p=top_p).cpu().tolist()
        for _ in range(8):
            assert k.sample(xs, us, temp=1.0, top_p=top_p).cpu().tolist() == first
        for i in (0, n - 1):
            p = P.filtered_probs(x[i], 1.0, top_p=top_p)
            assert p[first[i]] > 0


def test_distribution_of_many_draws(k):
    V, n = 50, 4000
    row = logits_rows(1, V, 9, 1.5)
    x = np.repeat(row, n, axis=0)
    u = np.random.default_rng(10).random((n, 2)).astype(np.float32)
    got = k.sample(torch.from_numpy(x).cuda(), torch.from_numpy(u).cuda(), temp=0.9, top_k=12).cpu().numpy()
    p = P.filtered_probs(row[0], 0.9, top_k=12)
    freq = np.bincount(got, minlength=V) / n
    assert np.all(freq[p == 0] == 0) and np.abs(freq - p).max() < 0.03


def test_penalties_edit_the_listed_logits(k):
    V = 300
    x = logits_rows(3, V, 11)
    rep = np.full((3, 64), -1, dtype=np.int32)
    hist = [[5, 9, 5, 200], [1], []]
    for i, h in enumerate(hist):
        d = list(dict.fromkeys(h))
        rep[i, :len(d)] = d
    dry_t = np.full((3, 4), -1, dtype=np.int32)
    dry_p = np.zeros((3, 4), dtype=np.float32)
    dry_t[0, 0], dry_p[0, 0] = 9, 1.5
    dry_t[2, 1], dry_p[2, 1] = 7, 0.25
    dev = torch.from_numpy(x.copy()).cuda()
    k.apply_penalties(dev, torch.from_numpy(rep).cuda(), 1.3, torch.from_numpy(dry_t).cuda(), torch.from_numpy(dry_p).cuda())
    want = np.stack([P.repeat_penalty(x[i], hist[i], 1.3) for i in range(3)])
    want[0, 9] -= 1.5
    want[2, 7] -= 0.25
    assert np.allclose(dev.cpu().numpy(), want, rtol=1e-6, atol=1e-7)


def test_xtc_removes_the_top_choices_but_the_last(k):
    """Probabilities 0.4, 0.3, 0.2 reach the threshold 0.15: with the chance taken the first two
    go and the third stays with the tail (src/sampler.zig:244-268)."""
    V = 64
    p = np.full(V, 0.1 / (V - 3))
    p[[10, 3, 40]] = [0.4, 0.3, 0.2]
    x = np.log(p).astype(np.float32)[None].repeat(200, 0)
    u = np.random.default_rng(12).random((200, 2)).astype(np.float32)
    u[:100, 1] = 0.9          # chance not taken
    u[100:, 1] = 0.1          # chance taken
    got = k.sample(torch.from_numpy(x).cuda(), torch.from_numpy(u).cuda(), temp=1.0, xtc_probability=0.5,
                   xtc_threshold=0.15).cpu().numpy()
    assert {10, 3} & set(got[:100].tolist()) and not ({10, 3} & set(got[100:].tolist()))
    assert 40 in got[100:]
    kept = k.sample(torch.from_numpy(x).cuda(), torch.from_numpy(u).cuda(), temp=1.0, xtc_probability=0.5,
                    xtc_threshold=0.15, xtc_min_keep=V).cpu().numpy()
    assert {10, 3} & set(kept[100:].tolist()), "min_keep larger than what would stay: nothing is removed"


def test_uniforms_made_on_the_device_are_the_hosts(k):
    """Without uniforms the kernel computes them from (seed, request, the request's count of draws) as
    sampling.sampler.uniform does on the host, and advances the count of every request it drew for:
    the tokens equal those of the same rows with the host's uniforms, step after step, also when the
    rows are a changing subset of the requests and the seed uses all 64 bits."""
    from zinfer_b200.sampling.sampler import uniform
    V, n_req = 5000, 7
    seed = 0xF123456789ABCDEF
    draws_dev = torch.zeros(n_req, dtype=torch.int32, device="cuda")
    draws = [0] * n_req
    opts = dict(temp=0.9, top_k=50, top_p=0.9, min_p=0.02, xtc_probability=0.5, xtc_threshold=0.05)
    for step, rows in enumerate([[0, 1, 2, 3, 4, 5, 6], [6, 2, 4], [2], [0, 1, 2, 3, 4, 5, 6], [5, 0]]):
        x = torch.from_numpy(logits_rows(len(rows), V, 100 + step)).cuda()
        u = np.array([[uniform(seed, r, draws[r], 0), uniform(seed, r, draws[r], 1)] for r in rows], dtype=np.float32)
        want = k.sample(x, torch.from_numpy(u).cuda(), **opts).cpu().tolist()
        got = k.sample(x, None, seed=seed, req_ids=torch.tensor(rows, dtype=torch.int32).cuda(), draws=draws_dev,
                       **opts).cpu().tolist()
        assert got == want, f"step {step}: {got} != {want}"
        for r in rows:
            draws[r] += 1
        assert draws_dev.cpu().tolist() == draws


@pytest.mark.parametrize("opts", [dict(temp=1.0, top_p=0.9), dict(temp=0.7, min_p=0.02), dict(temp=1.2, top_p=0.8, min_p=0.01),
                                  dict(temp=0.9, top_k=1024, top_p=0.95), dict(temp=0.9, top_k=1025, top_p=0.95),
                                  dict(temp=1.0, top_k=3000)])
@pytest.mark.parametrize("scale", [8.0, 1.0])
def test_short_list_and_whole_row_give_the_plain_chain(k, opts, scale):
    """Peaked rows (scale 8: the survivors of top-p and min-p lie among the 1,024 best, so the chain
    runs on the short list) and flat rows (scale 1: they do not, and the passes over the whole row
    take over), top-k at and beyond the list's length: the draws are the plain implementation's."""
    n, V = 32, 65536
    x = logits_rows(n, V, 77, scale)
    x[3, 100] = np.nan
    u = np.random.default_rng(5).random((n, 2)).astype(np.float32)
    xs, us = torch.from_numpy(x).cuda(), torch.from_numpy(u).cuda()
    got = k.sample(xs, us, **opts).cpu().numpy()
    assert np.array_equal(got, k.sample(xs, us, **opts).cpu().numpy()), "two runs differ"
    exact = 0
    for i in range(n):
        row = np.where(np.isnan(x[i]), -np.inf, x[i])
        p = P.filtered_probs(row, opts["temp"], opts.get("top_k", 0), opts.get("top_p", 1.0), opts.get("min_p", 0.0))
        assert p[got[i]] > 0, f"row {i}: token {got[i]} is outside the support"
        exact += int(got[i] == expected_pick(p, float(u[i, 0])))
    assert exact >= n - 1, f"only {exact} of {n} draws equal the plain implementation's"


def test_more_ties_than_the_short_list_holds(k):
    """2,000 tokens share the value at which top-k cuts: the deciding bin holds more than the short list
    can, the passes over the whole row decide, and the cut still falls in index order."""
    V = 6000
    x = np.full((2, V), -3.0, dtype=np.float32)
    x[:, 1000:3000] = 1.5
    x[:, 4000] = 2.5
    u = np.array([[0.9999, 0], [0.0, 0]], dtype=np.float32)
    got = k.sample(torch.from_numpy(x).cuda(), torch.from_numpy(u).cuda(), temp=1.0, top_k=5).cpu().tolist()
    assert got == [4000, 1000]          # the survivors are 4000 and 1000..1003; the draw walks them in index order
    got = k.sample(torch.from_numpy(x).cuda(), torch.from_numpy(np.array([[0.5, 0], [0.7, 0]], dtype=np.float32)).cuda(),
                   temp=1.0, top_k=5).cpu().tolist()
    assert set(got) <= {1000, 1001, 1002, 1003, 4000}


def test_repetition_penalty_from_the_window_on_the_device(k):
    """The device keeps each request's last 64 tokens as a ring: tokens appended one by one (more than
    64 of them, with repeats) and the penalty read from the ring equal the plain implementation's
    penalty on the host's history, for rows that are a changing subset of the requests."""
    W = k.recent_window()
    V, n_req = 500, 4
    rng = np.random.default_rng(9)
    recent = torch.full((n_req, W), -1, dtype=torch.int32, device="cuda")
    seen = torch.zeros(n_req, dtype=torch.int32, device="cuda")
    hist = [[] for _ in range(n_req)]
    for step in range(150):
        rows = sorted(rng.choice(n_req, size=rng.integers(1, n_req + 1), replace=False).tolist())
        toks = rng.integers(0, 40, size=len(rows)).astype(np.int32)          # few values: many repeats
        req = torch.tensor(rows, dtype=torch.int32).cuda()
        if step % 10 == 9:
            x = logits_rows(len(rows), V, 300 + step)
            dev = torch.from_numpy(x).cuda()
            k.penalize_recent(dev, recent, seen, req, 1.3)
            want = np.stack([P.repeat_penalty(x[i], hist[r], 1.3) if hist[r] else x[i] for i, r in enumerate(rows)])
            assert np.array_equal(dev.cpu().numpy(), want), f"step {step}"
        k.recent_append(torch.from_numpy(toks).cuda(), recent, seen, req)
        for r, t in zip(rows, toks.tolist()):
            hist[r].append(t)
    assert seen.cpu().tolist() == [len(h) for h in hist] and max(len(h) for h in hist) > W
