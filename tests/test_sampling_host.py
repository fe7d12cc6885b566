"""Host side of sampling: the counter-based random numbers, the distinct recent tokens, and the
DRY penalties against a brute-force search for repeated endings."""
import numpy as np

from zinfer_b200.sampling import SamplingParams, dry_penalties, recent_distinct, uniform


def test_uniforms_depend_only_on_their_arguments():
    a = [uniform(7, r, d, 0) for r in range(4) for d in range(50)]
    assert a == [uniform(7, r, d, 0) for r in range(4) for d in range(50)]
    assert all(0.0 <= x < 1.0 for x in a) and len(set(a)) > 190
    assert abs(np.mean(a) - 0.5) < 0.08
    assert uniform(7, 1, 2, 0) != uniform(8, 1, 2, 0) != uniform(7, 2, 1, 0) != uniform(7, 1, 2, 1)


def test_recent_distinct_is_the_last_64_each_once():
    h = list(range(100)) + [5, 99, 5]
    d = recent_distinct(h)
    assert d == list(range(39, 100)) + [5] and len(set(d)) == len(d)


def brute_dry(history, p, breakers=()):
    """For every earlier position k whose preceding tokens repeat the text's ending for n >= allowed
    tokens (not crossing a breaker), the token at k is penalised with the longest such n."""
    h = list(history)[-p.dry_range:]
    L = len(h)
    if L <= p.dry_allowed_length:
        return {}
    limit = L
    for k in range(L):
        if h[L - 1 - k] in breakers:
            limit = k
            break
    if limit < p.dry_allowed_length:
        return {}
    best = {}
    for k in range(1, L):               # h[k] is the continuation candidate; the match ends at k-1
        n = 0
        while n < min(k, limit) and n < L - (L - k) - 0 and h[k - 1 - n] == h[L - 1 - n]:
            n += 1
        if n >= p.dry_allowed_length and h[k] not in breakers:
            best[h[k]] = max(best.get(h[k], 0), n)
    return {t: p.dry_multiplier * p.dry_base ** (n - p.dry_allowed_length) for t, n in best.items()}


def test_dry_penalties_match_brute_force():
    p = SamplingParams(dry_multiplier=0.8, dry_base=1.75, dry_allowed_length=2, dry_range=64)
    rng = np.random.default_rng(0)
    for trial in range(200):
        h = rng.integers(0, 4, size=int(rng.integers(3, 40))).tolist()
        breakers = (3,) if trial % 3 == 0 else ()
        got = dry_penalties(h, p, breakers)
        want = brute_dry(h, p, breakers)
        assert got.keys() == want.keys(), (h, got, want)
        assert all(abs(got[t] - want[t]) < 1e-9 for t in got), (h, got, want)
    assert dry_penalties([1, 2, 3], SamplingParams(), ()) == {}          # multiplier 0 = off
    assert dry_penalties([1, 2, 3, 9, 1, 2, 3], p) == {9: 0.8 * 1.75}    # ending "1 2 3" seen before, then 9
