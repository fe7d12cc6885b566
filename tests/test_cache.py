"""The cache's bookkeeping on the host: slots and pages are never lost, held twice or freed
twice; groups have storage of their own; a window gives pages back; errors change nothing."""
import numpy as np
import pytest
import torch

from zinfer_b200.cache import CacheError, CacheManager, CallCacheSpec, ContextFull, NoFreeSlot, OutOfPages
from zinfer_b200.parts.base import KVRequest, StateRequest

FULL = KVRequest(2, 16, 0)
WIN = KVRequest(2, 16, 40)
STATE = StateRequest((2, 8))


def make(calls=None, max_slots=4, max_tokens=256, max_seq_len=128, page=16):
    if calls is None:
        calls = [CallCacheSpec(state=STATE), CallCacheSpec(kv=FULL), CallCacheSpec(state=STATE), CallCacheSpec(kv=FULL)]
    return CacheManager(calls, max_slots, max_tokens, max_seq_len, page, torch.float32, "cpu")


def test_groups_have_their_own_storage():
    calls = [CallCacheSpec(kv=WIN), CallCacheSpec(state=STATE), CallCacheSpec(kv=FULL), CallCacheSpec(kv=WIN),
             CallCacheSpec(kv=FULL, kv_owner=2), CallCacheSpec(state=StateRequest((3,)))]
    c = make(calls)
    assert len(c.groups) == 2
    assert c.groups[0].k.shape == (2, 16, 2, 16, 16) and c.groups[1].k.shape == (1, 16, 2, 16, 16)
    assert c.kv_view(0).group == c.kv_view(3).group != c.kv_view(2).group
    assert c.kv_view(0).k.data_ptr() != c.kv_view(3).k.data_ptr()
    assert c.kv_view(4).k.data_ptr() == c.kv_view(2).k.data_ptr()      # reads call 2's cache
    assert c.writes_kv(2) and not c.writes_kv(4) and c.kv_view(1) is None
    assert c.state_view(1).shape == (4, 2, 8) and c.state_view(5).shape == (4, 3) and c.state_view(0) is None
    assert len(c.state_tensors) == 2


def test_reading_a_cache_that_nobody_owns_is_refused():
    with pytest.raises(CacheError, match="owns none"):
        make([CallCacheSpec(state=STATE), CallCacheSpec(kv=FULL, kv_owner=0)])
    with pytest.raises(CacheError, match="different layout"):
        make([CallCacheSpec(kv=FULL), CallCacheSpec(kv=WIN, kv_owner=0)])


def test_slots_and_pages_go_round():
    c = make()
    a = c.alloc_slots(3)
    assert sorted(a) == [0, 1, 2] and c.free_slot_count() == 1
    c.reserve(a, [5, 17, 64])
    c.advance(a, [5, 17, 64])
    assert [len(c.groups[0].pages_held(s)) for s in a] == [1, 2, 4]
    assert c.free_page_count() == [16 - 7]
    c.check_consistency()
    c.reserve([a[0]], [12])            # 5 + 12 = 17 -> one more page
    c.advance([a[0]], [12])
    assert len(c.groups[0].pages_held(a[0])) == 2 and int(c.lengths[a[0]]) == 17
    held = set(c.groups[0].pages_held(a[1]))
    c.free_slots([a[1]])
    assert c.free_page_count() == [16 - 6] and c.free_slot_count() == 2
    b = c.alloc_slots(2)
    assert a[1] in b and int(c.lengths[a[1]]) == 0 and c.groups[0].pages_held(a[1]) == []
    c.reserve([a[1]], [20])
    assert set(c.groups[0].pages_held(a[1])) & held, "freed pages are used again"
    c.check_consistency()
    c.free_slots([a[0], a[2]] + b)
    assert c.free_page_count() == [16] and c.free_slot_count() == 4
    assert (c.groups[0].table_host == -1).all()
    c.check_consistency()


def test_double_free_and_unknown_slot_raise():
    c = make()
    s = c.alloc_slots(2)
    c.free_slots([s[0]])
    with pytest.raises(CacheError, match="not held"):
        c.free_slots([s[0]])
    with pytest.raises(CacheError, match="twice"):
        c.free_slots([s[1], s[1]])
    with pytest.raises(CacheError, match="not held"):
        c.free_slots([7])
    with pytest.raises(CacheError, match="not held"):
        c.reserve([s[0]], [1])
    c.check_consistency()


def test_capacity_errors_change_nothing():
    c = make(max_slots=3, max_tokens=64, max_seq_len=48)
    with pytest.raises(NoFreeSlot):
        c.alloc_slots(4)
    assert c.free_slot_count() == 3
    s = c.alloc_slots(3)
    c.reserve(s[:2], [30, 16])
    before = (c.free_page_count(), c.groups[0].table_host.copy())
    with pytest.raises(OutOfPages):
        c.reserve([s[2], s[1]], [17, 1])         # needs 2 + 1 pages, 1 is free
    with pytest.raises(ContextFull):
        c.reserve([s[2], s[0]], [1, 49])
    assert c.free_page_count() == before[0] and np.array_equal(c.groups[0].table_host, before[1])
    c.check_consistency()


def test_state_rows_are_zeroed_when_a_slot_is_handed_out():
    c = make()
    for st in c.state_tensors:
        st.fill_(7.0)
    s = c.alloc_slots(2)
    st = c.state_view(0)
    assert (st[s] == 0).all() and (st[[x for x in range(4) if x not in s]] == 7).all()
    st[s[0]] = 3.0
    c.free_slots([s[0]])
    again = c.alloc_slots(1)
    assert again == [s[0]] and (c.state_view(0)[s[0]] == 0).all() and (c.state_view(2)[s[0]] == 0).all()


def test_window_group_gives_pages_back_and_full_group_keeps_them():
    calls = [CallCacheSpec(kv=WIN), CallCacheSpec(kv=FULL)]
    c = make(calls, max_slots=2, max_tokens=256, max_seq_len=256)
    win, full = c.groups
    s = c.alloc_slots(1)[0]
    c.reserve([s], [100])
    assert len(win.pages_held(s)) == 7                 # the whole prompt is needed during its step
    c.advance([s], [100])
    # the next query stands at 100 and sees keys 61..100: pages 0..2 (positions 0..47) can go
    assert len(win.pages_held(s)) == 4 and (win.table_host[s, :3] == -1).all() and win.table_host[s, 3] >= 0
    assert len(full.pages_held(s)) == 7
    for _ in range(60):
        c.reserve([s], [1])
        c.advance([s], [1])
    assert len(full.pages_held(s)) == 10 and len(win.pages_held(s)) <= 4
    c.check_consistency()
    c.free_slots([s])
    assert c.free_page_count() == [16, 16]
    c.check_consistency()


def test_random_walk_never_loses_anything():
    rng = np.random.default_rng(0)
    calls = [CallCacheSpec(kv=WIN), CallCacheSpec(kv=FULL), CallCacheSpec(state=STATE)]
    c = make(calls, max_slots=5, max_tokens=320, max_seq_len=200)
    live = []
    for _ in range(400):
        op = rng.integers(0, 3)
        try:
            if op == 0:
                live += c.alloc_slots(int(rng.integers(1, 3)))
            elif op == 1 and live:
                pick = [s for s in live if rng.random() < 0.6] or live[:1]
                n = [int(rng.integers(1, 40)) for _ in pick]
                c.reserve(pick, n)
                c.advance(pick, n)
            elif op == 2 and live:
                s = live.pop(int(rng.integers(0, len(live))))
                c.free_slots([s])
        except (NoFreeSlot, OutOfPages, ContextFull):
            pass
        c.check_consistency()
        for g in c.groups:
            for s in live:
                need = -(-int(c.lengths[s]) // 16)
                assert g.n_pages_of[s] >= need
    c.free_slots(live)
    assert c.free_page_count() == [20, 20] and c.free_slot_count() == 5
