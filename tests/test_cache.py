"""The cache's bookkeeping: no page or slot lost, held twice or freed twice."""
import random

import pytest

from exl3_server_b200.cache import CacheError, CacheFull, PagePool, SequenceCache, SlotTable
from exl3_server_b200.parts import KVRequest, StateRequest


def make_cache(max_tokens=64 * 10, window=0, mixed=False, **kw):
    reqs = [(KVRequest(2, 16, window if (mixed and i % 2 == 0) or (not mixed and window) else 0), None, None)
            for i in range(4)]
    return SequenceCache(reqs, max_tokens, allocate=False, **kw)


def test_page_pool_alloc_free_and_reuse():
    p = PagePool(4)
    a = p.alloc(3)
    assert a == [0, 1, 2] and p.n_free == 1
    p.free([1])
    assert p.alloc(1) == [1]                    # the page given back last is used next
    with pytest.raises(CacheFull):
        p.alloc(2)
    assert p.n_free == 1                        # a refused request takes nothing
    p.check()


def test_page_pool_refuses_double_free_and_strangers():
    p = PagePool(4)
    a = p.alloc(2)
    p.free(a)
    with pytest.raises(CacheError, match="not held"):
        p.free([a[0]])
    with pytest.raises(CacheError, match="not held"):
        p.free([3])
    with pytest.raises(CacheError, match="not held"):
        p.free([99])
    b = p.alloc(1)
    with pytest.raises(CacheError):
        p.free([b[0], b[0]])
    p.check() if p.n_held == 0 else None


def test_slot_table():
    s = SlotTable(3)
    a, b, c = s.alloc(), s.alloc(), s.alloc()
    assert sorted([a, b, c]) == [0, 1, 2]
    with pytest.raises(CacheFull):
        s.alloc()
    s.free(b)
    with pytest.raises(CacheError, match="not live"):
        s.free(b)
    assert s.alloc() == b                       # used again
    s.check()


def test_sequences_grow_in_pages_and_give_them_back():
    c = make_cache(max_tokens=64 * 6)
    a, b = c.open(), c.open()
    c.reserve({a: 65, b: 1})
    c.commit(a, 65)
    c.commit(b, 1)
    assert c.tokens_held() == 128 + 64
    assert c.groups[0].pool.n_held == 3
    c.check()
    with pytest.raises(CacheFull):
        c.reserve({a: 64 * 3 + 1, b: 64 * 2 + 1})   # 4 + 3 pages wanted, 6 exist
    assert c.groups[0].pool.n_held == 3         # all or nothing
    c.close(a)
    assert c.groups[0].pool.n_held == 1
    with pytest.raises(CacheError, match="not live"):
        c.close(a)
    with pytest.raises(CacheError, match="not live"):
        c.length(a)
    again = c.open()
    assert again == a and c.length(again) == 0  # the slot is used again, empty
    c.close(b)
    c.close(again)
    c.check()
    assert c.tokens_held() == 0 and c.groups[0].pool.n_free == 6


def test_groups_by_need_have_their_own_storage():
    c = make_cache(window=32, mixed=True)
    assert len(c.groups) == 2
    assert sorted(len(g.owners) for g in c.groups) == [2, 2]
    assert {g.request.window for g in c.groups} == {0, 32}
    s = c.open()
    c.reserve({s: 200})
    c.commit(s, 200)
    full = next(g for g in c.groups if g.request.window == 0)
    win = next(g for g in c.groups if g.request.window == 32)
    assert [p >= 0 for p in full.pages[s]] == [True] * 4
    # keys below 200 - 32 + 1 = 169 are out of sight: pages 0 and 1 went back, page 2 holds 169..191
    assert [p >= 0 for p in win.pages[s]] == [False, False, True, True]
    assert win.pool.n_held == 2 and full.pool.n_held == 4
    c.check()
    c.close(s)
    c.check()
    assert win.pool.n_held == 0


def test_shared_cache_entries_own_nothing():
    reqs = [(KVRequest(2, 16), None, None), (KVRequest(2, 16), None, 0), (None, StateRequest((4,)), None)]
    c = SequenceCache(reqs, 256, allocate=False)
    assert c.entry_group[1] == c.entry_group[0] and not c.entry_owns[1] and c.entry_owns[0]
    assert c.entry_group[2] is None
    assert len(c.groups[0].owners) == 1
    with pytest.raises(CacheError, match="owns none"):
        SequenceCache([(KVRequest(2, 16), None, None), (KVRequest(2, 16), None, 0), (KVRequest(2, 16), None, 1)],
                      256, allocate=False)


def test_truncate():
    c = make_cache()
    s = c.open()
    c.reserve({s: 130})
    c.commit(s, 130)
    c.truncate(s, 64)
    assert c.length(s) == 64 and c.groups[0].pool.n_held == 1
    with pytest.raises(CacheError):
        c.truncate(s, 65)
    c.check()


def test_random_traffic_keeps_the_books():
    rng = random.Random(0)
    c = make_cache(max_tokens=64 * 40, window=100, mixed=True)
    live = {}
    for _ in range(2000):
        op = rng.random()
        if op < 0.25 and len(live) < 12:
            live[c.open()] = 0
        elif op < 0.45 and live:
            s = rng.choice(list(live))
            c.close(s)
            del live[s]
        elif live:
            s = rng.choice(list(live))
            n = live[s] + rng.choice([1, 1, 1, 7, 64, 130])
            try:
                c.reserve({s: n})
            except CacheFull:
                continue
            c.commit(s, n)
            live[s] = n
        c.check()
        assert c.tokens_held() == sum((n + 63) // 64 * 64 for n in live.values())
    for s in list(live):
        c.close(s)
    c.check()
    assert all(g.pool.n_held == 0 for g in c.groups) and c.slots.n_free == c.slots.n_slots


def test_a_reader_cannot_look_further_back_than_the_cache_it_reads_keeps():
    own = (KVRequest(2, 16, 32), None, None)
    SequenceCache([own, (KVRequest(2, 16, 32), None, 0)], 640, allocate=False)       # the same window: fine
    SequenceCache([own, (KVRequest(2, 16, 8), None, 0)], 640, allocate=False)        # a narrower one: fine
    SequenceCache([(KVRequest(2, 16, 0), None, None), (KVRequest(2, 16, 8), None, 0)], 640, allocate=False)
    with pytest.raises(CacheError, match="keeps only a window of 32"):
        SequenceCache([own, (KVRequest(2, 16, 0), None, 0)], 640, allocate=False)    # every key wanted
    with pytest.raises(CacheError, match="keeps only a window of 32"):
        SequenceCache([own, (KVRequest(2, 16, 64), None, 0)], 640, allocate=False)   # a wider window


def test_pages_leave_a_window_as_soon_as_no_query_can_see_them():
    c = SequenceCache([(KVRequest(2, 16, 100), None, None)], 64 * 8, allocate=False)
    # page 0 (keys 0..63) is last needed by the query at position 162, which sees keys 63..162; a sequence of
    # 163 tokens has its next query at position 163
    assert not c.gives_back_at(162)
    assert c.gives_back_at(163) and not c.gives_back_at(164)
    assert c.gives_back_at(227) and not c.gives_back_at(226)
    full = SequenceCache([(KVRequest(2, 16, 0), None, None)], 64 * 8, allocate=False)
    assert not any(full.gives_back_at(n) for n in range(1, 400))


def test_keys_and_values_of_different_widths_make_a_group_of_their_own():
    import torch
    reqs = [(KVRequest(2, 16), None, None), (KVRequest(2, 16, 0, value_dim=32), None, None),
            (KVRequest(2, 16, 0, value_dim=32), None, None)]
    c = SequenceCache(reqs, 640, dtype=torch.float32, device="cpu")
    assert len(c.groups) == 2 and [len(g.owners) for g in c.groups] == [1, 2]
    assert c.groups[0].k.shape[-1] == 16 and c.groups[0].v.shape[-1] == 16
    assert c.groups[1].k.shape[-1] == 16 and c.groups[1].v.shape[-1] == 32
    assert c.groups[0].bytes_per_token(4) == 2 * (16 + 16) * 4 and c.groups[1].bytes_per_token(4) == 2 * 2 * (16 + 32) * 4
    with pytest.raises(CacheError, match="head shapes differ"):
        SequenceCache([reqs[1], (KVRequest(2, 16), None, 0)], 640, allocate=False)


def test_guard_words_around_the_pools_show_a_stray_write():
    import torch
    c = SequenceCache([(KVRequest(2, 16), None, None)], 640, dtype=torch.float32, device="cpu")
    g = c.groups[0]
    c.check_guards()
    assert float(g.k.abs().sum()) == 0.0 and g.k.is_contiguous() and g.k.data_ptr() % 16 == 0
    g._v_store[-3] = 0.0                                   # what a write one page beyond the pool would do
    with pytest.raises(CacheError, match="guard words"):
        c.check_guards()
