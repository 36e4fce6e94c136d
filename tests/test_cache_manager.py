"""The page allocator and the cache manager: no page lost, held twice or freed twice, under random
orders of requests; windows give pages back; prefix sharing; state slots (CPU)."""

from __future__ import annotations

import random

import pytest
from hypothesis import given, settings
from hypothesis import strategies as st

from tokenmill_b200.cache import AllocStatus, CacheManager, OutOfPages, PageAllocator, chain_hash


def test_allocator_basics_and_double_free():
    a = PageAllocator(4)
    got = a.allocate(3)
    assert sorted(got) == [0, 1, 2] and a.num_free == 1
    with pytest.raises(OutOfPages):
        a.allocate(2)
    assert a.num_free == 1                         # a refused request changes nothing
    a.release([got[1]])
    with pytest.raises(RuntimeError, match="double free"):
        a.release([got[1]])
    assert a.allocate(1) == [got[1]]               # the page released last is reused first
    a.check_invariants()


@settings(max_examples=200, deadline=None)
@given(st.lists(st.tuples(st.booleans(), st.integers(0, 6)), max_size=80), st.integers(1, 12))
def test_allocator_random_ops_never_lose_or_double_a_page(ops, n):
    a = PageAllocator(n)
    held: list[int] = []
    for is_alloc, k in ops:
        if is_alloc:
            if k > a.num_free:
                with pytest.raises(OutOfPages):
                    a.allocate(k)
            else:
                got = a.allocate(k)
                assert not set(got) & set(held) and len(set(got)) == len(got)
                held += got
        elif held:
            k = min(k, len(held))
            random.Random(k).shuffle(held)
            a.release(held[:k])
            held = held[k:]
        a.check_invariants()
        assert a.num_free + len(held) == n


def test_allocator_caching_revive_and_evict_lru():
    evicted = []
    a = PageAllocator(3, enable_caching=True, on_evict=evicted.append)
    p = a.allocate(3)
    a.mark_cached(p[0])
    a.mark_cached(p[1])
    a.release([p[0]])
    a.release([p[1]])
    a.release([p[2]])
    assert a.num_free == 3
    a.share(p[0])                                   # revive from the evictable list
    assert a.refcount[p[0]] == 1 and a.num_free == 2
    assert a.allocate(1) == [p[2]]                  # plain free pages go first
    assert a.allocate(1) == [p[1]] and evicted == [p[1]]
    a.release([p[2]])                               # never published: it is plainly free now
    with pytest.raises(RuntimeError, match="free, not cached"):
        a.share(p[2])
    a.check_invariants()


def _tokens(n, seed=0):
    rng = random.Random(seed)
    return [rng.randrange(1000) for _ in range(n)]


def test_manager_admission_growth_release():
    m = CacheManager(8, page_size=4, watermark=0.25)              # watermark: 2 pages kept back
    h = m.new_handle()
    assert m.admission_status(h, _tokens(40)) == AllocStatus.NEVER    # 10 pages can never fit
    assert m.admission_status(h, _tokens(28)) == AllocStatus.NEVER    # 7 + 2 > 8
    assert m.admission_status(h, _tokens(24)) == AllocStatus.OK       # 6 pages, 2 left
    assert m.allocate(h, _tokens(24)) == 0
    assert [len(t) for t in h.tables] == [6] and m.num_free_pages == 2
    h2 = m.new_handle()
    assert m.admission_status(h2, _tokens(4)) == AllocStatus.LATER     # 1 page would leave 1 < 2
    assert m.slot(h, 0, 13) == h.tables[0][3] * 4 + 1
    assert m.can_grow(h, 24) and m.can_grow(h, 32) and not m.can_grow(h, 33)
    m.grow(h, 25)
    assert len(h.tables[0]) == 7
    with pytest.raises(OutOfPages):
        m.grow(h, 40)
    m.free(h)
    assert m.all_free
    with pytest.raises(RuntimeError):
        m.allocators[0].release([0])
    m.check_invariants()


def test_manager_groups_have_tables_of_their_own_and_windows_give_pages_back():
    m = CacheManager([10, 10], page_size=4, windows=[None, 6], watermark=0.0)
    h = m.new_handle()
    m.allocate(h, _tokens(20))
    assert [len(t) for t in h.tables] == [5, 5]
    assert m.release_behind_window(h, 5) == 0        # keys >= 0 still readable: 5 - 6 + 1 = 0
    assert m.release_behind_window(h, 13) == 2       # future queries read keys >= 8: pages 0, 1 go
    assert h.tables[1][:2] == [-1, -1] and all(p >= 0 for p in h.tables[0])
    assert m.allocators[1].num_free == 7 and m.allocators[0].num_free == 5
    assert m.release_behind_window(h, 13) == 0       # nothing is released twice
    with pytest.raises(RuntimeError, match="given back"):
        m.slot(h, 1, 3)
    m.grow(h, 24)
    assert [len(t) for t in h.tables] == [6, 6]
    m.free(h)
    assert m.all_free
    m.check_invariants()


def test_manager_prefix_sharing_and_hashes():
    m = CacheManager(12, page_size=4, watermark=0.0, enable_prefix_caching=True)
    toks = _tokens(18)
    a, b = m.new_handle(), m.new_handle()
    assert m.allocate(a, toks) == 0
    m.register_computed(a, toks, 18)                 # pages 0..3 are full and published
    assert a.num_registered_pages == 4
    other = toks[:9] + _tokens(9, seed=5)
    assert m.allocate(b, other) == 8                 # two full pages shared, the third differs
    assert b.tables[0][:2] == a.tables[0][:2] and b.tables[0][2] != a.tables[0][2]
    assert m.allocators[0].refcount[a.tables[0][0]] == 2
    assert m.prefix_hit_tokens == 8 and m.prefix_query_tokens == 36
    # an exact repeat still computes its last token: (18 - 1) // 4 = 4 pages reusable
    c = m.new_handle()
    assert m.allocate(c, toks) == 16
    m.free(a)
    m.free(b)
    m.free(c)
    assert m.all_free                                # published pages count as free (evictable)
    d = m.new_handle()
    assert m.allocate(d, toks) == 16                 # revived from the evictable list
    m.free(d)
    m.check_invariants()
    assert chain_hash(None, [1, 2]) != chain_hash(0, [1, 2]) and chain_hash(5, [1, 2]) == chain_hash(5, [1, 2])


def test_prefix_caching_is_off_when_a_group_has_a_window_or_state():
    assert not CacheManager([4, 4], 4, windows=[None, 8], enable_prefix_caching=True).enable_prefix_caching
    assert not CacheManager(4, 4, enable_prefix_caching=True, num_state_slots=2).enable_prefix_caching


def test_state_slots_follow_the_request():
    m = CacheManager(8, page_size=4, watermark=0.0, num_state_slots=2)
    a, b, c = m.new_handle(), m.new_handle(), m.new_handle()
    m.allocate(a, _tokens(3))
    m.allocate(b, _tokens(3))
    assert {a.state_slot, b.state_slot} == {0, 1} and a.fresh_state
    assert m.admission_status(c, _tokens(3)) == AllocStatus.LATER      # pages there, no slot
    with pytest.raises(OutOfPages):
        m.allocate(c, _tokens(3))
    assert not c.holds_pages
    m.free(a)
    assert a.state_slot == -1 and m.admission_status(c, _tokens(3)) == AllocStatus.OK
    m.allocate(c, _tokens(3))
    m.free(b)
    m.free(c)
    assert m.all_free
    m.check_invariants()


@settings(max_examples=60, deadline=None)
@given(st.integers(0, 10 ** 6), st.booleans(), st.booleans())
def test_manager_random_request_orders_conserve_pages(seed, caching, windowed):
    rng = random.Random(seed)
    windows = [None, 10] if windowed else [None]
    m = CacheManager([24] * len(windows), page_size=4, windows=windows, watermark=0.0,
                     enable_prefix_caching=caching)
    shared = _tokens(16, seed=1)
    live: list[tuple] = []
    for _ in range(60):
        op = rng.random()
        if op < 0.4 or not live:
            toks = (shared[:rng.choice([0, 8, 16])] + _tokens(rng.randrange(1, 30), seed=rng.randrange(99)))
            h = m.new_handle()
            if m.admission_status(h, toks) == AllocStatus.OK:
                done = m.allocate(h, toks)
                assert done % 4 == 0 and done < len(toks)
                live.append((h, toks, done))
        elif op < 0.7:
            i = rng.randrange(len(live))
            h, toks, done = live[i]
            if done < len(toks):
                done = min(len(toks), done + rng.randrange(1, 9))
            elif m.can_grow(h, len(toks) + 1):
                toks = toks + [rng.randrange(1000)]
                m.grow(h, len(toks))
                done = len(toks)
            m.register_computed(h, toks, done)
            m.release_behind_window(h, done)
            live[i] = (h, toks, done)
        else:
            h, _, _ = live.pop(rng.randrange(len(live)))
            m.free(h)
        m.check_invariants()
        for g, alloc in enumerate(m.allocators):
            refs: dict[int, int] = {}
            for h, _, _ in live:
                for p in h.tables[g]:
                    if p >= 0:
                        refs[p] = refs.get(p, 0) + 1
            assert all(alloc.refcount[p] == n for p, n in refs.items())          # held exactly as tables say
            assert sum(1 for r in alloc.refcount if r > 0) == len(refs)           # nothing held by nobody
            if not caching:
                assert all(n == 1 for n in refs.values())                         # no page held twice
    for h, _, _ in live:
        m.free(h)
    assert m.all_free
