"""The cache manager's host side: no page is lost, held twice or freed twice,
under random orders of requests; windows give pages back; the prefix tree
shares and evicts.  No GPU."""

import random

import pytest

from ullm_b200.cache import CacheManager, OutOfPages, PageAllocator, PrefixTree, SlotAllocator, plan_groups
from ullm_b200.parts import CacheNeed, StateNeed

FULL = CacheNeed(2, 16, None)
WIN = CacheNeed(2, 16, 24)


def manager(needs, num_pages=16, page=4, max_requests=4, per_request=16, prefix=True):
    return CacheManager(needs, page, num_pages, max_requests, per_request, device=None, enable_prefix_cache=prefix)


def test_page_allocator_refuses_double_free():
    a = PageAllocator(4)
    p = a.alloc(3)
    assert a.alloc(2) is None and a.num_free == 1
    a.free(p[:2])
    with pytest.raises(ValueError, match="freed twice"):
        a.free(p[:1])
    with pytest.raises(ValueError, match="not of this pool"):
        a.free([9])
    s = SlotAllocator(2)
    x, y = s.alloc(), s.alloc()
    assert s.alloc() is None
    s.free(x)
    with pytest.raises(ValueError, match="twice"):
        s.free(x)


def test_groups_by_need_and_shared_caches():
    needs = [(FULL, None, None), (WIN, None, None), (FULL, None, None), (FULL, None, 0), (None, StateNeed((3,)), None)]
    groups, where = plan_groups(needs)
    assert [g.executions for g in groups] == [[0, 2], [1]]
    assert where == [(0, 0), (1, 0), (0, 1), (0, 0), None]
    with pytest.raises(ValueError, match="different geometry"):
        plan_groups([(FULL, None, None), (CacheNeed(1, 16, None), None, 0)])


def test_reserve_commit_release_and_slot_mapping():
    m = manager([(FULL, None, None)], prefix=False)
    rc = m.admit("a")
    m.reserve(rc, 6)
    assert len(rc.pages[0]) == 2 and m.num_free_pages() == 14
    sm = m.slot_mapping(rc, 0, 6)
    assert sm == [rc.pages[0][0] * 4 + i for i in range(4)] + [rc.pages[0][1] * 4, rc.pages[0][1] * 4 + 1]
    m.commit(rc, 6)
    m.reserve(rc, 2)  # fits the second page
    assert len(rc.pages[0]) == 2
    m.commit(rc, 2)
    m.reserve(rc, 1)
    assert len(rc.pages[0]) == 3
    m.check_invariants()
    m.release(rc)
    assert m.num_free_pages() == 16
    with pytest.raises(ValueError, match="not live"):
        m.release(rc)


def test_out_of_pages_is_all_or_nothing():
    m = manager([(FULL, None, None), (WIN, None, None)], num_pages=3, prefix=False)
    rc = m.admit("a")
    with pytest.raises(OutOfPages):
        m.reserve(rc, 13)
    assert rc.pages == [[], []] and m.num_free_pages(0) == 3 and m.num_free_pages(1) == 3
    assert not m.can_reserve(rc, 13) and m.can_reserve(rc, 12)
    m.check_invariants()


def test_window_gives_pages_back_as_it_passes():
    m = manager([(WIN, None, None)], num_pages=10, page=4, per_request=64, prefix=False)
    rc = m.admit("a")
    held = []
    for step in range(100):
        m.reserve(rc, 1)
        m.commit(rc, 1)
        live = [p for p in rc.pages[0] if p >= 0]
        held.append(len(live))
        # every position the next token can see is on a live page
        lo = max(0, rc.num_tokens - 24 + 1)
        for pos in range(lo, rc.num_tokens):
            assert rc.pages[0][pos // 4] >= 0
        m.check_invariants()
    assert max(held) <= 24 // 4 + 2, "a windowed request holds about window/page_size pages"
    m.release(rc)
    assert m.num_free_pages() == 10


def test_prefix_tree_shares_full_pages_and_evicts_lru():
    m = manager([(FULL, None, None)], num_pages=8, page=4)
    toks = list(range(100, 114))  # 14 tokens: 3 full pages + 2
    a = m.admit("a", toks)
    assert a.num_cached_tokens == 0
    m.reserve(a, 14)
    m.commit(a, 14)
    pages_a = list(a.pages[0])
    m.release(a, toks)
    assert m.tree.num_pages == 3 and m.num_free_pages() == 5
    b = m.admit("b", toks[:12] + [7, 8])
    assert b.num_cached_tokens == 8 or b.num_cached_tokens == 12
    assert b.pages[0] == pages_a[: b.num_cached_tokens // 4]
    # at least one token is left to compute even on a full match
    c = m.admit("c", toks[:12])
    assert c.num_cached_tokens == 8
    m.check_invariants()
    m.reserve(b, 14 - b.num_cached_tokens)
    m.commit(b, 14 - b.num_cached_tokens)
    m.release(b, toks[:12] + [7, 8])
    m.release(c)
    m.check_invariants()
    # eviction on demand: a request that needs every page gets them
    d = m.admit("d")
    m.reserve(d, 32)
    assert m.tree.num_pages == 0 and m.num_free_pages() == 0
    m.check_invariants()
    m.release(d)
    assert m.num_free_pages() == 8


def test_available_pages_do_not_walk_the_prefix_tree():
    """`num_available_pages` is asked for every running request in every step: with thousands of pages in the
    prefix tree it must not visit them (a walk per call made a decode step of 48 requests take 57 ms)."""
    import time

    m = manager([(FULL, None, None)], num_pages=6000, page=4, per_request=128)
    for r in range(50):  # 50 finished requests of 100 pages each, no common prefix
        toks = [r * 1000 + i for i in range(400)]
        a = m.admit(f"r{r}", toks)
        m.reserve(a, 400)
        m.commit(a, 400)
        m.release(a, toks)
    assert m.tree.num_pages == 5000
    live = m.admit("live", [7 * 1000 + i for i in range(400)])  # holds 99 of the tree's pages
    assert m.tree.num_evictable() == m.tree.count_evictable_by_walk() == 5000 - len(live.prefix_nodes)
    t0 = time.perf_counter()
    for _ in range(2000):
        m.num_available_pages(0)
    assert time.perf_counter() - t0 < 0.05, "2,000 calls took longer than 50 ms"
    m.release(live)
    m.check_invariants()


def test_eviction_queue_does_not_grow_without_evictions():
    """A pool with room to spare never evicts; the queue of eviction candidates must not grow with every request
    that finishes (it is rebuilt from the tree when stale entries pile up), and eviction still takes the least
    recently used pages first afterwards."""
    m = manager([(FULL, None, None)], num_pages=64, page=4, per_request=16)
    toks = {r: [r * 100 + i for i in range(16)] for r in range(3)}
    for _ in range(2000):
        for r in (0, 1, 2):
            a = m.admit(f"r{r}", toks[r])
            need = 16 - a.num_tokens
            m.reserve(a, need)
            m.commit(a, need)
            m.release(a, toks[r])
    assert m.tree.num_pages == 12
    assert len(m.tree._heap) <= 4 * m.tree.num_pages + 1024 + 8
    m.check_invariants()
    # request 0 was released first in every round: its last page is the least recently used leaf
    chain0 = m.tree.match(toks[0], 4)
    assert len(chain0) == 4
    assert m.tree.evict(1) == [chain0[-1].page]


def test_two_fresh_requests_with_one_prefix_leak_nothing():
    """The reference loses the second request's duplicate slots here
    (ullm/core/kv_cache.py:379: freed only when old_prefix_len != 0)."""
    m = manager([(FULL, None, None)], num_pages=8, page=4)
    toks = list(range(8))
    a, b = m.admit("a", toks + [1]), m.admit("b", toks + [2])
    for rc in (a, b):
        m.reserve(rc, 9)
        m.commit(rc, 9)
    m.release(a, toks + [1])
    m.release(b, toks + [2])
    m.check_invariants()
    assert m.tree.num_pages == 2 and m.num_free_pages() == 6


@pytest.mark.parametrize("seed", range(12))
@pytest.mark.parametrize("needs", [
    [(FULL, None, None)],
    [(FULL, None, None), (WIN, None, None), (FULL, None, None)],
    [(WIN, None, None), (FULL, StateNeed((2,)), None)],
])
def test_random_orders_keep_the_accounting(seed, needs):
    rng = random.Random(seed)
    page = rng.choice([1, 4, 16])
    m = manager(needs, num_pages=rng.randint(6, 24), page=page, max_requests=4, per_request=64)
    vocab = 5  # small, so prefixes collide
    live: dict[str, list[int]] = {}
    n = 0
    for _ in range(300):
        op = rng.random()
        if op < 0.3 and len(live) < 4:
            n += 1
            toks = [rng.randrange(vocab) for _ in range(rng.randint(1, 40))]
            rc = m.admit(f"r{n}", toks)
            assert rc is not None
            live[f"r{n}"] = toks
            assert rc.num_tokens == rc.num_cached_tokens < max(len(toks), 1) or rc.num_tokens == 0
        elif op < 0.8 and live:
            rid = rng.choice(list(live))
            rc = m.requests[rid]
            want = rng.randint(1, 9)
            left = len(live[rid]) - rc.num_tokens
            if left <= 0:
                live[rid].append(rng.randrange(vocab))
                left = 1
            k = min(want, left)
            if m.can_reserve(rc, k):
                m.reserve(rc, k)
                m.commit(rc, k)
            else:
                with pytest.raises(OutOfPages):
                    m.reserve(rc, k)
        elif live:
            rid = rng.choice(list(live))
            rc = m.requests[rid]
            m.release(rc, live[rid][: rc.num_tokens] if rng.random() < 0.7 else None)
            del live[rid]
        m.check_invariants()
    for rid in list(live):
        m.release(m.requests[rid], None)
    m.check_invariants()
    evict = m.tree.num_evictable() if m.tree is not None else 0
    for g in range(len(m.groups)):
        assert m.num_free_pages(g) + (evict if g == 0 else 0) == m.num_pages
    assert m.slots.num_free == 4
