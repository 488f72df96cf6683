"""Cache manager: no page lost, held twice or freed twice, under random orders of requests (no GPU)."""
import random

import pytest

from lucciola_b200.cache import NO_PAGE, CacheGroup, CacheManager, PagePool, PagePoolError, plan_groups
from lucciola_b200.parts import KVPages, StateSlot


def test_pool_fifo_and_errors():
    p = PagePool(3)
    assert [p.allocate() for _ in range(3)] == [0, 1, 2] and not p.can_allocate(1)
    with pytest.raises(PagePoolError, match="no free page"):
        p.allocate()
    p.free(1); p.free(0)
    assert p.allocate() == 1           # freed pages queue up behind: first freed, first reused
    with pytest.raises(PagePoolError, match="freed twice"):
        p.free(2); p.free(2)
    with pytest.raises(PagePoolError, match="not in the pool"):
        p.free(7)
    assert p.high_water == 3


def test_groups_from_cache_requests():
    reqs = [KVPages(2, 16), KVPages(2, 16, window=8), KVPages(2, 16), StateSlot((4,)), None, KVPages(1, 32)]
    groups, state_ids = plan_groups(reqs)
    assert [g.cache_ids for g in groups] == [(0, 2), (1,), (5,)] and state_ids == [3]
    assert [g.window for g in groups] == [0, 8, 0]


def _mgr(pages=10, page=4, window=0, slots=4):
    groups = [CacheGroup(2, 16, 0, (0,))] + ([CacheGroup(2, 16, window, (1,))] if window else [])
    return CacheManager(groups, page, pages, slots)


def test_extend_is_all_or_nothing_and_pages_return():
    m = _mgr(pages=5, page=4)
    m.admit("a"); m.admit("b")
    assert m.extend("a", 9) and m.block_table("a", 0) == [0, 1, 2]
    assert m.extend("a", 12) and len(m.block_table("a", 0)) == 3          # still inside the third page
    assert not m.can_extend("b", 9) and not m.extend("b", 9)
    assert m.block_table("b", 0) == [] and m.pools[0].num_free == 2        # nothing taken
    assert m.max_extension("b", 100) == 8
    assert m.extend("b", 8)
    m.check_invariants()
    m.release("a")
    assert m.pools[0].num_free == 3 and not m.has_request("a")
    assert m.extend("b", 20)
    assert m.block_table("b", 0) == [3, 4, 0, 1, 2]                        # pages of "a" are used again
    m.check_invariants()
    with pytest.raises(PagePoolError):
        m.extend("b", 4)                                                    # cannot shrink
    with pytest.raises(PagePoolError, match="already admitted"):
        m.admit("b")


def test_slots():
    m = _mgr(slots=2)
    s = {m.admit("a"), m.admit("b")}
    assert s == {0, 1} and not m.can_admit()
    with pytest.raises(PagePoolError, match="no free state slot"):
        m.admit("c")
    m.release("a")
    assert m.can_admit() and m.admit("c") in (0, 1)
    m.check_invariants()


def test_window_group_gives_pages_back_as_the_window_passes():
    m = _mgr(pages=8, page=4, window=6)
    m.admit("a")
    assert m.extend("a", 16)
    assert len(m.block_table("a", 0)) == 4 and len(m.block_table("a", 1)) == 4
    # The next query is at position 16 and sees keys 11..16: pages 0 and 1 (positions 0..7) are out of sight.
    assert m.release_behind_window("a") == 2
    assert m.block_table("a", 1)[:2] == [NO_PAGE, NO_PAGE] and NO_PAGE not in m.block_table("a", 0)
    assert m.pools[1].num_free == 6 and m.pools[0].num_free == 4
    assert m.extend("a", 17) and m.release_behind_window("a") == 1       # next query, at 17, sees keys 12..17: page 2 (8..11) goes
    m.check_invariants()
    assert m.block_table("a", 1)[:3] == [NO_PAGE] * 3 and m.block_table("a", 1)[3] != NO_PAGE
    assert m.extend("a", 20) and m.release_behind_window("a") == 0       # keys 15..20 still need page 3 (12..15)
    assert m.extend("a", 21) and m.release_behind_window("a") == 1
    m.release("a")
    assert m.pools[1].num_free == 8 and m.pools[0].num_free == 8
    m.check_invariants()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_every_page_accounted_for(seed):
    rng = random.Random(seed)
    window = rng.choice([0, 5, 13])
    m = _mgr(pages=rng.randint(6, 20), page=rng.choice([2, 4, 8]), window=window, slots=5)
    live: dict[str, int] = {}
    next_id = 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and m.can_admit():
            rid = f"r{next_id}"; next_id += 1
            m.admit(rid); live[rid] = 0
        elif op < 0.8 and live:
            rid = rng.choice(sorted(live))
            new = live[rid] + rng.randint(1, 9)
            free_before = [p.num_free for p in m.pools]
            if m.extend(rid, new):
                live[rid] = new
                m.release_behind_window(rid)
            else:
                assert [p.num_free for p in m.pools] == free_before      # a failed extend takes nothing
                grown = m.max_extension(rid, new)
                assert live[rid] <= grown < new and m.extend(rid, grown)
                live[rid] = grown
        elif live:
            rid = rng.choice(sorted(live))
            m.release(rid); del live[rid]
            with pytest.raises(KeyError):
                m.release(rid)                                             # nothing is freed twice
        m.check_invariants()
        for rid, n in live.items():
            t = m.block_table(rid, 0)
            assert len(t) == -(-n // m.page_size) and NO_PAGE not in t
            if window:
                tw = m.block_table(rid, 1)
                first_visible = max(0, n - window + 1) // m.page_size
                assert all(p != NO_PAGE for p in tw[first_visible:]) and len(tw) == len(t)
    for rid in list(live):
        m.release(rid)
    assert all(p.num_free == p.num_pages for p in m.pools)


def test_extend_by_one_equals_extend_and_is_all_or_nothing():
    """The decoding batch's one-pass extension takes the same pages as one extend() per request, and nothing when
    a group lacks pages."""
    import random
    from lucciola_b200.cache.manager import CacheGroup, CacheManager
    groups = [CacheGroup(2, 16, 0, (0,)), CacheGroup(2, 16, 6, (1,))]
    rnd = random.Random(3)
    a, b = CacheManager(groups, 4, 40, 4), CacheManager(groups, 4, 40, 4)
    rids = ["x", "y", "z"]
    for m in (a, b):
        for i, rid in enumerate(rids):
            m.admit(rid)
            assert m.extend(rid, 3 + 5 * i)
    for step in range(30):
        batch = [r for r in rids if rnd.random() < 0.8] or rids[:1]
        starts = a.extend_by_one(batch)
        assert starts == [b.length(r) for r in batch]
        for r in batch:
            assert b.extend(r, b.length(r) + 1)
        for r in rids:
            assert a.length(r) == b.length(r)
            for g in range(2):
                assert len(a.block_table(r, g)) == len(b.block_table(r, g))
            a.release_behind_window(r); b.release_behind_window(r)
        a.check_invariants(); b.check_invariants()
        assert [p.num_free for p in a.pools] == [p.num_free for p in b.pools]
    # all or nothing: with too few pages left for the whole batch nothing changes
    small = CacheManager([CacheGroup(1, 8, 0, (0,))], 4, 3, 4)
    for rid in ("p", "q"):
        small.admit(rid)
        assert small.extend(rid, 4)                 # one page each, full
    before = ([small.length(r) for r in ("p", "q")], small.pools[0].num_free)
    assert small.pools[0].num_free == 1
    assert small.extend_by_one(["p", "q"]) is None   # both need a new page, one is free
    assert ([small.length(r) for r in ("p", "q")], small.pools[0].num_free) == before
    small.check_invariants()
    assert small.extend_by_one(["p"]) == [4]
