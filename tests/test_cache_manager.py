"""The cache manager: no page lost, held twice or freed twice, under random orders of requests;
windows give pages back; state slots (no GPU)."""
import random

import pytest

import sys

from dinfer_b200.cache.block_pool import BlockPool, PoolError, StateSlots
from dinfer_b200.cache.manager import CacheManager, GroupSpec
from dinfer_b200.cache.native import NativeCacheManager

PythonCacheManager = CacheManager


@pytest.fixture(params=["python", "native"], autouse=True)
def implementation(request, monkeypatch):
    """Every test of this file runs twice: on the Python cache manager and on the one whose bookkeeping is C++."""
    if request.param == "native":
        monkeypatch.setattr(sys.modules[__name__], "CacheManager", NativeCacheManager)
    return request.param



def test_pool_reuses_freed_pages_first():
    p = BlockPool(4)
    a = p.allocate(3)
    assert a == [0, 1, 2] and p.num_free == 1
    p.free([1])
    assert p.allocate(1) == [1]                 # the page just freed is used again at once
    with pytest.raises(PoolError):
        p.allocate(2)
    p.free([0])
    with pytest.raises(PoolError, match="not held"):
        p.free([0])
    with pytest.raises(PoolError, match="not of this pool"):
        p.free([9])


def test_allocate_is_incremental_and_all_or_nothing():
    m = CacheManager([GroupSpec()], block_size=4, num_blocks=5, max_num_seqs=4)
    assert m.allocate("a", 5) and m.block_table("a", 0) == [0, 1]
    assert m.allocate("a", 8) and m.block_table("a", 0) == [0, 1]        # still covered: nothing new
    assert m.allocate("a", 9) and len(m.block_table("a", 0)) == 3
    assert not m.allocate("b", 12)                                       # needs 3, 2 free
    assert "b" not in m and m.num_free_blocks() == 2                     # state untouched
    m.check_invariants()
    assert m.allocate("b", 8)
    m.free("a")
    assert m.num_free_blocks() == 3
    with pytest.raises(PoolError):
        m.free("a")
    m.check_invariants()


def test_window_group_gives_pages_back():
    m = CacheManager([GroupSpec(), GroupSpec(window=6)], block_size=4, num_blocks=[16, 16], max_num_seqs=2)
    assert m.allocate("a", 20)
    assert len(m.block_table("a", 0)) == 5 and len(m.block_table("a", 1)) == 5
    m.advance("a", 20)           # next query at 20 sees keys >= 15: blocks 0..2 (positions < 12) are passed
    assert m.block_table("a", 1)[:3] == [-1, -1, -1] and all(b >= 0 for b in m.block_table("a", 1)[3:])
    assert all(b >= 0 for b in m.block_table("a", 0))
    assert m.num_free_blocks(1) == 16 - 2
    m.check_invariants()
    assert m.allocate("a", 21)
    assert len(m.block_table("a", 1)) == 6
    m.advance("a", 21)
    m.free("a")
    assert m.num_free_blocks(0) == 16 and m.num_free_blocks(1) == 16
    m.check_invariants()


def test_groups_fail_together():
    m = CacheManager([GroupSpec(), GroupSpec(window=4)], block_size=4, num_blocks=[8, 2], max_num_seqs=2)
    assert not m.allocate("a", 12)              # the window group has only 2 pages
    assert m.num_free_blocks(0) == 8 and m.num_free_blocks(1) == 2 and "a" not in m
    assert m.state_slots.num_free == 2


def test_state_slots():
    s = StateSlots(2)
    assert s.acquire("a") == 0 and s.acquire("a") == 0
    assert s.take_fresh("a") is True and s.take_fresh("a") is False
    assert s.acquire("b") == 1 and s.acquire("c") is None
    s.release("a")
    assert s.acquire("c") == 0 and s.take_fresh("c") is True     # a reused slot is fresh again
    m = CacheManager([GroupSpec()], 4, 8, max_num_seqs=1)
    assert m.allocate("a", 1) and not m.allocate("b", 1)         # no slot for a second request
    m.free("a")
    assert m.allocate("b", 1)


@pytest.mark.parametrize("seed", range(6))
def test_random_orders(seed):
    rng = random.Random(seed)
    bs = rng.choice([1, 4, 16])
    own = rng.choice([2, 8]) if seed % 3 == 1 else None          # a page size of the second group's own
    groups = [GroupSpec(), GroupSpec(window=rng.choice([3, 7, 16]), block_size=own)] if seed % 2 else [GroupSpec()]
    sizes = [g.block_size or bs for g in groups]
    m = CacheManager(groups, bs, [rng.randrange(8, 40) for _ in groups], max_num_seqs=5)
    assert m.block_sizes == sizes
    live = {}
    next_id = 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 7:
            live[next_id] = 0
            next_id += 1
        elif op < 0.85 and live:
            r = rng.choice(list(live))
            grow = rng.choice([1, 1, 1, 2, 5, 17])
            before = [m.num_free_blocks(g) for g in range(len(groups))]
            ok = m.allocate(r, live[r] + grow)
            if ok:
                live[r] += grow
                m.advance(r, live[r])
                for g in range(len(groups)):          # every position a query may still see has a page
                    t = m.block_table(r, g)
                    w = groups[g].window
                    first = 0 if w is None else max(0, live[r] - w + 1)
                    assert all(t[p // sizes[g]] >= 0 for p in range(first, live[r]))
                    assert len(t) == (live[r] + sizes[g] - 1) // sizes[g] or len(t) * sizes[g] >= live[r]
            else:
                assert [m.num_free_blocks(g) for g in range(len(groups))] == before
                if r not in m:
                    del live[r]
        elif live:
            r = rng.choice(list(live))
            if r in m:
                m.free(r)
            del live[r]
        m.check_invariants()
    for r in list(live):
        if r in m:
            m.free(r)
    m.check_invariants()
    assert all(m.num_free_blocks(g) == m.pools[g].num_blocks for g in range(len(groups)))
    assert m.state_slots.num_free == 5


# ---------------------------------------------------------------- prefix cache

def _run_tokens(m, rid, toks, chunk=7):
    """Bring request ``rid`` with tokens ``toks`` through begin / allocate / advance; the tokens computed."""
    start = m.begin(rid, toks)
    done, computed = start, 0
    while done < len(toks):
        n = min(chunk, len(toks) - done)
        assert m.allocate(rid, done + n)
        m.advance(rid, done + n, toks[done:done + n])
        done += n
        computed += n
    return start, computed


def test_prefix_cache_hits_whole_pages_and_never_the_last_token():
    m = CacheManager([GroupSpec()], 4, 32, 8, enable_prefix_caching=True)
    a = list(range(100, 118))                       # 18 tokens: 4 full pages + 2
    assert _run_tokens(m, "a", a) == (0, 18)
    m.check_invariants()
    # the same tokens again: 4 pages are cached, but the last token must be run -> (18-1)//4 = 4 pages
    assert _run_tokens(m, "b", a) == (16, 2)
    assert m.block_table("b", 0)[:4] == m.block_table("a", 0)[:4]
    assert m.block_table("b", 0)[4] != m.block_table("a", 0)[4]
    # exactly 16 tokens: only 3 pages may be taken, the last token has to run
    assert _run_tokens(m, "c", a[:16]) == (12, 4)
    # a different token in page 1 breaks the chain after page 0
    d = a[:5] + [999] + a[6:]
    assert _run_tokens(m, "d", d)[0] == 4
    m.check_invariants()
    for r in ("a", "b", "c", "d"):
        m.free(r)
    m.check_invariants()
    assert m.num_free_blocks() == 32
    # freed, but still findable until the pages are needed
    assert _run_tokens(m, "e", a)[0] == 16
    m.check_invariants()


def test_prefix_cache_eviction_is_least_recently_used_and_unhashed_pages_go_first():
    m = CacheManager([GroupSpec()], 4, 8, 8, enable_prefix_caching=True)
    a, b = list(range(8)), list(range(50, 58))
    _run_tokens(m, "a", a + [1])                    # 2 hashed pages + 1 page in use
    _run_tokens(m, "b", b + [1])
    m.free("a"); m.free("b")                        # a's pages are older on the free list than b's
    m.check_invariants()
    pool = m.pools[0]
    assert pool.num_free == 8 and pool.evictions == 0
    # 8 pages free: 2 never used, 2 unhashed (the partly filled ones), 4 hashed.  Taking 5 evicts one hashed
    # page: the deepest page of the request freed first.
    assert m.allocate("x", 20)
    assert pool.evictions == 1
    m.free("x")                                     # unhashed pages: they are used before the hashed ones
    assert _run_tokens(m, "b2", b + [2])[0] == 8    # b's chain is whole
    m.free("b2")
    assert _run_tokens(m, "a2", a + [2])[0] == 4    # a's second page is gone, its first still there
    m.check_invariants()


def test_prefix_cache_random_orders_keep_the_books():
    rng = random.Random(11)
    m = CacheManager([GroupSpec(), GroupSpec()], 4, 40, 6, enable_prefix_caching=True)
    stems = [[rng.randrange(50) for _ in range(rng.randrange(4, 30))] for _ in range(4)]
    live = {}
    hits = 0
    for step in range(600):
        if live and (len(live) >= 6 or rng.random() < 0.4):
            rid = rng.choice(list(live))
            toks, done = live[rid]
            if done >= len(toks) or rng.random() < 0.2:
                m.free(rid)
                del live[rid]
            else:
                n = min(rng.randrange(1, 9), len(toks) - done)
                if m.allocate(rid, done + n):
                    m.advance(rid, done + n, toks[done:done + n])
                    live[rid] = (toks, done + n)
                else:                                   # out of pages: give up (a preemption)
                    m.free(rid)
                    del live[rid]
        else:
            rid = f"r{step}"
            toks = rng.choice(stems) + [rng.randrange(50) for _ in range(rng.randrange(1, 10))]
            start = m.begin(rid, toks)
            assert start % 4 == 0 and start <= len(toks) - 1
            hits += start
            if start or m.allocate(rid, 1):
                if rid in m:
                    live[rid] = (toks, start)
        m.check_invariants()
    assert hits > 0 and m.prefix_hits == hits
    for rid in list(live):
        m.free(rid)
    m.check_invariants()
    assert all(p.num_free == p.num_blocks for p in m.pools)


def test_prefix_cache_refuses_windowed_groups():
    with pytest.raises(ValueError):
        CacheManager([GroupSpec(window=8)], 4, 8, 2, enable_prefix_caching=True)


def test_tokens_that_are_not_known_yet():
    """``advance`` may be told of a computed token whose id the host has not read (negative); the page it
    completes gets its hash when ``resolve`` brings the id, and not before."""
    m = CacheManager([GroupSpec()], 4, 16, 4, enable_prefix_caching=True)
    assert m.allocate("a", 8)
    m.advance("a", 7, [1, 2, 3, 4, 5, 6, 7])
    m.advance("a", 8, [-1])                           # computed on the device from the last sampling
    assert m.begin("probe", [1, 2, 3, 4, 5, 6, 7, 9, 0]) == 4      # only the first page is findable
    m.free("probe")
    assert m.allocate("a", 9)
    m.resolve("a", [9])
    m.advance("a", 9, [-2])
    assert m.begin("probe", [1, 2, 3, 4, 5, 6, 7, 9, 0]) == 8
    m.free("probe")
    assert m.allocate("a", 10)
    with pytest.raises(PoolError, match="do not make"):
        m.advance("a", 10, [33])                      # a known token cannot follow one that is still unknown
    with pytest.raises(PoolError, match="more tokens resolved"):
        m.resolve("a", [1, 2])                        # more than was computed
    m.resolve("a", [11])
    m.free("a")
    m.check_invariants()
    assert m.num_free_blocks() == 16


def test_a_batch_is_asked_for_as_a_whole():
    """``can_allocate_all`` answers for a step's whole batch and changes nothing."""
    m = CacheManager([GroupSpec(), GroupSpec(window=8)], 4, [6, 6], max_num_seqs=2)
    assert m.allocate("a", 9)                                   # 3 pages of each group
    before = (m.num_free_blocks(0), m.num_free_blocks(1), m.state_slots.num_free)
    assert m.can_allocate_all([("a", 12), ("b", 12)])            # 0 + 3 pages
    assert not m.can_allocate_all([("a", 13), ("b", 12)])        # 1 + 3 pages of 3 free
    assert not m.can_allocate_all([("a", 10), ("b", 1), ("c", 1)])   # one state slot free, two newcomers
    assert (m.num_free_blocks(0), m.num_free_blocks(1), m.state_slots.num_free) == before
    assert m.requests() == ["a"]
    m.check_invariants()


def test_both_implementations_hand_out_the_same_pages_in_the_same_order():
    """One random sequence of requests that come, grow, finish and repeat beginnings, driven through the Python and
    the C++ cache manager side by side: the same answers, the same page ids in every table, the same free counts,
    the same state slots, the same prefix hits and evictions (their page hashes differ, what they find does not)."""
    rng = random.Random(2024)
    for prefix, groups in ((False, [GroupSpec(), GroupSpec(window=9)]), (True, [GroupSpec(), GroupSpec()]),
                           (False, [GroupSpec(block_size=16), GroupSpec(window=9, block_size=2)])):
        a = PythonCacheManager(groups, 4, [30, 30], 5, enable_prefix_caching=prefix)
        b = NativeCacheManager(groups, 4, [30, 30], 5, enable_prefix_caching=prefix)
        stems = [[rng.randrange(40) for _ in range(rng.randrange(4, 40))] for _ in range(3)]
        live = {}
        for step in range(1500):
            r = rng.random()
            if live and r < 0.25:
                rid = rng.choice(list(live))
                assert (rid in a) == (rid in b)
                if rid in a:
                    a.free(rid); b.free(rid)
                del live[rid]
            elif r < 0.5:
                rid = f"r{step}"
                toks = list(rng.choice(stems)) + [rng.randrange(40) for _ in range(rng.randrange(1, 12))]
                ha, hb = a.begin(rid, toks), b.begin(rid, toks)
                assert ha == hb
                live[rid] = (toks, ha)
            elif live:
                rid = rng.choice(list(live))
                toks, done = live[rid]
                n = min(rng.randrange(1, 9), len(toks) - done)
                if n > 0:
                    assert a.can_allocate(rid, done + n) == b.can_allocate(rid, done + n)
                    oa, ob = a.allocate(rid, done + n), b.allocate(rid, done + n)
                    assert oa == ob
                    if oa:
                        a.advance(rid, done + n, toks[done:done + n]); b.advance(rid, done + n, toks[done:done + n])
                        live[rid] = (toks, done + n)
                    elif rid not in a:
                        del live[rid]
            assert a.requests() == b.requests()
            for rid in a.requests():
                assert [a.block_table(rid, g) for g in range(2)] == [b.block_table(rid, g) for g in range(2)]
                assert (a.num_tokens(rid), a.num_computed(rid)) == (b.num_tokens(rid), b.num_computed(rid))
                assert a.state_slots.slot(rid) == b.state_slots.slot(rid)
            assert [p.num_free for p in a.pools] == [p.num_free for p in b.pools]
            assert [p.evictions for p in a.pools] == [p.evictions for p in b.pools]
            assert a.state_slots.num_free == b.state_slots.num_free
            assert (a.prefix_queries, a.prefix_hits) == (b.prefix_queries, b.prefix_hits)
            if step % 50 == 0:
                a.check_invariants(); b.check_invariants()
        a.check_invariants(); b.check_invariants()


def test_groups_with_page_sizes_of_their_own():
    """A group may have its own page size: its table is as long as its pages need, a window gives back what its own
    pages have passed, and the prefix cache, whose hashes name the tokens of a page, wants one size for all."""
    m = CacheManager([GroupSpec(), GroupSpec(window=6, block_size=2), GroupSpec(block_size=16)], block_size=4,
                     num_blocks=[8, 16, 2], max_num_seqs=2)
    assert m.block_sizes == [4, 2, 16]
    assert m.allocate("a", 11)
    assert [len(m.block_table("a", g)) for g in range(3)] == [3, 6, 1]
    m.advance("a", 11)
    assert m.block_table("a", 1)[:3] == [-1, -1, -1] and all(b >= 0 for b in m.block_table("a", 1)[3:])   # keys 6.. stay
    assert m.allocate("a", 32) and not m.can_allocate("a", 33)      # the third group's two pages of 16 are the limit
    assert [len(m.block_table("a", g)) for g in range(3)] == [8, 16, 2]
    m.free("a")
    m.check_invariants()
    assert [m.num_free_blocks(g) for g in range(3)] == [8, 16, 2]
    with pytest.raises(ValueError):
        CacheManager([GroupSpec(), GroupSpec(block_size=8)], 4, 8, 2, enable_prefix_caching=True)
