"""The cache manager without any tensor: no page lost, held twice or freed twice, under random orders of requests;
windows give pages back; state slots."""
import random

import pytest

from llm_infrence_engine_b200.cache import NULL_PAGE, CacheManager, OutOfPages, PagedKVSpec, PagePool


def test_pool_basics():
    p = PagePool(4)
    assert p.capacity == 3
    got = [p.allocate("a") for _ in range(3)]
    assert sorted(got) == [1, 2, 3] and NULL_PAGE not in got
    with pytest.raises(OutOfPages):
        p.allocate("a")
    p.free(2, "a")
    with pytest.raises(ValueError, match="twice"):
        p.free(2, "a")
    with pytest.raises(ValueError, match="belongs"):
        p.free(1, "b")
    with pytest.raises(ValueError):
        p.free(0, "a")
    assert p.allocate("b") == 2  # a page that came back is handed out again
    with pytest.raises(ValueError):
        PagePool(1)


def test_reserve_grows_and_free_returns_everything():
    m = CacheManager([PagedKVSpec(2, 16)], num_pages=9, page_size=4, max_seqs=2)
    assert m.capacity_tokens == 32
    slot = m.admit("r")
    m.reserve("r", 0, 5)
    assert len(m.block_table("r", 0)) == 2
    m.reserve("r", 5, 8)
    assert len(m.block_table("r", 0)) == 2      # still inside the second page
    m.reserve("r", 8, 9)
    assert len(m.block_table("r", 0)) == 3
    m.check_invariants()
    other = m.admit("s")
    assert other != slot
    with pytest.raises(OutOfPages):
        m.admit("t")                            # no third state slot
    with pytest.raises(OutOfPages):
        m.reserve("s", 0, 6 * 4)                # 6 pages wanted, 5 free: nothing is taken
    assert m.num_free_pages() == 5 and m.block_table("s", 0) == []
    assert m.can_reserve("s", 0, 20) and not m.can_reserve("s", 0, 20, spare=1)
    m.free("r")
    with pytest.raises(ValueError, match="twice"):
        m.free("r")
    m.free("s")
    m.check_invariants()
    assert m.num_free_pages() == 8 and m.num_free_slots() == 2


def test_window_gives_pages_back_as_it_passes():
    full, win = PagedKVSpec(1, 8), PagedKVSpec(1, 8, window=10)
    m = CacheManager([full, win], num_pages=20, page_size=4, max_seqs=1)
    m.admit("r")
    length = 0
    for step in (7, 1, 1, 9, 1, 1, 1, 30, 1):
        m.reserve("r", length, length + step)
        length += step
        m.check_invariants()
        t_full, t_win = m.block_table("r", 0), m.block_table("r", 1)
        assert NULL_PAGE not in t_full and len(t_full) == -(-length // 4)
        first_needed = max(0, (length - step) - 10 + 1) // 4   # the first query of the step looks back 10 keys
        assert all(p == NULL_PAGE for p in t_win[:first_needed])
        assert all(p != NULL_PAGE for p in t_win[first_needed:])
    m.release_passed("r", length)
    held = [p for p in m.block_table("r", 1) if p != NULL_PAGE]
    assert len(held) <= 10 // 4 + 2               # about a window's worth of pages stays
    m.free("r")
    m.check_invariants()
    assert m.num_free_pages(0) == m.num_free_pages(1) == 19


@pytest.mark.parametrize("seed", range(8))
def test_random_orders(seed):
    rng = random.Random(seed)
    groups = [PagedKVSpec(2, 16), PagedKVSpec(2, 16, window=rng.choice([5, 16, 33]))][: rng.choice([1, 2])]
    m = CacheManager(groups, num_pages=rng.choice([6, 17, 40]), page_size=rng.choice([1, 4, 16]), max_seqs=4)
    live, next_id = {}, 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and m.num_free_slots():
            m.admit(next_id)
            live[next_id] = 0
            next_id += 1
        elif op < 0.8 and live:
            r = rng.choice(list(live))
            step = rng.choice([1, 1, 1, 2, 7, 30])
            before = [list(m.block_table(r, g)) for g in range(len(groups))]
            free_before = [m.num_free_pages(g) for g in range(len(groups))]
            try:
                m.reserve(r, live[r], live[r] + step)
                live[r] += step
            except OutOfPages:
                # nothing was taken; windows may have given pages back, which only frees more
                assert all(m.num_free_pages(g) >= free_before[g] for g in range(len(groups)))
                assert all(len(m.block_table(r, g)) == len(before[g]) for g in range(len(groups)))
        elif live:
            r = rng.choice(list(live))
            m.free(r)
            del live[r]
        m.check_invariants()
    for r in list(live):
        m.free(r)
    m.check_invariants()
    assert all(p.num_free == p.capacity for p in m.pools) and m.num_free_slots() == 4


def test_prefix_sharing_takes_over_full_pages_and_keeps_one_token():
    """src/miniserve/paged.py:41-49,114-122, paged_engine.py:102-112,133-134: chained hashes of full pages, holders counted,
    a page without holders stays findable until it is the least recently used and the free list is empty."""
    m = CacheManager([PagedKVSpec(2, 16)], num_pages=7, page_size=4, max_seqs=3, prefix_sharing=True)
    a = list(range(100, 111))                      # 11 tokens: pages [100..103], [104..107] full, [108..110] not
    m.admit("a")
    assert m.share_prefix("a", a) == 0             # nothing cached yet
    m.reserve("a", 0, 11)
    m.register_full_pages("a", a)
    ta = list(m.block_table("a", 0))
    m.check_invariants()
    # the same 8 leading tokens: both full pages are taken over; a different 5th token: only the first
    m.admit("b")
    assert m.share_prefix("b", a[:8] + [7, 7]) == 8 and m.block_table("b", 0) == ta[:2]
    m.admit("c")
    assert m.share_prefix("c", a[:4] + [9] + a[5:]) == 4 and m.block_table("c", 0) == ta[:1]
    assert m.pools[0].holders(ta[0]) == 3 and m.pools[0].holders(ta[1]) == 2 and m.shared_tokens == 12
    m.check_invariants()
    m.reserve("b", 8, 10)
    m.reserve("c", 4, 11)
    m.check_invariants()
    # exactly the cached tokens again: one token at least is left to compute
    m.free("c")
    m.admit("d")
    assert m.share_prefix("d", a[:8]) == 4
    m.free("d")
    # holders go: the two named pages stay cached, the others are free; everything can be handed out
    m.free("a")
    m.free("b")
    m.check_invariants()
    pool = m.pools[0]
    assert pool.num_free == pool.capacity and sum(pool.name_of(p) is not None for p in pool.idle_pages()) == 2
    assert [pool.name_of(p) is not None for p in pool.idle_pages()] == [False] * 4 + [True] * 2   # named pages are handed out last
    m.admit("e")
    assert m.share_prefix("e", a) == 8             # found again after their holders had gone
    m.free("e")
    m.admit("f")
    m.reserve("f", 0, 24)                           # all six pages: the cached ones are evicted, oldest first
    assert pool.names_given_up == 2 and not pool.idle_pages() and all(pool.name_of(p) is None for p in range(1, 7))
    m.check_invariants()
    m.free("f")
    m.admit("g")
    assert m.share_prefix("g", a) == 0
    m.free("g")
    m.check_invariants()


def test_prefix_sharing_is_refused_where_pages_are_not_all_a_request_has():
    win = CacheManager([PagedKVSpec(1, 8), PagedKVSpec(1, 8, window=6)], num_pages=9, page_size=4, max_seqs=1, prefix_sharing=True)
    assert not win.prefix_sharing
    one = CacheManager([PagedKVSpec(1, 8, window=6)], num_pages=9, page_size=4, max_seqs=1, prefix_sharing=True)
    assert not one.prefix_sharing
    one.admit("a")
    assert one.share_prefix("a", list(range(20))) == 0


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_with_prefix_sharing(seed):
    """Requests whose tokens share leading pages come and go in random order: no page lost, no holder miscounted, and a
    taken-over page always holds exactly the tokens its new holder expects."""
    rng = random.Random(100 + seed)
    ps = rng.choice([2, 4])
    m = CacheManager([PagedKVSpec(1, 8)], num_pages=rng.choice([9, 20]), page_size=ps, max_seqs=4, prefix_sharing=True)
    stems = [[rng.randrange(5) for _ in range(12)] for _ in range(3)]
    content = {}  # page -> tokens written there (what a device would hold)
    live = {}
    for step in range(400):
        if live and (len(live) == 4 or rng.random() < 0.4):
            name = rng.choice(list(live))
            m.free(name)
            del live[name]
        else:
            name = f"r{step}"
            toks = list(rng.choice(stems)[:rng.randrange(1, 12)]) + [rng.randrange(5) for _ in range(rng.randrange(1, 6))]
            m.admit(name)
            have = m.share_prefix(name, toks)
            assert have % ps == 0 and have < len(toks)
            for i, page in enumerate(m.block_table(name, 0)):
                assert content[page] == toks[i * ps:(i + 1) * ps]
            if not m.can_reserve(name, have, len(toks)):
                m.free(name)
                m.check_invariants()
                continue
            m.reserve(name, have, len(toks))
            for i, page in enumerate(m.block_table(name, 0)):
                if i * ps >= have:
                    content[page] = toks[i * ps:(i + 1) * ps]
            m.register_full_pages(name, toks)
            live[name] = toks
        m.check_invariants()
    for name in list(live):
        m.free(name)
    m.check_invariants()
    assert m.pools[0].num_free == m.pools[0].capacity
