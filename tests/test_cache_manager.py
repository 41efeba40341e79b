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
