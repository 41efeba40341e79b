"""The scheduler's decisions, without a model: budget, portions, order, admission, what happens when pages run out."""
import pytest

from llm_infrence_engine_b200.cache import CacheManager, PagedKVSpec
from llm_infrence_engine_b200.engine import Request, Scheduler


def make(num_pages=20, page_size=4, max_seqs=4, max_len=64, budget=16):
    cache = CacheManager([PagedKVSpec(1, 8)], num_pages, page_size, max_seqs)
    return cache, Scheduler(cache, max_seqs, max_len, budget)


def run_step(s, emit=lambda r: 1):
    """What the engine does around ``schedule``: advance, append a token for requests whose known tokens are all in, finish at the limit."""
    plan = s.schedule()
    s.advance(plan)
    for it in plan.items:
        if it.samples:
            it.req.output_ids.append(emit(it.req))
            if len(it.req.output_ids) >= it.req.max_new_tokens:
                s.finish(it.req)
    s.cache.check_invariants()
    return plan


def show(plan):
    return [(it.req.id, it.start, it.count, it.samples) for it in plan.items]


def test_prompt_is_cut_under_the_budget_and_decodes_come_first():
    cache, s = make(num_pages=40, budget=16)
    a = s.add(Request(list(range(40)), max_new_tokens=3))
    assert show(run_step(s)) == [(0, 0, 16, False)]
    b = s.add(Request(list(range(5)), max_new_tokens=3))
    assert show(run_step(s)) == [(0, 16, 16, False)]           # the running prompt takes the whole budget; b waits
    assert show(run_step(s)) == [(0, 32, 8, True), (1, 0, 5, True)]   # the last portion samples; b fits beside it
    assert a.output_ids == [1] and b.output_ids == [1]
    c = s.add(Request(list(range(30)), max_new_tokens=2))
    p = run_step(s)
    assert show(p) == [(0, 40, 1, True), (1, 5, 1, True), (2, 0, 14, False)]  # decoded tokens first, then the new prompt's portion
    p = run_step(s)
    assert show(p)[:2] == [(0, 41, 1, True), (1, 6, 1, True)] and show(p)[2] == (2, 14, 14, False)
    assert a.state == "finished" and b.state == "finished"
    assert show(run_step(s)) == [(2, 28, 2, True)]             # a portion may be as short as two tokens
    while s.has_work():
        run_step(s)
    assert cache.num_free_pages() == 39 and cache.num_free_slots() == 4


def test_admission_is_first_come_first_served_with_a_spare_page_per_running_request():
    cache, s = make(num_pages=9, page_size=4, budget=64, max_len=32)   # 8 pages = 32 tokens
    a = s.add(Request(list(range(14)), max_new_tokens=2))   # 4 pages
    b = s.add(Request(list(range(14)), max_new_tokens=2))   # 4 pages, but one spare page for a is wanted
    c = s.add(Request(list(range(2)), max_new_tokens=2))    # would fit, but may not overtake b
    p = run_step(s)
    assert show(p) == [(0, 0, 14, True)] and p.admitted == 1
    assert [r.id for r in s.waiting] == [1, 2]
    run_step(s)
    assert a.state == "finished"
    p = run_step(s)
    assert [it.req.id for it in p.items] == [1, 2] and p.admitted == 2


def test_max_seqs_limits_the_running_set():
    cache, s = make(max_seqs=2, budget=64)
    reqs = [s.add(Request([1, 2, 3], max_new_tokens=4)) for _ in range(3)]
    p = run_step(s)
    assert p.admitted == 2 and len(s.running) == 2 and len(s.waiting) == 1


def test_pages_run_out_youngest_is_preempted_and_recomputes():
    cache, s = make(num_pages=7, page_size=4, budget=64, max_len=24)   # 6 pages = 24 tokens
    a = s.add(Request(list(range(7)), max_new_tokens=12))   # 2 pages now, 5 at the end
    b = s.add(Request(list(range(7)), max_new_tokens=12))
    run_step(s, emit=lambda r: 100 + len(r.output_ids))
    assert len(s.running) == 2 and s.preemptions == 0
    preempted_at = None
    for step in range(40):
        if not s.has_work():
            break
        plan = run_step(s, emit=lambda r: 100 + len(r.output_ids))
        if plan.preempted and preempted_at is None:
            preempted_at = step
            assert b.state == "waiting" and b.num_computed == 0 and b.preemptions == 1   # the youngest goes
            assert s.waiting[0] is b                                                   # to the FRONT of the queue
            assert not cache.holds(b.id) and plan.admitted == 0
            assert all(it.req is a for it in plan.items)
    assert preempted_at is not None
    assert a.output_ids == [100 + i for i in range(12)] and b.output_ids == [100 + i for i in range(12)]
    assert a.preemptions == 0
    assert cache.num_free_pages() == 6 and cache.num_free_slots() == 4


def test_resumed_request_recomputes_prompt_plus_output():
    cache, s = make(num_pages=7, page_size=4, budget=8, max_len=24)
    a = s.add(Request(list(range(7)), max_new_tokens=12))
    b = s.add(Request(list(range(7)), max_new_tokens=12))
    seen = []
    for _ in range(60):
        if not s.has_work():
            break
        plan = run_step(s)
        seen += [(it.req.id, it.start, it.count) for it in plan.items if it.req is b]
    resumed = [x for x in seen if x[1] == 0]
    assert len(resumed) >= 2                     # first admission and at least one resume from position 0
    assert resumed[1][2] == 8                    # the resume recomputes under the budget: a portion of 8 of prompt + output
    assert b.state == "finished" and len(b.output_ids) == 12


def test_refusals():
    cache, s = make(num_pages=5, page_size=4, max_len=64)
    with pytest.raises(ValueError, match="empty"):
        s.add(Request([]))
    with pytest.raises(ValueError, match="max_len"):
        s.add(Request([1] * 10, max_new_tokens=60))
    with pytest.raises(ValueError, match="never fit"):
        s.add(Request([1] * 10, max_new_tokens=10))   # 20 tokens, the pool holds 16
    assert not s.has_work()


def test_cancel_frees_at_the_next_step():
    cache, s = make()
    a = s.add(Request([1, 2, 3], max_new_tokens=50))
    b = s.add(Request([1, 2, 3], max_new_tokens=50))
    run_step(s)
    a.cancelled = True
    c = s.add(Request([4], max_new_tokens=5))
    c.cancelled = True
    plan = run_step(s)
    assert {r.id for r in plan.aborted} == {a.id, c.id}
    assert a.state == "finished" and not cache.holds(a.id) and [it.req.id for it in plan.items] == [b.id]
