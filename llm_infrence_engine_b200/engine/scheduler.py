"""The scheduler: which requests bring which tokens to the next step. Host only, no tensors.

Every step it

1. drops cancelled requests (src/miniserve/engine.py:168-177);
2. gives each running request its next tokens under the step's token budget: first the requests
   that decode (one token each), then prompts that are still being read, oldest first, each cut
   to what is left of the budget (the reference never cuts a prompt: it prefills whole prompts,
   one request per forward, src/miniserve/paged_engine.py:126-127);
3. admits waiting requests in arrival order while a state slot is free, budget is left and the
   pages for the portion are there with one spare page per running request
   (paged_engine.py:115-119); if the head of the queue does not fit, nobody behind it is tried
   (paged_engine.py:90-91).

When a running request needs a page and the pool is empty, the youngest running request is
preempted: its pages and slot go back, it returns to the FRONT of the queue and later recomputes
prompt plus output so far (paged_engine.py:152-164,179-187). If the victim is the request that
asked, it simply waits. A request that could never fit alone is refused when it is added
(paged_engine.py:58-59), so the oldest request can always go on and the engine never stalls.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, List, Optional

from ..cache.manager import CacheManager, OutOfPages
from .request import Request


@dataclass
class Scheduled:
    req: Request
    start: int        # = req.num_computed
    count: int        # tokens it brings
    samples: bool     # the portion ends the known tokens: its last logits are sampled


@dataclass
class StepPlan:
    items: List[Scheduled] = field(default_factory=list)
    admitted: int = 0
    preempted: int = 0
    aborted: List[Request] = field(default_factory=list)

    @property
    def num_tokens(self) -> int:
        return sum(s.count for s in self.items)


class Scheduler:
    def __init__(self, cache: CacheManager, max_seqs: int, max_len: int, max_num_batched_tokens: int):
        self.cache = cache
        self.max_seqs, self.max_len, self.budget = max_seqs, max_len, max_num_batched_tokens
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.preemptions = 0
        self._admit_counter = 0
        self._next_id = 0

    # ------------------------------------------------------------------ requests in and out
    def add(self, req: Request) -> Request:
        need = len(req.prompt_ids) + req.max_new_tokens
        if not req.prompt_ids:
            raise ValueError("empty prompt")  # engine.py:147-148
        if req.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be at least 1")
        if need > self.max_len:
            raise ValueError(f"request needs {need} cache positions but max_len is {self.max_len}")  # engine.py:144-146
        if need > self.cache.capacity_tokens:
            raise ValueError("request can never fit in the page pool")  # paged_engine.py:58-59
        req.id = self._next_id
        self._next_id += 1
        req.state = "waiting"
        self.waiting.append(req)
        return req

    def has_work(self) -> bool:
        return bool(self.waiting) or bool(self.running)

    def finish(self, req: Request) -> None:
        """A request ends: everything it holds goes back. (It may be waiting: preempted while its last token was on its way.)"""
        if req in self.running:
            self.running.remove(req)
            self.cache.free(req.id)
        elif req in self.waiting:
            self.waiting.remove(req)
        req.state = "finished"

    def _preempt(self, victim: Request) -> None:
        self.running.remove(victim)
        self.cache.free(victim.id)
        victim.state = "waiting"
        victim.num_computed = 0
        victim.preemptions += 1
        self.preemptions += 1
        self.waiting.appendleft(victim)

    # ------------------------------------------------------------------ one step's decisions
    def schedule(self) -> StepPlan:
        plan = StepPlan()
        for r in [r for r in self.waiting if r.cancelled]:
            self.waiting.remove(r)
            r.state = "finished"
            plan.aborted.append(r)
        for r in [r for r in self.running if r.cancelled]:
            self.finish(r)
            plan.aborted.append(r)

        budget = self.budget
        before = self.preemptions
        # running requests: those that decode first, then prompts in progress, each group oldest first
        order = sorted(self.running, key=lambda r: (r.num_tokens - r.num_computed > 1, r.admit_seq))
        for r in order:
            if r.state != "running" or budget <= 0:
                continue
            if r.in_flight and len(r.output_ids) + r.in_flight >= r.max_new_tokens:
                continue  # the token on its way is its last
            pending = r.num_tokens - r.num_computed
            count = min(pending, budget)
            while True:
                try:
                    self.cache.reserve(r.id, r.num_computed, r.num_computed + count)
                    break
                except OutOfPages:
                    victim = max(self.running, key=lambda x: x.admit_seq)
                    self._preempt(victim)
                    plan.items = [s for s in plan.items if s.req is not victim]
                    if victim is r:
                        break
            if r.state != "running":
                continue
            plan.items.append(Scheduled(r, r.num_computed, count, count == pending))
            budget -= count
        budget = self.budget - plan.num_tokens
        plan.preempted = self.preemptions - before

        # admission, in arrival order; nothing is admitted in a step that had to preempt
        while self.waiting and not plan.preempted and budget > 0 and len(self.running) < self.max_seqs \
                and self.cache.num_free_slots() > 0:
            r = self.waiting[0]
            if r.in_flight:
                break  # preempted with a token still on the device: it comes back once that token has been read
            self.cache.admit(r.id)
            # with prefix sharing: the leading full pages that the cache already holds are taken over, not computed
            # (src/miniserve/paged_engine.py:102-112); at least one token is always left
            have = self.cache.share_prefix(r.id, r.tokens(0, r.num_tokens))
            pending = r.num_tokens - have
            count = min(pending, budget)
            if not self.cache.can_reserve(r.id, have, have + count, spare=len(self.running)):
                self.cache.free(r.id)
                self.cache.shared_tokens -= have  # not admitted after all
                break
            self.cache.reserve(r.id, have, have + count)
            self.waiting.popleft()
            self._admit_counter += 1
            r.admit_seq = self._admit_counter
            r.state = "running"
            r.num_computed = have
            self.running.append(r)
            plan.items.append(Scheduled(r, have, count, count == pending))
            plan.admitted += 1
            budget -= count
        return plan

    def advance(self, plan: StepPlan) -> None:
        """The step ran: what it computed is in the cache now."""
        for s in plan.items:
            s.req.num_computed = s.start + s.count
            if self.cache.prefix_sharing and self.cache.holds(s.req.id):
                # pages that are now full of tokens the host knows become findable (a token still on the device is not known)
                known = min(s.req.num_computed, len(s.req.prompt_ids) + len(s.req.output_ids))
                self.cache.register_full_pages(s.req.id, s.req.tokens(0, known))
