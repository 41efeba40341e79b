"""Book-keeping of the cache on the host: pages, block tables and state slots. No tensors here.

Layers whose mixers ask for the same ``PagedKVSpec`` form a group. A group has a pool of pages of
its own and every live request has one block table per group; the page with id 0 is the null page
(the reference reserves block 0 the same way, src/miniserve/paged.py:34,68). A request holds

* a state slot, from admission to the end: the row of every per-request array, and of every
  fixed-size state tensor (an architecture without such state still gets the slot);
* in each group the pages that cover the positions it still has to read: all of them, or for a
  windowed group those from ``length - window + 1`` on; pages that the window has passed go back
  to the pool at once and their entry in the block table becomes the null page.

Pages come back when a request ends, is preempted, or a window has passed them, and are handed
out again without being cleared: a position beyond a request's length is never read. The
reference's allocator (src/miniserve/paged.py:52-135) keeps reference counts for prefix sharing;
this one has single owners and checks for double frees and lost pages instead.
"""
from __future__ import annotations

from collections import deque
from typing import Dict, Hashable, List, Optional, Sequence

from .spec import NULL_PAGE, PagedKVSpec


class OutOfPages(Exception):
    """A group's pool has too few free pages for what was asked."""


class PagePool:
    """Free list of one group's pages. Page 0 is never handed out."""

    def __init__(self, num_pages: int):
        if num_pages < 2:
            raise ValueError("a pool needs at least 2 pages (page 0 is the null page)")
        self.num_pages = num_pages
        self._free = deque(range(1, num_pages))
        self._owner: List[Optional[Hashable]] = [None] * num_pages

    @property
    def capacity(self) -> int:
        return self.num_pages - 1

    @property
    def num_free(self) -> int:
        return len(self._free)

    def allocate(self, owner: Hashable) -> int:
        if not self._free:
            raise OutOfPages()
        page = self._free.popleft()
        self._owner[page] = owner
        return page

    def free(self, page: int, owner: Hashable) -> None:
        if page == NULL_PAGE or not 0 < page < self.num_pages:
            raise ValueError(f"page {page} cannot be freed")
        if self._owner[page] is None:
            raise ValueError(f"page {page} freed twice")
        if self._owner[page] != owner:
            raise ValueError(f"page {page} belongs to {self._owner[page]!r}, not to {owner!r}")
        self._owner[page] = None
        self._free.append(page)

    def owner(self, page: int) -> Optional[Hashable]:
        return self._owner[page]


class _Held:
    """What one live request holds."""

    __slots__ = ("slot", "tables", "length", "versions", "released")

    def __init__(self, slot: int, num_groups: int, version: int):
        self.slot = slot
        self.tables: List[List[int]] = [[] for _ in range(num_groups)]
        self.length = 0  # positions covered so far
        self.versions = [version] * num_groups  # changes whenever the group's table changes; never repeats
        self.released = [0] * num_groups        # pages below this index were given back (windowed groups)


class CacheManager:
    def __init__(self, groups: Sequence[PagedKVSpec], num_pages: int, page_size: int, max_seqs: int):
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.groups = list(groups)
        self.page_size = page_size
        self.max_seqs = max_seqs
        self.pools = [PagePool(num_pages) for _ in self.groups]
        self._free_slots = deque(range(max_seqs))
        self._held: Dict[Hashable, _Held] = {}
        self._version = 0
        self.max_blocks_per_seq = 0  # grows with the longest table seen; informational

    # ------------------------------------------------------------------ capacity
    @property
    def capacity_tokens(self) -> int:
        """Tokens one request alone could hold (the smallest pool decides)."""
        if not self.pools:
            return 1 << 62
        return min(p.capacity for p in self.pools) * self.page_size

    def num_free_pages(self, group: int = 0) -> int:
        return self.pools[group].num_free if self.pools else 1 << 62

    def num_free_slots(self) -> int:
        return len(self._free_slots)

    def holds(self, req: Hashable) -> bool:
        return req in self._held

    def slot(self, req: Hashable) -> int:
        return self._held[req].slot

    def block_table(self, req: Hashable, group: int) -> List[int]:
        return self._held[req].tables[group]

    def table_version(self, req: Hashable, group: int) -> int:
        """A number that changes whenever the request's table in ``group`` changes and is never used twice,
        so a mirror of the table (for instance on the device) knows when it is stale."""
        return self._held[req].versions[group]

    def _bump(self, held: "_Held", group: int) -> None:
        self._version += 1
        held.versions[group] = self._version

    # ------------------------------------------------------------------ lifecycle
    def admit(self, req: Hashable) -> int:
        """Give ``req`` a state slot and empty block tables; returns the slot."""
        if req in self._held:
            raise ValueError(f"request {req!r} is already admitted")
        if not self._free_slots:
            raise OutOfPages("no free state slot")
        slot = self._free_slots.popleft()
        self._version += 1
        self._held[req] = _Held(slot, len(self.groups), self._version)
        return slot

    def _first_needed_page(self, group: int, context_len: int) -> int:
        """Index of the first page that a query at position >= context_len can still read."""
        w = self.groups[group].window
        if w is None:
            return 0
        return max(0, context_len - w + 1) // self.page_size

    def _missing(self, held: "_Held", g: int, context_len: int, new_len: int) -> int:
        """Pages ``reserve`` would take from group ``g``'s pool, not counting those it gives back first. Pages from the
        first needed one up to the end of the table are always held, so only the table's growth counts."""
        want = -(-new_len // self.page_size)
        first = self._first_needed_page(g, context_len)
        return max(0, want - max(len(held.tables[g]), first))

    def _passed(self, held: "_Held", g: int, context_len: int) -> int:
        """Pages of group ``g`` that ``release_passed`` would give back."""
        if self.groups[g].window is None:
            return 0
        first = min(self._first_needed_page(g, context_len), len(held.tables[g]))
        return max(0, first - held.released[g])

    def pages_missing(self, req: Hashable, context_len: int, new_len: int) -> List[int]:
        """Per group, how many pages ``reserve`` would have to find in the pool beyond those it frees first."""
        held = self._held[req]
        return [max(0, self._missing(held, g, context_len, new_len) - self._passed(held, g, context_len))
                for g in range(len(self.groups))]

    def can_reserve(self, req: Hashable, context_len: int, new_len: int, spare: int = 0) -> bool:
        missing = self.pages_missing(req, context_len, new_len)
        return all(self.pools[g].num_free >= m + spare for g, m in enumerate(missing))

    def reserve(self, req: Hashable, context_len: int, new_len: int) -> None:
        """Make the pages for a step that appends positions ``context_len .. new_len - 1``.

        First gives back pages that the window has passed (no query from ``context_len`` on reads
        them), then takes what is missing. Takes nothing if any group cannot be served.
        """
        if new_len < context_len:
            raise ValueError("new_len is less than context_len")
        held = self._held[req]
        self.release_passed(req, context_len)
        groups = range(len(self.groups))
        for g in groups:
            missing = self._missing(held, g, context_len, new_len)
            if self.pools[g].num_free < missing:
                raise OutOfPages(f"group {g}: {missing} pages wanted, {self.pools[g].num_free} free")
        for g in groups:
            table = held.tables[g]
            want = -(-new_len // self.page_size)
            if len(table) >= want:
                continue
            first = self._first_needed_page(g, context_len)
            while len(table) < want:
                table.append(self.pools[g].allocate(req) if len(table) >= first else NULL_PAGE)
            held.released[g] = max(held.released[g], min(first, len(table)))
            self._bump(held, g)
            self.max_blocks_per_seq = max(self.max_blocks_per_seq, len(table))
        held.length = max(held.length, new_len)

    def release_passed(self, req: Hashable, context_len: int) -> int:
        """Give back the pages of windowed groups that no query at ``context_len`` or later reads."""
        held = self._held[req]
        n = 0
        for g in range(len(self.groups)):
            if self.groups[g].window is None:
                continue
            table = held.tables[g]
            upto = min(self._first_needed_page(g, context_len), len(table))
            if upto <= held.released[g]:
                continue
            for i in range(held.released[g], upto):
                if table[i] != NULL_PAGE:
                    self.pools[g].free(table[i], req)
                    table[i] = NULL_PAGE
                    n += 1
            held.released[g] = upto
            self._bump(held, g)
        return n

    def free(self, req: Hashable) -> None:
        """Give back everything ``req`` holds: its pages in every group and its state slot."""
        held = self._held.pop(req, None)
        if held is None:
            raise ValueError(f"request {req!r} holds nothing (freed twice?)")
        for g, table in enumerate(held.tables):
            for page in table:
                if page != NULL_PAGE:
                    self.pools[g].free(page, req)
        self._free_slots.append(held.slot)

    # ------------------------------------------------------------------ checking
    def check_invariants(self) -> None:
        """No page lost, held twice or both free and held; no slot lost or shared."""
        slots = [h.slot for h in self._held.values()]
        assert len(set(slots)) == len(slots), "a state slot is held twice"
        assert not set(slots) & set(self._free_slots), "a state slot is both free and held"
        assert len(slots) + len(self._free_slots) == self.max_seqs, "a state slot is lost"
        for g, pool in enumerate(self.pools):
            seen: Dict[int, Hashable] = {}
            for req, held in self._held.items():
                for page in held.tables[g]:
                    if page == NULL_PAGE:
                        continue
                    assert page not in seen, f"group {g}: page {page} held by {seen[page]!r} and {req!r}"
                    seen[page] = req
                    assert pool.owner(page) == req, f"group {g}: page {page} owner mismatch"
            free = list(pool._free)
            assert len(set(free)) == len(free), f"group {g}: a page is in the free list twice"
            assert not set(free) & set(seen), f"group {g}: a page is both free and held"
            assert NULL_PAGE not in free and NULL_PAGE not in seen
            assert len(free) + len(seen) == pool.capacity, f"group {g}: {pool.capacity - len(free) - len(seen)} pages lost"
