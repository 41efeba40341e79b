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
out again without being cleared: a position beyond a request's length is never read.

Prefix sharing (off unless asked for; one group of unwindowed pages and no fixed-size state only),
after the reference's allocator (src/miniserve/paged.py:41-49,85-122, paged_engine.py:102-112,133-134):
a page that is full of tokens gets the hash of those tokens chained to the hash of the page before
it. A new request first takes over the pages whose hashes match the leading full pages of its
tokens (always leaving at least one token to compute), so several requests may hold one page: pages
carry a count of holders. A named page whose last holder has gone stays findable by its name until
every nameless idle page is in use and it is the one that was let go of longest ago.
"""
from __future__ import annotations

import hashlib
from collections import OrderedDict, deque
from typing import Dict, Hashable, List, Optional, Sequence

from .spec import NULL_PAGE, PagedKVSpec


class OutOfPages(Exception):
    """A group's pool has too few free pages for what was asked."""


class PagePool:
    """One group's pages. Page 0 is never handed out.

    A page is either in use (it has users: one request, or several with prefix sharing) or idle. The idle pages stand
    in ONE queue in the order in which they will be handed out: a page that carries no name goes to the head when its
    last user lets go (it is worth nothing, and was touched most recently), a named page (a full page of known tokens,
    findable by ``find``) goes to the tail. So names survive as long as any nameless page is left, and then the name
    that was let go of longest ago is given up first."""

    def __init__(self, num_pages: int):
        if num_pages < 2:
            raise ValueError("a pool needs at least 2 pages (page 0 is the null page)")
        self.num_pages = num_pages
        self._idle: "OrderedDict[int, None]" = OrderedDict((page, None) for page in range(1, num_pages))
        self._users: List[List[Hashable]] = [[] for _ in range(num_pages)]
        self._name_of: Dict[int, bytes] = {}
        self._page_named: Dict[bytes, int] = {}
        self.names_given_up = 0   # named pages that had to be handed out again because no nameless page was idle

    @property
    def capacity(self) -> int:
        return self.num_pages - 1

    @property
    def num_free(self) -> int:
        """Pages that ``allocate`` can hand out: every idle page, named or not."""
        return len(self._idle)

    def allocate(self, owner: Hashable = None) -> int:
        if not self._idle:
            raise OutOfPages()
        page, _ = self._idle.popitem(last=False)
        name = self._name_of.pop(page, None)
        if name is not None:  # the head of the queue is a named page only when every idle page is named
            del self._page_named[name]
            self.names_given_up += 1
        self._users[page] = [owner]
        return page

    def share(self, page: int, owner: Hashable = None) -> None:
        """One more user of a page that ``find`` returned; an idle page leaves the queue."""
        if not self._users[page]:
            del self._idle[page]
        self._users[page].append(owner)

    def free(self, page: int, owner: Hashable = None) -> None:
        """One user less; the last one makes the page idle."""
        if page == NULL_PAGE or not 0 < page < self.num_pages:
            raise ValueError(f"page {page} cannot be freed")
        users = self._users[page]
        if not users:
            raise ValueError(f"page {page} freed twice")
        if owner not in users:
            raise ValueError(f"page {page} belongs to {users!r}, not to {owner!r}")
        users.remove(owner)
        if not users:
            self._idle[page] = None                          # tail: behind every other idle page
            if page not in self._name_of:
                self._idle.move_to_end(page, last=False)     # nameless: to the head, the next to be handed out

    def holders(self, page: int) -> int:
        return len(self._users[page])

    def set_name(self, page: int, name: bytes) -> None:
        """Name a full page by the hash of its tokens. If another page already has the name, this one stays nameless."""
        if page not in self._name_of and name not in self._page_named:
            self._name_of[page] = name
            self._page_named[name] = page

    def find(self, name: bytes) -> Optional[int]:
        return self._page_named.get(name)

    def idle_pages(self) -> List[int]:
        """The idle pages in the order in which they would be handed out."""
        return list(self._idle)

    def name_of(self, page: int) -> Optional[bytes]:
        return self._name_of.get(page)


class _Held:
    """What one live request holds."""

    __slots__ = ("slot", "tables", "length", "versions", "released", "hashes")

    def __init__(self, slot: int, num_groups: int, version: int):
        self.slot = slot
        self.tables: List[List[int]] = [[] for _ in range(num_groups)]
        self.length = 0  # positions covered so far
        self.versions = [version] * num_groups  # changes whenever the group's table changes; never repeats
        self.released = [0] * num_groups        # pages below this index were given back (windowed groups)
        self.hashes: List[bytes] = []           # chained hashes of the leading full pages (prefix sharing)


class CacheManager:
    def __init__(self, groups: Sequence[PagedKVSpec], num_pages: int, page_size: int, max_seqs: int, prefix_sharing: bool = False):
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.groups = list(groups)
        self._windowed = any(g.window is not None for g in self.groups)
        # pages can only be shared where a request's pages are all it has: one group, no window (a windowed group gives pages
        # back as it goes), and the caller says that no fixed-size state exists (``prefix_sharing`` is its promise)
        self.prefix_sharing = bool(prefix_sharing) and len(self.groups) == 1 and self.groups[0].window is None
        self.shared_tokens = 0  # tokens that requests found in the cache instead of computing them
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

    # ------------------------------------------------------------------ prefix sharing
    def _chain(self, before: bytes, tokens: Sequence[int]) -> bytes:
        h = hashlib.blake2b(before, digest_size=16)
        h.update(b"".join(int(t).to_bytes(4, "little", signed=True) for t in tokens))
        return h.digest()

    def share_prefix(self, req: Hashable, tokens: Sequence[int]) -> int:
        """Right after ``admit``: take over the cached pages that hold the leading full pages of ``tokens``. Returns how
        many tokens they cover (a multiple of the page size, and less than ``len(tokens)``: one token at least is left to
        compute, src/miniserve/paged_engine.py:105-110)."""
        if not self.prefix_sharing:
            return 0
        held = self._held[req]
        if held.tables[0]:
            raise ValueError("share_prefix comes before the request's first reserve")
        pool, ps = self.pools[0], self.page_size
        digest = b""
        for i in range((len(tokens) - 1) // ps):
            digest = self._chain(digest, tokens[i * ps:(i + 1) * ps])
            page = pool.find(digest)
            if page is None:
                break
            pool.share(page, req)
            held.tables[0].append(page)
            held.hashes.append(digest)
        n = len(held.tables[0])
        if n:
            held.length = n * ps
            self._bump(held, 0)
            self.max_blocks_per_seq = max(self.max_blocks_per_seq, n)
            self.shared_tokens += n * ps
        return n * ps

    def register_full_pages(self, req: Hashable, tokens: Sequence[int]) -> None:
        """``tokens`` (from the request's first) are in the cache: name the pages they fill completely, so that later requests
        with the same leading tokens find them (src/miniserve/paged_engine.py:133-134)."""
        if not self.prefix_sharing:
            return
        held = self._held[req]
        pool, ps = self.pools[0], self.page_size
        full = min(len(tokens) // ps, len(held.tables[0]))
        while len(held.hashes) < full:
            i = len(held.hashes)
            digest = self._chain(held.hashes[-1] if held.hashes else b"", tokens[i * ps:(i + 1) * ps])
            held.hashes.append(digest)
            pool.set_name(held.tables[0][i], digest)

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
        want = -(-new_len // self.page_size)
        if not self._windowed:
            for table in held.tables:
                if len(table) < want:
                    break
            else:  # the usual decode step: the last page still has room
                if new_len > held.length:
                    held.length = new_len
                return
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
            holders: Dict[int, int] = {}
            for req, held in self._held.items():
                mine = [page for page in held.tables[g] if page != NULL_PAGE]
                assert len(set(mine)) == len(mine), f"group {g}: request {req!r} holds a page twice"
                for page in mine:
                    holders[page] = holders.get(page, 0) + 1
            for page, n in holders.items():
                assert pool.holders(page) == n, f"group {g}: page {page} has {n} holders, the pool counts {pool.holders(page)}"
                assert n == 1 or self.prefix_sharing, f"group {g}: page {page} is held {n} times"
            idle = pool.idle_pages()
            assert len(set(idle)) == len(idle), f"group {g}: a page is idle twice"
            assert not set(idle) & set(holders), f"group {g}: a page is both idle and held"
            assert NULL_PAGE not in idle and NULL_PAGE not in holders
            assert all(pool.holders(page) == 0 for page in idle), f"group {g}: an idle page has users"
            named = [pool.name_of(page) is not None for page in idle]
            assert named == sorted(named), f"group {g}: a named page would be handed out before a nameless one"
            assert all(pool.find(pool.name_of(page)) == page for page in range(1, pool.num_pages) if pool.name_of(page) is not None)
            lost = pool.capacity - len(idle) - len(holders)
            assert lost == 0, f"group {g}: {lost} pages lost"
