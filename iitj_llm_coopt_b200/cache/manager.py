"""The cache manager: paged keys and values with a block table per request, and slots for
per-request state of fixed size.

Bookkeeping follows the reference's BlockManager (engine/block_manager.py:26-110: a pool of
fixed-size pages, free ids in a FIFO, a table of page ids per sequence, token p at slot
table[p // page] * page + p % page, `ensure` that raises before it allocates anything,
`free` at the end of a request).  What is added here:

* Groups.  Layers (cache entries) whose `CacheNeed` is equal share one group.  Each paged
  group has its own pool of pages, of its own size, its own table per request and its own
  rule for giving pages back: a group that keeps every token returns pages when the request
  ends; a group with a window also returns, after each step, the pages that every later
  query's window has passed (their table entry becomes -1 and is never read again).  A
  windowed group never holds more than a window and a step's new tokens per request, so its
  pool is sized for that (`pool_pages`), not for whole contexts.
  One page id addresses the same page in every cache entry of its group, as in the
  reference (engine/model.py:148-155: one K and V tensor per layer, same block ids).
* State slots.  Every admitted request holds one slot id in [0, max_requests); groups of
  kind "state" keep a [entries, max_requests, *state_shape] buffer indexed by it.  The
  slot exists even when no layer keeps state (Llama: zero bytes).

* State that starts at zero.  `admit` clears the request's slot in every state group, so a part
  with state never has to know whether a portion is a request's first.

Device storage of a paged group: [entries, pages of the group + 1, 2, kv_heads, page_size, head_dim] (the last
page is the group's padding page, never handed out)
(K plane then V plane of a page; one head's rows of a page are contiguous).
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

import numpy as np
import torch


class OutOfPages(Exception):
    """Raised by `ensure` when some group cannot provide the pages; nothing was allocated."""


class CacheError(RuntimeError):
    pass


class PagePool:
    """Free-list bookkeeping of one group's pages (host only)."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = num_pages
        self.free: deque = deque(range(num_pages))   # FIFO reuse, as engine/block_manager.py:30, 63-66
        self.held: set = set()

    @property
    def num_free(self) -> int:
        return len(self.free)

    def take(self) -> int:
        if not self.free:
            raise OutOfPages("no free page")
        p = self.free.popleft()
        self.held.add(p)
        return p

    def give(self, page: int) -> None:
        if page not in self.held:
            raise CacheError(f"page {page} is given back but is not held (freed twice?)")
        self.held.remove(page)
        self.free.append(page)


@dataclass
class PagedGroup:
    need: object
    entries: list                      # cache entry indices in this group, in order
    pool: PagePool
    page_size: int
    tables: dict = field(default_factory=dict)      # request -> [page id or -1]
    storage: torch.Tensor | None = None             # [entries, pages, 2, kv_heads, page_size, head_dim]
    # The tables once more, as the step function copies them to the device: row s holds the page ids of the
    # request in state slot s (0 where it has no page, or gave it back), the last row is the padding row.
    matrix: np.ndarray | None = None                # [max_requests + 1, columns] int32
    lengths: np.ndarray | None = None               # [max_requests + 1] int32: len(tables[request]) by slot

    def columns(self, n: int) -> None:
        """Makes room for tables of n pages."""
        if n > self.matrix.shape[1]:
            grown = np.zeros((self.matrix.shape[0], max(n, 2 * self.matrix.shape[1])), dtype=np.int32)
            grown[:, :self.matrix.shape[1]] = self.matrix
            self.matrix = grown

    def pages_for(self, tokens: int) -> int:
        return -(-tokens // self.page_size)

    def extra_pages(self, request, total_tokens: int) -> int:
        return max(0, self.pages_for(total_tokens) - len(self.tables.get(request, ())))

    def first_needed_page(self, stored_tokens: int) -> int:
        """Logical pages below this index hold no key that a query at position >= stored_tokens can see."""
        w = self.need.window
        if w <= 0:
            return 0
        return max(0, stored_tokens - w + 1) // self.page_size


@dataclass
class StateGroup:
    need: object
    entries: list
    storage: torch.Tensor | None = None             # [entries, max_requests, *state_shape]


class CacheManager:
    def __init__(self, needs: list, page_size: int, num_pages: int, max_requests: int,
                 dtype: torch.dtype = torch.bfloat16, device=None, max_step_tokens: int | None = None):
        """needs[i] is the CacheNeed of cache entry i.  `num_pages` is the pool of a group that keeps every token;
        a group with a window gets `pool_pages(...)` pages if `max_step_tokens` (the most tokens one step brings)
        is given, else `num_pages` too.  `device=None` keeps bookkeeping only (no storage is allocated), which is
        all the scheduler and the CPU tests use."""
        self.page_size, self.num_pages, self.max_requests = page_size, num_pages, max_requests
        self.dtype, self.device, self.max_step_tokens = dtype, device, max_step_tokens
        self.groups: list = []
        self.entry_group: list = []       # entry -> (group index, index of the entry inside the group)
        by_need: dict = {}
        for entry, need in enumerate(needs):
            if need.kind == "none":
                self.entry_group.append((None, 0))
                continue
            if need not in by_need:
                by_need[need] = len(self.groups)
                if need.kind == "paged_kv":
                    pages = self.pool_pages(need, page_size, num_pages, max_requests, max_step_tokens)
                    self.groups.append(PagedGroup(need, [], PagePool(pages), page_size))
                elif need.kind == "state":
                    self.groups.append(StateGroup(need, []))
                else:
                    raise ValueError(f"unknown cache need kind {need.kind!r}")
            g = by_need[need]
            self.entry_group.append((g, len(self.groups[g].entries)))
            self.groups[g].entries.append(entry)
        self.paged = [i for i, g in enumerate(self.groups) if isinstance(g, PagedGroup)]
        self.windowed = any(self.groups[i].need.window > 0 for i in self.paged)
        for i in self.paged:
            g = self.groups[i]
            g.matrix = np.zeros((max_requests + 1, 16), dtype=np.int32)
            g.matrix[max_requests, 0] = g.pool.num_pages     # the padding row: one page, the group's padding page
            g.lengths = np.zeros(max_requests + 1, dtype=np.int32)
            g.lengths[max_requests] = 1
        # per-request records
        self.stored: dict = {}            # request -> tokens whose keys/values (or state) are in the cache
        self.room: dict = {}              # request -> tokens that the pages it holds can take (least over the groups)
        self.slot_of: dict = {}           # request -> state slot
        self.free_slots: deque = deque(range(max_requests))
        self._views: dict = {}
        if device is not None:
            self._allocate()

    # ---- storage -------------------------------------------------------------------------
    def _allocate(self) -> None:
        for g in self.groups:
            if isinstance(g, PagedGroup):
                n = g.need
                # one page more than the pool hands out: the group's padding page.  Rows that only pad a batch to a
                # size with a captured graph read and write there (the reference keeps such a scratch page too,
                # engine/engine.py:207-211)
                g.storage = torch.zeros((len(g.entries), g.pool.num_pages + 1, 2, n.kv_heads, self.page_size, n.head_dim),
                                        dtype=self.dtype, device=self.device)
            else:
                dt = getattr(torch, g.need.state_dtype)
                g.storage = torch.zeros((len(g.entries), self.max_requests + 1) + tuple(g.need.state_shape),
                                        dtype=dt, device=self.device)

    @staticmethod
    def pool_pages(need, page_size: int, num_pages: int, max_requests: int, max_step_tokens: int | None) -> int:
        """Pages of the pool of a paged group.  A group that keeps every token gets `num_pages`.  A group with a
        window holds, per request, the pages its window touches (window / page, and one more at either end) and,
        until the step is over, the pages of the step's new tokens, of which all requests together bring at most
        `max_step_tokens`: that, if it is less."""
        if need.window <= 0 or max_step_tokens is None:
            return num_pages
        per_request = -(-need.window // page_size) + 2
        return min(num_pages, max_requests * per_request + -(-max_step_tokens // page_size) + max_requests)

    @property
    def pad_slot(self) -> int:
        """The state slot of padding rows."""
        return self.max_requests

    @staticmethod
    def bytes_for(needs: list, page_size: int, num_pages: int, itemsize: int, max_requests: int,
                  max_step_tokens: int | None) -> int:
        """Bytes of the paged storage with `num_pages` pages: every cache entry pays for the pages of its group's pool."""
        return sum(2 * n.kv_heads * n.head_dim * page_size * itemsize
                   * (CacheManager.pool_pages(n, page_size, num_pages, max_requests, max_step_tokens) + 1)
                   for n in needs if n.kind == "paged_kv")

    @staticmethod
    def pages_for_bytes(needs: list, page_size: int, budget_bytes: float, itemsize: int, max_requests: int,
                        max_step_tokens: int | None) -> int:
        """The largest `num_pages` whose paged storage fits `budget_bytes` (0 if not even one page does)."""
        def cost(pages):
            return CacheManager.bytes_for(needs, page_size, pages, itemsize, max_requests, max_step_tokens)
        if cost(1) > budget_bytes:
            return 0
        lo, hi = 1, 2
        while cost(hi) <= budget_bytes and hi < (1 << 40):
            lo, hi = hi, hi * 2
        while hi - lo > 1:                         # cost is monotone in the page count
            mid = (lo + hi) // 2
            lo, hi = (mid, hi) if cost(mid) <= budget_bytes else (lo, mid)
        return lo

    def view(self, entry: int):
        """(group index, storage of that cache entry): [pages, 2, kv_heads, page, head_dim] or
        [max_requests, *state_shape]."""
        cached = self._views.get(entry)
        if cached is not None:
            return cached
        g, local = self.entry_group[entry]
        if g is None:
            return None, None
        storage = self.groups[g].storage
        self._views[entry] = (g, storage[local] if storage is not None else None)
        return self._views[entry]

    # ---- requests ------------------------------------------------------------------------
    def admit(self, request) -> int:
        """Registers a request (no tokens stored yet) and gives it a state slot."""
        if request in self.stored:
            raise CacheError(f"request {request!r} is already admitted")
        if not self.free_slots:
            raise CacheError(f"all {self.max_requests} request slots are in use")
        self.stored[request] = 0
        slot = self.slot_of[request] = self.free_slots.popleft()
        for g in self.groups:
            if isinstance(g, PagedGroup):
                g.tables[request] = []
                g.lengths[slot] = 0
            elif g.storage is not None:
                g.storage[:, slot].zero_()         # state starts at zero, whoever held the slot before
        self._set_room(request)
        return slot

    def has(self, request) -> bool:
        return request in self.stored

    def num_tokens(self, request) -> int:
        return self.stored[request]

    def release(self, request) -> int:
        """Gives back everything the request holds; returns the number of pages returned."""
        if request not in self.stored:
            raise CacheError(f"request {request!r} is not admitted (released twice?)")
        n = 0
        slot = self.slot_of[request]
        for gi in self.paged:
            g = self.groups[gi]
            table = g.tables.pop(request)
            for p in table:
                if p >= 0:
                    g.pool.give(p)
                    n += 1
            g.matrix[slot, :len(table)] = 0
            g.lengths[slot] = 0
        self.free_slots.append(self.slot_of.pop(request))
        del self.stored[request]
        del self.room[request]
        return n

    # ---- capacity ------------------------------------------------------------------------
    @property
    def num_free(self) -> int:
        """Free pages of the paged group with the fewest."""
        return min((self.groups[gi].pool.num_free for gi in self.paged), default=self.num_pages)

    @property
    def usage(self) -> float:
        """The fullest paged group's share of pages in use."""
        return max((1.0 - self.groups[gi].pool.num_free / self.groups[gi].pool.num_pages for gi in self.paged), default=0.0)

    @property
    def capacity_tokens(self) -> int:
        """Tokens a lone request can hold: what the pools of the groups that keep every token take."""
        full = [self.groups[gi].pool.num_pages for gi in self.paged if self.groups[gi].need.window <= 0]
        return min(full, default=self.num_pages) * self.page_size

    def can_admit(self, tokens: int, watermark: float = 0.0) -> bool:
        """True if a new request's first `tokens` tokens fit every paged group while `watermark` of the group's
        pool stays free (the reference's admission rule, engine/engine.py:124-140, per group)."""
        for gi in self.paged:
            g = self.groups[gi]
            if g.pages_for(tokens) > g.pool.num_free - int(watermark * g.pool.num_pages):
                return False
        return True

    def can_grow_all(self, totals: list) -> bool:
        """True if every (request, total tokens) of `totals` can be served at once: per group, the new pages all of
        them need together are free."""
        for gi in self.paged:
            g = self.groups[gi]
            need = sum(g.extra_pages(r, t) for r, t in totals if t > self.room.get(r, 0))
            if need > g.pool.num_free:
                return False
        return True

    def extra_pages_needed(self, request, total_tokens: int) -> int:
        """Largest number of new pages any group needs so the request can hold total_tokens."""
        if total_tokens <= self.room.get(request, 0):
            return 0
        return max((self.groups[gi].extra_pages(request, total_tokens) for gi in self.paged), default=0)

    def can_fit(self, request, total_tokens: int) -> bool:
        if total_tokens <= self.room.get(request, 0):
            return True
        return all(self.groups[gi].extra_pages(request, total_tokens) <= self.groups[gi].pool.num_free
                   for gi in self.paged)

    def ensure(self, request, total_tokens: int) -> None:
        """Grow the request's tables so they can hold total_tokens tokens; all groups or none."""
        room = self.room.get(request)
        if room is None:
            raise CacheError(f"request {request!r} is not admitted")
        if total_tokens <= room:
            return
        for gi in self.paged:
            g = self.groups[gi]
            need = g.extra_pages(request, total_tokens)
            if need > g.pool.num_free:
                raise OutOfPages(f"request {request!r} needs {need} pages in group {gi}, {g.pool.num_free} free")
        slot = self.slot_of[request]
        for gi in self.paged:
            g = self.groups[gi]
            table = g.tables[request]
            old = len(table)
            for _ in range(g.extra_pages(request, total_tokens)):
                table.append(g.pool.take())
            if len(table) > old:
                g.columns(len(table))
                g.matrix[slot, old:len(table)] = table[old:]
                g.lengths[slot] = len(table)
        self._set_room(request)

    def _set_room(self, request) -> None:
        self.room[request] = min((len(self.groups[gi].tables[request]) * self.page_size for gi in self.paged), default=1 << 62)

    def advance(self, request, total_tokens: int) -> None:
        """Records that the cache now holds the request's first total_tokens tokens, and gives
        back the pages that a window has passed."""
        if total_tokens < self.stored[request]:
            raise CacheError("advance cannot go backwards; use truncate")
        if total_tokens > self.room[request]:
            raise CacheError(f"request {request!r}: {total_tokens} tokens exceed its reserved pages")
        self.stored[request] = total_tokens
        if not self.windowed:
            return
        slot = self.slot_of[request]
        for gi in self.paged:
            g = self.groups[gi]
            table = g.tables[request]
            for lp in range(min(g.first_needed_page(total_tokens), len(table))):
                if table[lp] >= 0:
                    g.pool.give(table[lp])
                    table[lp] = -1
                    g.matrix[slot, lp] = 0

    def advance_all(self, requests: list, totals: list) -> None:
        """`advance` for every request of a step."""
        if self.windowed:
            for request, total in zip(requests, totals):
                self.advance(request, total)
            return
        stored, room = self.stored, self.room
        for request, total in zip(requests, totals):
            if total < stored[request]:
                raise CacheError("advance cannot go backwards; use truncate")
            if total > room[request]:
                raise CacheError(f"request {request!r}: {total} tokens exceed its reserved pages")
            stored[request] = total

    def truncate(self, request, total_tokens: int) -> None:
        """Forget tokens beyond total_tokens and give back the trailing pages
        (engine/block_manager.py:95-103).  Not possible across pages a window already released."""
        for gi in self.paged:
            g = self.groups[gi]
            table = g.tables[request]
            keep = g.pages_for(total_tokens)
            if any(p < 0 for p in table[g.first_needed_page(total_tokens):keep]):
                raise CacheError("truncate would need pages that a window already gave back")
            old = len(table)
            while len(table) > keep:
                p = table.pop()
                if p >= 0:
                    g.pool.give(p)
            if old > keep:
                g.matrix[self.slot_of[request], keep:old] = 0
                g.lengths[self.slot_of[request]] = keep
        self.stored[request] = min(self.stored[request], total_tokens)
        self._set_room(request)

    # ---- what the step function needs ----------------------------------------------------
    def table(self, group: int, request) -> list:
        return self.groups[group].tables[request]

    def slots(self, group: int, request, start: int, end: int) -> list:
        """Cache slot (page * page_size + offset) of positions [start, end)."""
        table, ps = self.groups[group].tables[request], self.page_size
        out = []
        for p in range(start, end):
            page = table[p // ps]
            if page < 0:
                raise CacheError(f"request {request!r}: position {p} lies in a page already given back")
            out.append(page * ps + p % ps)
        return out

    def state_slot(self, request) -> int:
        return self.slot_of[request]

    # ---- invariants (tests) --------------------------------------------------------------
    def check(self) -> None:
        """Every page is either free or in exactly one table; slots likewise."""
        for gi in self.paged:
            g = self.groups[gi]
            in_tables = [p for t in g.tables.values() for p in t if p >= 0]
            if len(in_tables) != len(set(in_tables)):
                raise CacheError(f"group {gi}: a page is held twice")
            if set(in_tables) != g.pool.held:
                raise CacheError(f"group {gi}: tables and pool disagree about held pages")
            free = list(g.pool.free)
            if len(free) != len(set(free)) or set(free) & g.pool.held:
                raise CacheError(f"group {gi}: free list is inconsistent")
            if len(free) + len(in_tables) != g.pool.num_pages:
                raise CacheError(f"group {gi}: {g.pool.num_pages - len(free) - len(in_tables)} pages are lost")
            if set(g.tables) != set(self.stored):
                raise CacheError(f"group {gi}: tables exist for other requests than the admitted ones")
            rows = np.zeros_like(g.matrix)
            rows[self.max_requests, 0] = g.pool.num_pages
            sizes = np.zeros_like(g.lengths)
            sizes[self.max_requests] = 1
            for request, table in g.tables.items():
                rows[self.slot_of[request], :len(table)] = [max(p, 0) for p in table]
                sizes[self.slot_of[request]] = len(table)
            if not (np.array_equal(rows, g.matrix) and np.array_equal(sizes, g.lengths)):
                raise CacheError(f"group {gi}: the table matrix differs from the tables")
        used = list(self.slot_of.values())
        if len(used) != len(set(used)) or set(used) & set(self.free_slots) or \
                len(used) + len(self.free_slots) != self.max_requests:
            raise CacheError("state slots are inconsistent")
        for request in self.stored:
            want = min((len(self.groups[gi].tables[request]) * self.page_size for gi in self.paged), default=1 << 62)
            if self.room.get(request) != want:
                raise CacheError(f"request {request!r}: recorded room {self.room.get(request)} but its pages take {want}")
