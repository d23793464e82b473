"""The cache manager: keys and values in pages with a block table per request,
and slots for per-request state of fixed size.

Calls of the model's order whose mixers need the same kind of storage (the
same kv heads, head size and window) form a *group*.  A group owns its pages
(an allocator and one device pool) and every request has one block table per
group, because groups differ in what they keep: a group of all keys keeps every
page of a request, a group with a window gives a page back as soon as the
window has passed it.  Inside a group every call has its own layer of the pool,
addressed by the same table.  Beside the pages the manager owns the state
arenas: one tensor [state slots, *shape] per call whose mixer declares state;
a request takes one slot index when it opens (zeroed) and returns it when it
closes.  A model without state still gets slot indices: the arena is empty.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

from .allocator import PageAllocator, PageError, pages_for


class OutOfPages(RuntimeError):
    """The pool cannot hold what was asked; nothing was taken."""


@dataclass
class GroupLayout:
    kv_heads: int
    head_dim: int
    window: Optional[int]
    calls: List[int] = field(default_factory=list)   # calls of the order that write here


@dataclass
class RequestCache:
    """One request's hold on the cache: per group a block table (logical block
    -> page, -1 for a block not held), the tokens stored, the state slot."""

    request_id: object
    tables: List[List[int]]
    length: int = 0
    state_slot: int = -1
    closed: bool = False
    published: object = None     # where publishing the prompt's pages got to (None: not begun; False: broken)

    def pages_held(self, group: int) -> List[int]:
        return [p for p in self.tables[group] if p >= 0]


def plan_groups(needs) -> (List[GroupLayout], List[Optional[int]]):
    """Group the calls by what their mixer stores per token.  Returns the
    groups and, for each call, its group (None for a call without keys)."""
    groups: List[GroupLayout] = []
    group_of: List[Optional[int]] = []
    for call, need in enumerate(needs):
        if need is None or need.kv is None:
            group_of.append(None)
            continue
        key = (need.kv.kv_heads, need.kv.head_dim, need.kv.window)
        for g, layout in enumerate(groups):
            if (layout.kv_heads, layout.head_dim, layout.window) == key:
                break
        else:
            groups.append(GroupLayout(*key))
            g = len(groups) - 1
        groups[g].calls.append(call)
        group_of.append(g)
    return groups, group_of


class CachePlan:
    """The host side of the cache: allocators, tables, state slots.  It touches
    no device memory, so it is what the CPU tests exercise."""

    def __init__(self, needs, num_pages: int, page_size: int, max_requests: int,
                 share_prefixes: bool = False):
        self.page_size = page_size
        self.num_pages = num_pages
        self.max_requests = max_requests
        self.groups, self.group_of_call = plan_groups(needs)
        self.state_calls = [c for c, n in enumerate(needs) if n is not None and n.state is not None]
        self.allocators = [PageAllocator(num_pages, page_size) for _ in self.groups]
        self._free_slots = list(range(max_requests - 1, -1, -1))
        self.requests: Dict[object, RequestCache] = {}
        shareable = len(self.groups) == 1 and self.groups[0].window is None and not self.state_calls
        self.share_prefixes = bool(share_prefixes and shareable)

    # ---- requests ------------------------------------------------------------
    def open(self, request_id) -> RequestCache:
        if request_id in self.requests:
            raise ValueError(f"request {request_id!r} is already open")
        if not self._free_slots:
            raise OutOfPages(f"all {self.max_requests} request slots are in use")
        cache = RequestCache(request_id, [[] for _ in self.groups], 0, self._free_slots.pop())
        self.requests[request_id] = cache
        self.on_open(cache)
        return cache

    def on_open(self, cache: RequestCache) -> None:
        """Hook for the device side (zeroing the state slot)."""

    def first_needed_block(self, group: int, position: int) -> int:
        """The first logical block a query at `position` can still read."""
        window = self.groups[group].window
        if window is None:
            return 0
        return max(0, position - window) // self.page_size

    def pages_missing(self, cache: RequestCache, n_new: int) -> List[int]:
        """Per group, the pages a step of `n_new` more tokens still needs."""
        missing = []
        end_block = pages_for(cache.length + n_new, self.page_size)
        for g in range(len(self.groups)):
            table = cache.tables[g]
            if self.groups[g].window is None:
                # a table of all keys has no holes (every reserve fills it from block 0 on and
                # nothing is given back before the end): only blocks past its end are missing
                missing.append(max(0, end_block - len(table)))
                continue
            first = self.first_needed_block(g, cache.length)
            count = sum(1 for b in range(first, end_block) if b >= len(table) or table[b] < 0)
            missing.append(count)
        return missing

    def can_reserve(self, cache: RequestCache, n_new: int) -> bool:
        return all(m <= a.available for m, a in zip(self.pages_missing(cache, n_new), self.allocators))

    def reserve(self, cache: RequestCache, n_new: int) -> None:
        """Make sure pages exist for positions length .. length + n_new - 1 in
        every group; all or nothing."""
        if cache.closed:
            raise ValueError("the request is closed")
        if n_new < 0:
            raise ValueError("a step brings at least no tokens")
        missing = self.pages_missing(cache, n_new)
        for m, allocator in zip(missing, self.allocators):
            if m > allocator.available:
                raise OutOfPages(
                    f"request {cache.request_id!r} needs {m} more pages, {allocator.available} are left")
        end_block = pages_for(cache.length + n_new, self.page_size)
        for g, allocator in enumerate(self.allocators):
            table = cache.tables[g]
            if self.groups[g].window is None:
                while len(table) < end_block:          # no holes below the table's end (see pages_missing)
                    table.append(allocator.take())
                continue
            first = self.first_needed_block(g, cache.length)
            while len(table) < end_block:
                table.append(-1)
            for b in range(first, end_block):
                if table[b] < 0:
                    table[b] = allocator.take()

    def commit(self, cache: RequestCache, n_new: int) -> None:
        """The step ran: the request now holds n_new more tokens.  Pages that
        every later query's window has passed are given back."""
        cache.length += n_new
        for g, allocator in enumerate(self.allocators):
            if self.groups[g].window is None:
                continue
            table = cache.tables[g]
            for b in range(min(self.first_needed_block(g, cache.length), len(table))):
                if table[b] >= 0:
                    allocator.give_back(table[b])
                    table[b] = -1

    def adopt_prefix(self, cache: RequestCache, tokens: Sequence[int]) -> int:
        """Start a fresh request on pages that already hold the beginning of
        `tokens` (full pages only).  Returns the number of tokens adopted."""
        if not self.share_prefixes or cache.length or cache.tables[0]:
            return 0
        shared = self.allocators[0].take_shared_prefix(tokens)
        cache.tables[0] = list(shared)
        cache.length = len(shared) * self.page_size
        return cache.length

    def publish_prompt(self, cache: RequestCache, tokens: Sequence[int]) -> None:
        """Offer the full pages that hold `tokens` (the beginning of the request's prompt, as far
        as it is computed) to later requests.  Called again with more of the same prompt, only
        the pages that are new are hashed."""
        if not self.share_prefixes:
            return
        resume = cache.published
        if resume is False:
            return                       # the chain broke earlier: nothing behind it can be found
        cache.published = self.allocators[0].publish_prompt(tokens, cache.tables[0], resume)
        if cache.published is None:
            cache.published = False

    def release_pages(self, cache: RequestCache) -> None:
        """Give back every page (the request stays open with nothing stored):
        what preemption does before a later recompute."""
        for g, allocator in enumerate(self.allocators):
            for page in cache.tables[g]:
                if page >= 0:
                    allocator.give_back(page)
            cache.tables[g] = []
        cache.length = 0
        cache.published = None

    def close(self, cache: RequestCache) -> None:
        if cache.closed:
            raise PageError(f"request {cache.request_id!r} was closed twice")
        self.release_pages(cache)
        cache.closed = True
        self._free_slots.append(cache.state_slot)
        del self.requests[cache.request_id]

    # ---- sizes ------------------------------------------------------------------
    def pages_for_tokens(self, n_tokens: int) -> int:
        return pages_for(n_tokens, self.page_size)

    def check(self) -> None:
        """No page lost, none held twice by mistake: holders match the tables."""
        for g, allocator in enumerate(self.allocators):
            allocator.check()
            counts: Dict[int, int] = {}
            for cache in self.requests.values():
                for page in cache.tables[g]:
                    if page >= 0:
                        counts[page] = counts.get(page, 0) + 1
                    elif self.groups[g].window is None:
                        raise PageError(f"group {g} keeps all keys, yet request "
                                        f"{cache.request_id!r} has a hole in its table")
            for page in range(allocator.capacity):
                if allocator.holders(page) != counts.get(page, 0):
                    raise PageError(
                        f"group {g} page {page}: {allocator.holders(page)} holders, "
                        f"{counts.get(page, 0)} table entries")
        slots = [c.state_slot for c in self.requests.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots):
            raise PageError("a state slot is held twice")
        if len(slots) + len(self._free_slots) != self.max_requests:
            raise PageError("a state slot was lost")
