"""Pages of one cache group: who holds them, which are free, which are kept for
reuse by a later prompt with the same beginning.

Behaviour follows the reference's `BlockAllocator` (qwen-infer/src/paged.rs:
119-519): the free pages form a stack (the page freed last is handed out
first, the first page ever handed out is 0); a page has a count of holders;
`take_n` is all-or-nothing; a full page of a prompt can be published under the
chained hash of its token ids, and a page whose last holder leaves stays
"kept" (out of the free stack, least-recently-kept first in line for eviction)
when it is published; a lookup compares the parent page and the stored ids, so
two different pages with the same hash never share.
"""
from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

_FNV_OFFSET = 0xCBF29CE484222325
_FNV_PRIME = 0x100000001B3
_MASK = (1 << 64) - 1


class PageError(RuntimeError):
    """A page was freed twice, is unknown, or was published while not full."""


def prefix_hash(parent: int, tokens: Sequence[int]) -> int:
    """paged.rs:93-100: (offset ^ parent), then for each id: xor, multiply."""
    value = _FNV_OFFSET ^ parent
    for token in tokens:
        value ^= int(token) & 0xFFFFFFFF
        value = (value * _FNV_PRIME) & _MASK
    return value


def pages_for(length: int, page_size: int) -> int:
    return (length + page_size - 1) // page_size


@dataclass
class _Published:
    page: int
    parent_hash: int
    parent_page: Optional[int]
    tokens: Tuple[int, ...]


class PageAllocator:
    def __init__(self, num_pages: int, page_size: int):
        if num_pages < 0 or page_size <= 0:
            raise ValueError("a pool has a page count >= 0 and a page size > 0")
        self.capacity = num_pages
        self.page_size = page_size
        self._stack: List[int] = list(range(num_pages - 1, -1, -1))
        self._holders = [0] * num_pages
        self._hash_of: List[Optional[int]] = [None] * num_pages
        self._index: Dict[int, _Published] = {}
        self._kept: "OrderedDict[int, None]" = OrderedDict()   # published, no holder; oldest first
        self.live = 0
        self.peak_live = 0
        self.peak_occupied = 0

    # ---- counts -----------------------------------------------------------
    @property
    def free_count(self) -> int:
        return len(self._stack)

    @property
    def kept_count(self) -> int:
        return len(self._kept)

    @property
    def available(self) -> int:
        """Pages a caller can get now: free ones plus kept ones (evictable)."""
        return len(self._stack) + len(self._kept)

    @property
    def occupied(self) -> int:
        return self.live + len(self._kept)

    def holders(self, page: int) -> int:
        self._known(page)
        return self._holders[page]

    def all_released(self) -> bool:
        return self.live == 0 and not any(self._holders)

    def _known(self, page: int) -> None:
        if not isinstance(page, int) or not 0 <= page < self.capacity:
            raise PageError(f"page {page} was not issued by this allocator")

    def _peaks(self) -> None:
        self.peak_live = max(self.peak_live, self.live)
        self.peak_occupied = max(self.peak_occupied, self.occupied)

    # ---- taking and giving back ----------------------------------------------
    def take(self) -> Optional[int]:
        if self._stack:
            page = self._stack.pop()
        elif self._kept:
            page, _ = self._kept.popitem(last=False)
            self._forget(page)
        else:
            return None
        self._holders[page] = 1
        self.live += 1
        self._peaks()
        return page

    def take_n(self, n: int) -> Optional[List[int]]:
        if n > self.available:
            return None
        return [self.take() for _ in range(n)]

    def give_back(self, page: int) -> str:
        """One holder leaves.  Returns "shared" (others still hold it), "kept"
        (published, stays for reuse) or "freed" (back on the stack)."""
        self._known(page)
        if self._holders[page] == 0:
            raise PageError(f"double free of page {page}")
        self._holders[page] -= 1
        if self._holders[page]:
            return "shared"
        self.live -= 1
        if self._hash_of[page] is not None:
            self._kept[page] = None
            self._peaks()
            return "kept"
        self._stack.append(page)
        return "freed"

    def hold(self, page: int) -> None:
        """One more holder; revives a kept page."""
        self._known(page)
        if self._holders[page] == 0:
            if page not in self._kept:
                raise PageError(f"page {page} is free; it cannot gain a holder")
            del self._kept[page]
            self.live += 1
            self._peaks()
        self._holders[page] += 1

    def evict_kept(self) -> None:
        """Turn every kept page into a free one (oldest first)."""
        while self._kept:
            page, _ = self._kept.popitem(last=False)
            self._forget(page)
            self._stack.append(page)

    # ---- sharing the beginnings of prompts --------------------------------------
    def _forget(self, page: int) -> None:
        value = self._hash_of[page]
        self._hash_of[page] = None
        if value is not None and value in self._index and self._index[value].page == page:
            del self._index[value]

    def _lookup(self, value, parent_hash, parent_page, tokens) -> Optional[int]:
        entry = self._index.get(value)
        if entry is None or entry.parent_hash != parent_hash or entry.parent_page != parent_page \
                or entry.tokens != tuple(tokens):
            return None
        return entry.page

    def _publish(self, value, parent_hash, parent_page, tokens, page) -> None:
        if value in self._index or self._hash_of[page] is not None:
            return  # first publisher wins; a page is published once
        self._index[value] = _Published(page, parent_hash, parent_page, tuple(tokens))
        self._hash_of[page] = value

    def publish_prompt(self, tokens: Sequence[int], pages: Sequence[int], resume=None):
        """Publish every full page of a prompt, chained from its start; stops at
        the first page that cannot be found again under its own hash.  Returns where it
        got to, (pages done, their chain's hash, the last page) or None when the chain broke;
        handed back as `resume` with more tokens of the same prompt, the walk goes on from
        there instead of hashing the beginning again."""
        size = self.page_size
        first, parent_hash, parent_page = resume if resume is not None else (0, 0, None)
        for at in range(first, min(len(tokens) // size, len(pages))):
            chunk = tuple(int(t) for t in tokens[at * size:(at + 1) * size])
            page = pages[at]
            if page < 0 or self._holders[page] == 0:
                return None
            value = prefix_hash(parent_hash, chunk)
            self._publish(value, parent_hash, parent_page, chunk, page)
            if self._lookup(value, parent_hash, parent_page, chunk) != page:
                return None
            parent_hash, parent_page, first = value, page, at + 1
        return first, parent_hash, parent_page

    def take_shared_prefix(self, tokens: Sequence[int]) -> List[int]:
        """Pages that already hold the beginning of `tokens`, full pages only,
        from the start up to the first miss; each gains a holder."""
        size = self.page_size
        parent_hash, parent_page = 0, None
        shared: List[int] = []
        for at in range(len(tokens) // size):
            chunk = tuple(int(t) for t in tokens[at * size:(at + 1) * size])
            value = prefix_hash(parent_hash, chunk)
            page = self._lookup(value, parent_hash, parent_page, chunk)
            if page is None:
                break
            self.hold(page)
            shared.append(page)
            parent_hash, parent_page = value, page
        return shared

    # ---- invariants, for tests ---------------------------------------------------
    def check(self) -> None:
        """Every page is in exactly one place: free, kept, or held."""
        free, kept = set(self._stack), set(self._kept)
        if len(free) != len(self._stack):
            raise PageError("a page is on the free stack twice")
        held = {p for p in range(self.capacity) if self._holders[p] > 0}
        if free & kept or free & held or kept & held:
            raise PageError("a page is in two places at once")
        if len(free) + len(kept) + len(held) != self.capacity:
            raise PageError("a page was lost")
        if len(held) != self.live:
            raise PageError("the live count does not match the holders")
