"""Page pool and slot table: plain host-side bookkeeping, no device code.

The reference allocates nothing of the kind: OPT's cache is one contiguous buffer per batch line
(src/transformers_neuronx/decoder.py:1761-1816), and for its paged layout the block tables come
from an external server (src/transformers_neuronx/base.py:357-395).  This allocator is what that
server would be.
"""
from __future__ import annotations

from typing import Dict, Hashable, List, Optional


class OutOfPages(RuntimeError):
    """Raised when a pool cannot give the pages asked for; nothing has been taken then."""


class PagePool:
    """Fixed number of pages; a last-freed-first-reused stack, so that a test with few pages uses
    a freed page again at once.  Every page has at most one owner; giving back a page that is not
    held, or that another owner holds, is an error."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError(f"a page pool needs at least one page, got {num_pages}")
        self.num_pages = int(num_pages)
        self._free: List[int] = list(range(self.num_pages - 1, -1, -1))   # pop() gives page 0 first
        self._owner: List[Optional[Hashable]] = [None] * self.num_pages
        self.reuse_count = 0           # pages handed out that had been used before
        self._ever_used = [False] * self.num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_used(self) -> int:
        return self.num_pages - len(self._free)

    def alloc(self, n: int, owner: Hashable) -> List[int]:
        if owner is None:
            raise ValueError("a page needs an owner")
        if n > len(self._free):
            raise OutOfPages(f"{n} page(s) asked for, {len(self._free)} free of {self.num_pages}")
        pages = []
        for _ in range(n):
            p = self._free.pop()
            assert self._owner[p] is None, f"page {p} is on the free list but held by {self._owner[p]!r}"
            self._owner[p] = owner
            if self._ever_used[p]:
                self.reuse_count += 1
            self._ever_used[p] = True
            pages.append(p)
        return pages

    def free(self, pages, owner: Hashable) -> None:
        for p in pages:
            if not (0 <= p < self.num_pages):
                raise ValueError(f"page {p} does not exist (pool of {self.num_pages})")
            if self._owner[p] is None:
                raise ValueError(f"page {p} freed twice")
            if self._owner[p] != owner:
                raise ValueError(f"page {p} is held by {self._owner[p]!r}, not by {owner!r}")
        for p in pages:
            self._owner[p] = None
            self._free.append(p)

    def transfer(self, pages, owner: Hashable, new_owner: Hashable) -> None:
        """Held pages change hands (a request continues from what another one holds)."""
        if new_owner is None:
            raise ValueError("a page needs an owner")
        for p in pages:
            if not (0 <= p < self.num_pages) or self._owner[p] != owner:
                raise ValueError(f"page {p} is not held by {owner!r}")
        for p in pages:
            self._owner[p] = new_owner

    def owner_of(self, page: int):
        return self._owner[page]

    def check(self) -> None:
        """Invariant: every page is either free exactly once or held by exactly one owner."""
        seen = [0] * self.num_pages
        for p in self._free:
            seen[p] += 1
        for p in range(self.num_pages):
            held = self._owner[p] is not None
            if seen[p] + (1 if held else 0) != 1:
                raise AssertionError(f"page {p}: on the free list {seen[p]} time(s), held={held}")


class SlotTable:
    """Slots for per-request state of fixed size (a position counter, sampling state, the state
    of a recurrent mixer).  A slot is taken when a request is admitted and returned when it ends."""

    def __init__(self, num_slots: int):
        if num_slots <= 0:
            raise ValueError("a slot table needs at least one slot")
        self.num_slots = int(num_slots)
        self._free = list(range(self.num_slots - 1, -1, -1))
        self._owner: Dict[int, Hashable] = {}

    @property
    def num_free(self) -> int:
        return len(self._free)

    def take(self, owner: Hashable) -> int:
        if not self._free:
            raise OutOfPages(f"all {self.num_slots} request slots are taken")
        s = self._free.pop()
        self._owner[s] = owner
        return s

    def give_back(self, slot: int, owner: Hashable) -> None:
        if self._owner.get(slot) != owner:
            raise ValueError(f"slot {slot} is not held by {owner!r}")
        del self._owner[slot]
        self._free.append(slot)

    def check(self) -> None:
        if sorted(self._free + list(self._owner)) != list(range(self.num_slots)):
            raise AssertionError("slot table lost or duplicated a slot")
