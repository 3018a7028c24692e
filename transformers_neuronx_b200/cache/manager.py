"""The cache manager: what each live request holds, in every group of caches.

A *cache* belongs to one entry of the model's schedule (or to several, when a layer reads another
layer's cache).  Caches whose needs agree (paged keys/values with the same window; or state of fixed
size) form a *group*; a group of paged caches has its own page pool and, per request, its own block
table, because a windowed group gives pages back while a request is still running and a full group
does not.  All caches of a group share the request's block table (page p of every layer in the
group belongs to the same request), as the reference's layers share one shape of cache
(src/transformers_neuronx/decoder.py:2263).

This file is host-side bookkeeping only; device storage is made by ``CacheStorage`` (storage.py)
from the same group descriptions.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

from .allocator import OutOfPages, PagePool, SlotTable


# What a mixer keeps between steps is described by a *need*: any (hashable, comparable) object with
#
#   group_key                    ("paged", window, ...) for a cache that lives in pages, anything else
#                                for state that is indexed by the request's slot; needs with equal
#                                keys share a page pool and the request's block table
#   window                       (paged needs) None, or how many last positions are read
#   make_storage(page_size, num_pages, max_slots, act_dtype, device) -> the device tensor
#   bytes_per_page(page_size, act_dtype)   (paged needs) for sizing a pool
#   clear_on_admission           True: the slot's row is zeroed when a request takes the slot
#
# The two kinds below are what the package's own mixers use; another kind (keys and values in a
# compressed form, in another element type, ...) is a class with this interface, defined anywhere:
# neither this file nor storage.py has to know it.
def _element_size(dtype) -> int:
    import torch
    return torch.empty((), dtype=dtype).element_size()


@dataclass(frozen=True)
class PagedKVNeed:
    """Keys and values of every position (window None) or of the last `window` positions, in the
    engine's activation type: one tensor [pages, 2 (key, value), n_kv_heads, page_size, head_dim]."""
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    clear_on_admission = False

    @property
    def group_key(self):
        return ("paged", self.window)

    def make_storage(self, page_size, num_pages, max_slots, act_dtype, device):
        import torch
        # zeroed once: the tensor-core attention multiplies rows that no token has written yet by
        # probabilities that are exactly zero, so they must hold finite numbers
        return torch.zeros((num_pages, 2, self.n_kv_heads, page_size, self.head_dim), dtype=act_dtype, device=device)

    def bytes_per_page(self, page_size, act_dtype) -> int:
        return 2 * self.n_kv_heads * page_size * self.head_dim * _element_size(act_dtype)


@dataclass(frozen=True)
class FixedStateNeed:
    """State of fixed size per request, e.g. of a recurrent mixer: shape and dtype name; one tensor
    [slots, *shape].  A request that takes a slot finds its row zeroed."""
    shape: Tuple[int, ...]
    dtype: str = "float32"
    clear_on_admission = True

    @property
    def group_key(self):
        return ("state",)

    def make_storage(self, page_size, num_pages, max_slots, act_dtype, device):
        import torch
        return torch.zeros((max_slots,) + tuple(self.shape), dtype=getattr(torch, self.dtype), device=device)


@dataclass
class GroupInfo:
    key: tuple
    cache_ids: List[int]
    window: Optional[int] = None

    @property
    def paged(self) -> bool:
        return self.key[0] == "paged"


def group_needs(needs: Dict[int, object]) -> List[GroupInfo]:
    """{cache id -> need} -> groups, in order of first appearance."""
    groups: Dict[tuple, GroupInfo] = {}
    for cid in sorted(needs):
        need = needs[cid]
        if need is None:
            continue
        k = need.group_key
        if k not in groups:
            groups[k] = GroupInfo(key=k, cache_ids=[], window=getattr(need, "window", None))
        groups[k].cache_ids.append(cid)
    return list(groups.values())


@dataclass
class _Request:
    slot: int
    length: int = 0                                   # tokens whose keys/values are in the cache
    tables: List[List[int]] = field(default_factory=list)   # per paged group: page of each block, -1 once released


class CacheManager:
    def __init__(self, groups: Sequence[GroupInfo], page_size: int, num_pages: int, max_slots: int):
        self.groups = list(groups)
        self.page_size = int(page_size)
        self.paged_groups = [g for g in self.groups if g.paged]
        self.pools = [PagePool(num_pages) for _ in self.paged_groups]
        self.slots = SlotTable(max_slots)
        self._req: Dict[Hashable, _Request] = {}
        self.on_slot_taken = None      # called with the slot when a request is admitted (the storage clears state there)

    # ---- queries ------------------------------------------------------------------------
    def __contains__(self, rid) -> bool:
        return rid in self._req

    def length(self, rid) -> int:
        return self._req[rid].length

    def slot(self, rid) -> int:
        return self._req[rid].slot

    def block_table(self, rid, group: int = 0) -> List[int]:
        return self._req[rid].tables[group]

    def live_requests(self):
        return list(self._req)

    def _first_needed_block(self, g: GroupInfo, length: int) -> int:
        """First block that a query at position >= length still reads."""
        if g.window is None:
            return 0
        first_pos = max(0, length - g.window + 1)
        return first_pos // self.page_size

    def pages_needed(self, rid, n_new: int) -> List[int]:
        """Pages each paged group must add so that `rid` can hold n_new more tokens."""
        r = self._req[rid]
        blocks_after = -(-(r.length + n_new) // self.page_size)
        return [max(0, blocks_after - len(t)) for t in r.tables]

    def pages_for_tokens(self, n_tokens: int) -> int:
        return -(-n_tokens // self.page_size)

    def can_append(self, rid, n_new: int) -> bool:
        return all(n <= p.num_free for n, p in zip(self.pages_needed(rid, n_new), self.pools))

    def free_pages(self) -> List[int]:
        return [p.num_free for p in self.pools]

    # ---- life of a request --------------------------------------------------------------
    def add_request(self, rid) -> int:
        if rid in self._req:
            raise ValueError(f"request {rid!r} is already live")
        slot = self.slots.take(rid)
        self._req[rid] = _Request(slot=slot, tables=[[] for _ in self.paged_groups])
        if self.on_slot_taken is not None:
            self.on_slot_taken(slot)
        return slot

    def append(self, rid, n_new: int) -> int:
        """Reserves room for n_new more tokens; returns the position of the first of them.
        Takes either all pages needed in all groups or none (OutOfPages)."""
        if n_new <= 0:
            raise ValueError("append needs at least one token")
        r = self._req[rid]
        need = self.pages_needed(rid, n_new)
        for n, pool in zip(need, self.pools):
            if n > pool.num_free:
                raise OutOfPages(f"request {rid!r} needs {n} page(s), {pool.num_free} free")
        for n, pool, table in zip(need, self.pools, r.tables):
            table.extend(pool.alloc(n, rid))
        start = r.length
        r.length += n_new
        return start

    def release_behind_window(self, rid) -> int:
        """After a step: pages that no later query of `rid` can read go back to their pool."""
        r = self._req[rid]
        n = 0
        for g, pool, table in zip(self.paged_groups, self.pools, r.tables):
            first = min(self._first_needed_block(g, r.length), len(table))
            gone = [p for p in table[:first] if p >= 0]
            if gone:
                pool.free(gone, rid)
                n += len(gone)
                for b in range(first):
                    table[b] = -1
        return n

    def free_request(self, rid) -> None:
        r = self._req.pop(rid)
        for pool, table in zip(self.pools, r.tables):
            pool.free([p for p in table if p >= 0], rid)
        self.slots.give_back(r.slot, rid)

    def reorder(self, rids: Sequence[Hashable], sources: Sequence[int]):
        """Request rids[i] goes on from what rids[sources[i]] holds now: what beam search asks of a cache
        after every step (the reference gathers whole cache lines by these indices,
        src/transformers_neuronx/decoder.py:2303-2320).  All named requests hold the same number of tokens.

        No page is allocated or freed: the first request to name a source takes over that source's pages
        as they are; every further one takes the pages of a request that nobody continues from, and
        those pages must be overwritten with the source's.  Returns (per paged group the list of
        (source page, destination page) to copy, the list of (source slot, destination slot) of state of
        fixed size to copy); the caller copies on the device before the next step."""
        n = len(rids)
        if len(sources) != n or len(set(rids)) != n or any(not (0 <= s < n) for s in sources):
            raise ValueError("reorder needs one source index (into the list of requests) per request")
        reqs = [self._req[r] for r in rids]
        if len({r.length for r in reqs}) > 1:
            raise ValueError("the requests of a reorder must hold the same number of tokens")
        old = [r.tables for r in reqs]
        first_claim, extra = {}, []
        for i, s in enumerate(sources):
            if s in first_claim:
                extra.append(i)
            else:
                first_claim[s] = i
        orphans = [u for u in range(n) if u not in first_claim]          # as many as there are further claims
        takes = {i: s for s, i in first_claim.items()}                    # destination -> whose tables it takes
        takes.update(dict(zip(extra, orphans)))
        copies = [[] for _ in self.paged_groups]
        for i, u in zip(extra, orphans):
            for g in range(len(self.paged_groups)):
                for ps, pd in zip(old[sources[i]][g], old[u][g]):
                    if (ps < 0) != (pd < 0):
                        raise AssertionError("requests of equal length differ in the blocks they still hold")
                    if ps >= 0:
                        copies[g].append((ps, pd))
        for i, j in takes.items():
            if i != j:
                for pool, table in zip(self.pools, old[j]):
                    pool.transfer([p for p in table if p >= 0], rids[j], rids[i])
        new_tables = {i: old[j] for i, j in takes.items()}
        for i, r in enumerate(reqs):
            r.tables = new_tables[i]
        slot_copies = [(reqs[s].slot, reqs[i].slot) for i, s in enumerate(sources) if s != i]
        return copies, slot_copies

    def slot_of_position(self, rid, pos: int, group: int = 0) -> int:
        """Physical row (page * page_size + offset) of a position in a paged group."""
        page = self._req[rid].tables[group][pos // self.page_size]
        if page < 0:
            raise ValueError(f"position {pos} of request {rid!r} lies behind the window: its page was released")
        return page * self.page_size + pos % self.page_size

    def check(self) -> None:
        """No page lost, held twice or freed twice; every held page is in its owner's table."""
        for gi, pool in enumerate(self.pools):
            pool.check()
            held = {}
            for rid, r in self._req.items():
                for p in r.tables[gi]:
                    if p < 0:
                        continue
                    if p in held:
                        raise AssertionError(f"page {p} of group {gi} is in the tables of {held[p]!r} and {rid!r}")
                    held[p] = rid
                    if pool.owner_of(p) != rid:
                        raise AssertionError(f"page {p} of group {gi}: table of {rid!r}, owner {pool.owner_of(p)!r}")
            if len(held) != pool.num_used:
                raise AssertionError(f"group {gi}: {pool.num_used} pages held, {len(held)} in tables")
        self.slots.check()
