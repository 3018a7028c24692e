"""Device memory of the caches.  Each cache's need (cache/manager.py) makes its own tensor: for
paged keys and values [pages, 2 (key, value), n_kv_heads, page_size, head_dim] in the activation
type, for state of fixed size [slots, *shape].  What a request may read is decided by its own
length and block table, never by the contents of a page; pages are not cleared when they change
hands.  State of fixed size is different: a request that takes a slot must not see the last
owner's state, so its row is zeroed at admission (``clear_slot``)."""
from __future__ import annotations

from typing import Dict, List

import torch

from .manager import GroupInfo


class CacheStorage:
    def __init__(self, needs: Dict[int, object], groups: List[GroupInfo], page_size: int, num_pages: int,
                 max_slots: int, act_dtype, device):
        self.page_size, self.num_pages, self.max_slots = page_size, num_pages, max_slots
        self._tensors: Dict[int, torch.Tensor] = {}
        self._group: Dict[int, int] = {}
        self._cleared: List[torch.Tensor] = []
        paged = [g for g in groups if g.paged]
        for gi, g in enumerate(paged):
            for cid in g.cache_ids:
                self._group[cid] = gi
        for cid, need in needs.items():
            if need is None:
                continue
            if not hasattr(need, "make_storage"):
                raise TypeError(f"cache {cid}: {need!r} does not describe its storage (no make_storage)")
            t = need.make_storage(page_size, num_pages, max_slots, act_dtype, device)
            self._tensors[cid] = t
            self._group.setdefault(cid, -1)
            if getattr(need, "clear_on_admission", False):
                self._cleared.append(t)

    def tensor(self, cache_id: int) -> torch.Tensor:
        return self._tensors[cache_id]

    def group_of(self, cache_id: int) -> int:
        return self._group[cache_id]

    def clear_slot(self, slot: int) -> None:
        """Zeroes the slot's row of every state tensor that asks for it (a request was admitted)."""
        for t in self._cleared:
            t[slot].zero_()

    def copy(self, page_copies, slot_copies, device) -> None:
        """Carries out what CacheManager.reorder returned: pages of every paged cache of a group and the
        slots' rows of every state tensor are copied on the device (pages: sources and destinations are disjoint)."""
        from ..kernels import ops
        for cid, t in self._tensors.items():
            g = self._group[cid]
            if g >= 0:
                if page_copies[g]:
                    ops.copy_rows(t, torch.tensor(page_copies[g], dtype=torch.int32, device=device))
            elif slot_copies:
                # slots stay with their requests, so a slot may be source and destination at once:
                # read all sources first
                src = torch.tensor([s for s, _ in slot_copies], dtype=torch.long, device=device)
                dst = torch.tensor([d for _, d in slot_copies], dtype=torch.long, device=device)
                t[dst] = t[src].clone()

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self._tensors.values())

    @staticmethod
    def bytes_per_page(needs: Dict[int, object], page_size: int, act_dtype) -> int:
        return sum(n.bytes_per_page(page_size, act_dtype) for n in needs.values()
                   if n is not None and hasattr(n, "bytes_per_page"))
