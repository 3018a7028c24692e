"""Device memory of the caches: for a paged cache one tensor
[pages, 2 (key, value), n_kv_heads, page_size, head_dim] in the activation type, for state of fixed
size one tensor [slots, *shape].  What a request may read is decided by its own length and block
table, never by the contents of a page; pages are not cleared when they change hands.  The memory
is zeroed once, when it is made: the tensor-core attention multiplies rows that no token has
written yet by probabilities that are exactly zero, so they must hold finite numbers."""
from __future__ import annotations

from typing import Dict, List

import torch

from .manager import FixedStateNeed, GroupInfo, PagedKVNeed

_DT = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}


class CacheStorage:
    def __init__(self, needs: Dict[int, object], groups: List[GroupInfo], page_size: int, num_pages: int,
                 max_slots: int, act_dtype, device):
        self.page_size, self.num_pages, self.max_slots = page_size, num_pages, max_slots
        self._tensors: Dict[int, torch.Tensor] = {}
        self._group: Dict[int, int] = {}
        paged = [g for g in groups if g.paged]
        for gi, g in enumerate(paged):
            for cid in g.cache_ids:
                self._group[cid] = gi
        for cid, need in needs.items():
            if isinstance(need, PagedKVNeed):
                self._tensors[cid] = torch.zeros((num_pages, 2, need.n_kv_heads, page_size, need.head_dim),
                                                 dtype=act_dtype, device=device)
            elif isinstance(need, FixedStateNeed):
                self._tensors[cid] = torch.zeros((max_slots,) + tuple(need.shape), dtype=_DT[need.dtype],
                                                 device=device)
                self._group[cid] = -1
            elif need is not None:
                raise TypeError(f"cache {cid}: unknown kind of need {need!r}")

    def tensor(self, cache_id: int) -> torch.Tensor:
        return self._tensors[cache_id]

    def group_of(self, cache_id: int) -> int:
        return self._group[cache_id]

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self._tensors.values())

    @staticmethod
    def bytes_per_page(needs: Dict[int, object], page_size: int, act_dtype) -> int:
        el = torch.empty((), dtype=act_dtype).element_size()
        return sum(2 * n.n_kv_heads * page_size * n.head_dim * el for n in needs.values()
                   if isinstance(n, PagedKVNeed))
