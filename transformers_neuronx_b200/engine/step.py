"""The step function: a batch of (request, its next tokens) -> logits at the wanted places.

A step may hold any mix of portions of prompts and single decoded tokens, cut anywhere.  It runs
only the tokens it is given, as one batch, against the cache that earlier steps left, and appends
their keys and values to it.  The reference's OPT runs either one padded block of prompts or one
token per row, never both (src/transformers_neuronx/base.py:700-710); its chunked-prefill input
shaping for other models (base.py:384-441) is the nearest counterpart.

Host work per step: reserve pages, build the index arrays in one pinned buffer, copy it to the
device once, run the model.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..cache import CacheManager, CacheStorage, OutOfPages, group_needs
from ..parts.base import StepContext


@dataclass
class StepEntry:
    rid: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()          # places among `tokens` whose logits are asked for


@dataclass
class HostBatch:
    """The numbers of a step as Python lists, for parts that plan work on the host."""
    rids: List[Hashable] = field(default_factory=list)
    q_start: List[int] = field(default_factory=list)
    q_len: List[int] = field(default_factory=list)
    ctx_len: List[int] = field(default_factory=list)
    slots: List[int] = field(default_factory=list)


class StepRunner:
    """Owns the cache (bookkeeping and device memory) of one model and runs steps on it."""

    def __init__(self, model, page_size: int, num_pages: int, max_slots: int, max_model_len: int):
        self.model = model
        self.device = model.device
        self.act_dtype = model.act_dtype
        self.page_size = page_size
        self.max_model_len = max_model_len
        needs = model.cache_needs()
        groups = group_needs(needs)
        self.cache = CacheManager(groups, page_size, num_pages, max_slots)
        self.storage = CacheStorage(needs, groups, page_size, num_pages, max_slots, self.act_dtype, self.device)
        self.n_groups = len(self.cache.paged_groups)
        self.vocab = model.spec.vocab_size
        self._pinned = None
        self.steps_run = 0

    # ---- requests -------------------------------------------------------------------------------
    def add_request(self, rid) -> int:
        return self.cache.add_request(rid)

    def finish(self, rid) -> None:
        self.cache.free_request(rid)

    def pages_needed(self, entries: Sequence[StepEntry]) -> List[int]:
        tot = [0] * self.n_groups
        for e in entries:
            for g, n in enumerate(self.cache.pages_needed(e.rid, len(e.tokens))):
                tot[g] += n
        return tot

    # ---- one step -------------------------------------------------------------------------------
    def _pinned_buffer(self, n: int):
        """A pinned staging buffer that no copy in flight still reads: a ring of four, each with
        the event of its last copy."""
        if self._pinned is None:
            self._pinned = [[None, None] for _ in range(4)]
            self._pin_next = 0
        slot = self._pinned[self._pin_next]
        self._pin_next = (self._pin_next + 1) % len(self._pinned)
        if slot[1] is not None:
            slot[1].synchronize()
        if slot[0] is None or slot[0].numel() < n:
            slot[0] = torch.empty(max(n, 4096), dtype=torch.int32, pin_memory=True)
        return slot

    def prepare(self, entries: Sequence[StepEntry]) -> StepContext:
        """Reserves pages for every entry (all or none) and builds the step's index arrays."""
        if not entries:
            raise ValueError("a step needs at least one entry")
        seen = set()
        for e in entries:
            if e.rid in seen:
                raise ValueError(f"request {e.rid!r} appears twice in one step")
            seen.add(e.rid)
            if e.rid not in self.cache:
                raise KeyError(f"request {e.rid!r} is not live")
            if len(e.tokens) == 0:
                raise ValueError(f"request {e.rid!r}: a step entry needs at least one token")
            if self.cache.length(e.rid) + len(e.tokens) > self.max_model_len:
                raise ValueError(f"request {e.rid!r} would hold {self.cache.length(e.rid) + len(e.tokens)} "
                                 f"tokens; the limit is {self.max_model_len}")
            for w in e.want:
                if not (0 <= w < len(e.tokens)):
                    raise ValueError(f"request {e.rid!r}: wanted place {w} is not among its {len(e.tokens)} tokens")
            lo, hi = min(e.tokens), max(e.tokens)
            if lo < 0 or hi >= self.vocab:
                raise ValueError(f"request {e.rid!r}: token id out of range [0, {self.vocab}): {lo}..{hi}")
        need = self.pages_needed(entries)
        free = self.cache.free_pages()
        for g in range(self.n_groups):
            if need[g] > free[g]:
                raise OutOfPages(f"the step needs {need[g]} page(s) in cache group {g}, {free[g]} are free")

        hb = HostBatch()
        tokens, positions, token_request, logit_rows = [], [], [], []
        row = 0
        for r, e in enumerate(entries):
            start = self.cache.append(e.rid, len(e.tokens))
            n = len(e.tokens)
            hb.rids.append(e.rid); hb.q_start.append(row); hb.q_len.append(n); hb.ctx_len.append(start)
            hb.slots.append(self.cache.slot(e.rid))
            tokens.extend(int(t) for t in e.tokens)
            positions.extend(range(start, start + n))
            token_request.extend([r] * n)
            logit_rows.extend(row + int(w) for w in e.want)
            row += n
        N, R = row, len(entries)
        tok = np.asarray(tokens, dtype=np.int64)
        ps = self.page_size
        pos = np.asarray(positions, dtype=np.int32)
        treq = np.asarray(token_request, dtype=np.int32)
        parts = [tok.astype(np.int32), pos, treq,
                 np.asarray(hb.q_start, np.int32), np.asarray(hb.q_len, np.int32), np.asarray(hb.ctx_len, np.int32),
                 np.asarray(hb.slots, np.int32), np.asarray(logit_rows, np.int32)]
        # work lists of the attention kernels: 64-row tiles of portions, and rows that decode
        tile_req, tile_q0, decode_rows = [], [], []
        for r in range(R):
            if hb.q_len[r] == 1:
                decode_rows.append(hb.q_start[r])
            else:
                for q0 in range(0, hb.q_len[r], 64):
                    tile_req.append(r); tile_q0.append(q0)
        parts += [np.asarray(tile_req, np.int32), np.asarray(tile_q0, np.int32), np.asarray(decode_rows, np.int32)]
        n_fixed = len(parts)
        max_blocks = []
        for g in range(self.n_groups):
            tables = [self.cache.block_table(e.rid, g) for e in entries]
            mb = max(len(t) for t in tables)
            bt = np.full((R, mb), -1, dtype=np.int32)
            for r, t in enumerate(tables):
                bt[r, :len(t)] = t
            sm = bt[treq, pos // ps] * ps + pos % ps
            parts += [bt.reshape(-1), sm.astype(np.int32)]
            max_blocks.append(mb)
        sizes = [p.size for p in parts]
        # each section starts on a 16-byte boundary
        offs, o = [], 0
        for s in sizes:
            offs.append(o)
            o += (s + 3) // 4 * 4
        slot = self._pinned_buffer(o)
        pinned = slot[0]
        host = pinned.numpy()
        for p, off in zip(parts, offs):
            host[off:off + p.size] = p
        dev = torch.empty(o, dtype=torch.int32, device=self.device)
        dev.copy_(pinned[:o], non_blocking=True)
        if slot[1] is None:
            slot[1] = torch.cuda.Event()
        slot[1].record()

        def sec(i):
            return dev[offs[i]:offs[i] + sizes[i]]

        ctx = StepContext(self.device, self.act_dtype)
        ctx.n_tokens, ctx.n_requests = N, R
        ctx.token_ids, ctx.positions, ctx.token_request = sec(0), sec(1), sec(2)
        ctx.q_start, ctx.q_len, ctx.ctx_len, ctx.state_slots = sec(3), sec(4), sec(5), sec(6)
        ctx.logit_rows = sec(7)
        ctx.tile_req, ctx.tile_q0, ctx.decode_rows = sec(8), sec(9), sec(10)
        ctx.n_prefill_tiles, ctx.n_decode_rows = len(tile_req), len(decode_rows)
        ctx.max_decode_ctx = max([hb.ctx_len[r] + 1 for r in range(R) if hb.q_len[r] == 1], default=0)
        for g in range(self.n_groups):
            ctx.block_tables.append(sec(n_fixed + 2 * g).view(R, max_blocks[g]))
            ctx.slot_mapping.append(sec(n_fixed + 2 * g + 1))
        ctx.host = hb
        ctx.storage = self.storage
        ctx.page_size = ps
        ctx.decode_only = all(n == 1 for n in hb.q_len)
        ctx.max_ctx = max(c + n for c, n in zip(hb.ctx_len, hb.q_len))
        ctx.h2d_bytes = o * 4
        self.last_h2d_bytes = o * 4
        return ctx

    @torch.no_grad()
    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Runs one step; returns the 32-bit logits [wanted, vocab] (a device tensor) in the order
        of the entries and of their `want`."""
        ctx = self.prepare(entries)
        logits = self.model.forward(ctx)
        for e in entries:
            self.cache.release_behind_window(e.rid)
        self.steps_run += 1
        return logits
