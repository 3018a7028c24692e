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

import gc
import warnings
from dataclasses import dataclass, field
from typing import Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..cache import CacheManager, CacheStorage, OutOfPages, group_needs
from ..kernels import ops
from ..parts.base import StepContext


@dataclass
class StepEntry:
    rid: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()          # places among `tokens` whose logits are asked for
    from_device: Optional[int] = None  # the (single) token is row `from_device` of the ids sampled last step


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

    def __init__(self, model, page_size: int, num_pages: int, max_slots: int, max_model_len: int,
                 use_cuda_graphs: bool = False, max_graph_batch: int = 256, max_graphs: int = 128):
        self.model = model
        self.device = model.device
        self.act_dtype = model.act_dtype
        self.page_size = page_size
        self.max_model_len = max_model_len
        needs = model.cache_needs()
        groups = group_needs(needs)
        self.cache = CacheManager(groups, page_size, num_pages, max_slots)
        self.storage = CacheStorage(needs, groups, page_size, num_pages, max_slots, self.act_dtype, self.device)
        self.cache.on_slot_taken = self.storage.clear_slot
        self.n_groups = len(self.cache.paged_groups)
        self.vocab = model.spec.vocab_size
        self._pinned = None
        self.steps_run = 0
        self.last_h2d_bytes = 0
        # decode-only steps can be replayed as CUDA graphs, one per (batch bucket, context bucket)
        self.use_cuda_graphs = bool(use_cuda_graphs) and getattr(model, "graph_safe", True)
        # Parts that do not declare themselves graph_safe keep the whole model out of CUDA graphs: say so
        # once, by name, instead of losing the graphs silently.
        self.graph_blockers = sorted({type(p).__name__ for p in getattr(model, "all_parts", lambda: [])()
                                      if not getattr(p, "graph_safe", False)})
        if use_cuda_graphs and self.graph_blockers:
            warnings.warn("steps of this model are not captured in CUDA graphs: " + ", ".join(self.graph_blockers) +
                          " do(es) not declare graph_safe (parts/base.py)")
        self.max_graph_batch = max_graph_batch
        self.max_graphs = max_graphs              # shapes kept as graphs (each holds its buffers)
        self._graphs = {}
        self._graph_pool = None
        self._decode_layouts = {}
        self._table_arrays = {}
        self._arange_cache = None
        self.extra_dev = None                     # device copy of the last step's `extra` section

    # ---- requests -------------------------------------------------------------------------------
    def add_request(self, rid) -> int:
        return self.cache.add_request(rid)

    def finish(self, rid) -> None:
        self.cache.free_request(rid)
        self.forget(rid)

    def forget(self, rid) -> None:
        """Drops what the runner keeps about a request whose pages were given back."""
        for g in range(self.n_groups):
            self._table_arrays.pop((rid, g), None)

    def reorder(self, rids: Sequence, sources: Sequence[int]) -> None:
        """Request rids[i] goes on from what rids[sources[i]] holds now (beam search).  The requests hold
        equally many tokens; pages change hands where they can and are copied where two requests go on
        from the same one."""
        if all(s == i for i, s in enumerate(sources)):
            return
        page_copies, slot_copies = self.cache.reorder(list(rids), [int(s) for s in sources])
        self.storage.copy(page_copies, slot_copies, self.device)
        for rid in rids:
            self.forget(rid)

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

    def _validate(self, entries: Sequence[StepEntry]) -> None:
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
            if e.from_device is not None and len(e.tokens) != 1:
                raise ValueError(f"request {e.rid!r}: a token taken from the device must be the entry's only token")
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

    EXTRA_WORDS = 16        # words per request of the section a caller may send along (sampling parameters)

    def _pack(self, entries: Sequence[StepEntry], pad=None, fixed_blocks: Optional[int] = None, extra=None):
        """Reserves the pages and builds the step's index arrays.  `extra` (int32 array, at most
        EXTRA_WORDS per request): the caller's own section, copied along as the last one.  pad = (tokens, requests, tiles,
        decode rows, wanted rows): the sizes of a captured step's arrays.  Padded token rows carry
        request -1 and slot -1, padded tiles request -1 and padded decode rows -1, all of which the
        kernels skip; padded wanted rows repeat row 0."""
        hb = HostBatch()
        tokens, positions, token_request, logit_rows, tok_src = [], [], [], [], []
        row = 0
        for r, e in enumerate(entries):
            start = self.cache.append(e.rid, len(e.tokens))
            n = len(e.tokens)
            tok_src.extend([-1] * n if e.from_device is None else [int(e.from_device)])
            hb.rids.append(e.rid); hb.q_start.append(row); hb.q_len.append(n); hb.ctx_len.append(start)
            hb.slots.append(self.cache.slot(e.rid))
            tokens.extend(int(t) for t in e.tokens)
            positions.extend(range(start, start + n))
            token_request.extend([r] * n)
            logit_rows.extend(row + int(w) for w in e.want)
            row += n
        N, R = row, len(entries)
        Np, Rp = (N, R) if pad is None else pad[:2]
        ps = self.page_size

        def padded(vals, size, fill):
            a = np.full(size, fill, dtype=np.int32)
            a[:len(vals)] = vals
            return a

        tok, pos, treq = padded(tokens, Np, 0), padded(positions, Np, 0), padded(token_request, Np, -1)
        tiles, decode_rows = [], []
        for r in range(R):
            if hb.q_len[r] == 1:
                decode_rows.append(hb.q_start[r])
            else:
                for q0 in range(0, hb.q_len[r], ops.ATTN_PREFILL_TILE):
                    last_key = hb.ctx_len[r] + min(hb.q_len[r], q0 + ops.ATTN_PREFILL_TILE)
                    tiles.append((last_key, r, q0))
        # The attention kernels start their work items from the end of the list: tiles with more
        # keys to read come later here, so that the long ones start first and the short ones fill in.
        tiles.sort()
        tile_req, tile_q0 = [t[1] for t in tiles], [t[2] for t in tiles]
        if pad is not None:
            Tp, Dp, Wp = pad[2:]
            tile_req = [-1] * (Tp - len(tile_req)) + tile_req          # padding first: the kernels start from the end
            tile_q0 = [0] * (Tp - len(tile_q0)) + tile_q0
            decode_rows = decode_rows + [-1] * (Dp - len(decode_rows))
            logit_rows = logit_rows + [0] * (Wp - len(logit_rows))
        parts = [tok, pos, treq, padded(hb.q_start, Rp, 0), padded(hb.q_len, Rp, 0), padded(hb.ctx_len, Rp, 0),
                 padded(hb.slots, Rp, 0), np.asarray(logit_rows, np.int32),
                 np.asarray(tile_req, np.int32), np.asarray(tile_q0, np.int32), np.asarray(decode_rows, np.int32),
                 padded(tok_src, Np, -1)]
        n_fixed = len(parts)
        max_blocks = []
        for g in range(self.n_groups):
            tables = [self.cache.block_table(e.rid, g) for e in entries]
            mb = max(len(t) for t in tables) if fixed_blocks is None else fixed_blocks
            bt = np.full((Rp, mb), -1, dtype=np.int32)
            for r, t in enumerate(tables):
                bt[r, :len(t)] = t
            sm = np.full(Np, -1, dtype=np.int32)
            sm[:N] = bt[treq[:N], pos[:N] // ps] * ps + pos[:N] % ps
            parts += [bt.reshape(-1), sm]
            max_blocks.append(mb)
        ex = np.zeros(Rp * self.EXTRA_WORDS, dtype=np.int32)
        if extra is not None:
            ex[:extra.size] = extra.reshape(-1)
        parts.append(ex)
        sizes = [p.size for p in parts]
        offs, o = [], 0                       # each section starts on a 16-byte boundary
        for sz in sizes:
            offs.append(o)
            o += (sz + 3) // 4 * 4
        slot = self._pinned_buffer(o)
        host = slot[0].numpy()
        for p, off in zip(parts, offs):
            host[off:off + p.size] = p
        return hb, slot, o, offs, sizes, max_blocks, n_fixed, (N, R, Np, Rp), (len(tile_req), len(decode_rows))

    def _context(self, dev, hb, offs, sizes, max_blocks, n_fixed, dims, counts) -> StepContext:
        N, R, Np, Rp = dims

        def sec(i):
            return dev[offs[i]:offs[i] + sizes[i]]

        ctx = StepContext(self.device, self.act_dtype)
        ctx.n_tokens, ctx.n_requests = Np, R
        ctx.token_ids, ctx.positions, ctx.token_request = sec(0), sec(1), sec(2)
        ctx.q_start, ctx.q_len, ctx.ctx_len, ctx.state_slots = sec(3), sec(4), sec(5), sec(6)
        ctx.logit_rows = sec(7)
        ctx.tile_req, ctx.tile_q0, ctx.decode_rows = sec(8), sec(9), sec(10)
        ctx.token_source = sec(11)
        ctx.n_prefill_tiles, ctx.n_decode_rows = counts
        for g in range(self.n_groups):
            ctx.block_tables.append(sec(n_fixed + 2 * g).view(Rp, max_blocks[g]))
            ctx.slot_mapping.append(sec(n_fixed + 2 * g + 1))
        ctx.extra = sec(n_fixed + 2 * self.n_groups)
        ctx.host = hb
        ctx.storage = self.storage
        ctx.page_size = self.page_size
        ctx.decode_only = all(n == 1 for n in hb.q_len)
        ctx.max_ctx = max(c + n for c, n in zip(hb.ctx_len, hb.q_len))
        ctx.max_decode_ctx = max([c + 1 for c, n in zip(hb.ctx_len, hb.q_len) if n == 1], default=0)
        return ctx

    def prepare(self, entries: Sequence[StepEntry], sampled: Optional[torch.Tensor] = None, extra=None) -> StepContext:
        """Reserves pages for every entry (all or none), builds the step's index arrays in pinned
        memory and copies them to the device in one transfer.  `sampled`: the ids the sampling kernel
        left on the device, for entries that take their token from there."""
        self._validate(entries)
        hb, slot, o, offs, sizes, max_blocks, n_fixed, dims, counts = self._pack(entries, extra=extra)
        dev = torch.empty(o, dtype=torch.int32, device=self.device)
        dev.copy_(slot[0][:o], non_blocking=True)
        if slot[1] is None:
            slot[1] = torch.cuda.Event()
        slot[1].record()
        self.last_h2d_bytes = o * 4
        ctx = self._context(dev, hb, offs, sizes, max_blocks, n_fixed, dims, counts)
        self._patch_tokens(entries, ctx, sampled)
        return ctx

    def _patch_tokens(self, entries, ctx, sampled) -> None:
        if any(e.from_device is not None for e in entries):
            if sampled is None:
                raise ValueError("an entry takes its token from the device but no sampled ids were given")
            ops.patch_tokens(ctx.token_ids, ctx.token_source, sampled)

    # ---- decode-only steps as CUDA graphs ----------------------------------------------------------
    def _graph_key(self, entries):
        R = len(entries)
        bucket = 1
        while bucket < R:
            bucket *= 2
        longest = max(self.cache.length(e.rid) for e in entries) + 1
        ctx_bucket = 256
        while ctx_bucket < longest:
            ctx_bucket *= 2
        return bucket, min(ctx_bucket, -(-self.max_model_len // self.page_size) * self.page_size)

    def _pack_decode(self, entries, bucket: int, fixed_blocks: int, extra=None):
        """_pack for a step in which every request has one token, with little host work: the same
        sections at the same offsets, filled with array operations; block tables are kept as arrays
        per request and only their new entries are copied."""
        R, ps, G = len(entries), self.page_size, self.n_groups
        hb = HostBatch()
        cache = self.cache
        toks, starts = [], []
        for e in entries:
            starts.append(cache.append(e.rid, 1))
            toks.append(int(e.tokens[0]))
            hb.rids.append(e.rid)
            hb.slots.append(cache.slot(e.rid))
        hb.q_start = list(range(R)); hb.q_len = [1] * R; hb.ctx_len = starts
        lay = self._decode_layouts.get((bucket, fixed_blocks))
        if lay is None:
            sizes = [bucket] * 8 + [0, 0, bucket, bucket]
            for _ in range(G):
                sizes += [bucket * fixed_blocks, bucket]
            sizes.append(bucket * self.EXTRA_WORDS)
            offs, o = [], 0
            for sz in sizes:
                offs.append(o)
                o += (sz + 3) // 4 * 4
            lay = (sizes, offs, o)
            self._decode_layouts[(bucket, fixed_blocks)] = lay
        sizes, offs, o = lay
        slot = self._pinned_buffer(o)
        host = slot[0].numpy()
        pos = np.asarray(starts, dtype=np.int32)

        def sec(i):
            return host[offs[i]:offs[i] + sizes[i]]

        ar = self._arange(bucket)
        for i, vals, fill in ((0, toks, 0), (1, pos, 0), (2, ar[:R], -1), (3, ar[:R], 0), (4, 1, 0), (5, pos, 0), (6, hb.slots, 0)):
            a = sec(i)
            a[:R] = vals
            a[R:] = fill
        sec(7)[:] = ar
        sec(10)[:] = ar
        src = sec(11)
        src[:R] = [-1 if e.from_device is None else int(e.from_device) for e in entries]
        src[R:] = -1
        n_fixed = 12
        for g in range(G):
            bt = sec(n_fixed + 2 * g).reshape(bucket, fixed_blocks)
            for r, e in enumerate(entries):
                bt[r] = self._table_array(e.rid, g, fixed_blocks)
            bt[R:] = -1
            sm = sec(n_fixed + 2 * g + 1)
            sm[:R] = bt[ar[:R], pos // ps] * ps + pos % ps
            sm[R:] = -1
        if extra is not None:
            sec(n_fixed + 2 * G)[:extra.size] = extra.reshape(-1)
        return hb, slot, o, offs, sizes, [fixed_blocks] * G, n_fixed, (R, R, bucket, bucket), (0, bucket)

    def _arange(self, n: int):
        if self._arange_cache is None or self._arange_cache.size < n:
            self._arange_cache = np.arange(max(n, 256), dtype=np.int32)
        return self._arange_cache[:n]

    def _table_array(self, rid, g: int, width: int):
        """The request's block table of group g as an int32 array of `width` entries (-1 beyond its
        blocks), brought up to date from the cache manager's list."""
        table = self.cache.block_table(rid, g)
        key = (rid, g)
        ent = self._table_arrays.get(key)
        if ent is None or ent[0].size != width or ent[2] is not table:
            arr = np.full(width, -1, dtype=np.int32)
            ent = [arr, 0, table]
            self._table_arrays[key] = ent
        arr, filled = ent[0], ent[1]
        n = len(table)
        if n > filled:
            arr[filled:n] = table[filled:n]
            ent[1] = n
        if self.cache.paged_groups[g].window is not None:       # released blocks turn to -1
            first = next((i for i, p in enumerate(table) if p >= 0), n)
            arr[:first] = -1
        return arr

    def _graph_step(self, entries, sampled=None, extra=None) -> torch.Tensor:
        key = self._graph_key(entries)
        bucket, ctx_bucket = key
        fixed_blocks = -(-ctx_bucket // self.page_size)
        packed = self._pack_decode(entries, bucket, fixed_blocks, extra)
        return self._wanted_rows(self._run_captured(key, packed, entries, sampled, ctx_bucket), entries)

    # ---- small steps with prompt portions as CUDA graphs --------------------------------------------
    SMALL_STEP_TOKENS = 128        # a step of at most this many tokens ...
    SMALL_STEP_REQUESTS = 8        # ... of at most this many requests is launch-bound: it is captured

    def _small_step_key(self, entries):
        """The graph a step with prompt portions runs as, or None when it is large enough for the
        kernels to hide the host's work: (tokens, requests, tiles, decode rows, wanted rows) padded
        to a few sizes, and the context bucket."""
        N = sum(len(e.tokens) for e in entries)
        R = len(entries)
        if N > self.SMALL_STEP_TOKENS or R > self.SMALL_STEP_REQUESTS or N == R:
            return None
        Np = 16
        while Np < N:
            Np *= 2
        Rp = self.SMALL_STEP_REQUESTS
        W = sum(len(e.want) for e in entries)
        if W > max(Np, Rp):
            return None
        Wp = 0 if W == 0 else (Rp if W <= Rp else Np)
        Dp = Rp if any(len(e.tokens) == 1 for e in entries) else 0
        tiles = sum(-(-len(e.tokens) // ops.ATTN_PREFILL_TILE) for e in entries if len(e.tokens) > 1)
        if tiles > Rp:
            return None
        longest = max(self.cache.length(e.rid) + len(e.tokens) for e in entries)
        ctx_bucket = 256
        while ctx_bucket < longest:
            ctx_bucket *= 2
        ctx_bucket = min(ctx_bucket, -(-self.max_model_len // self.page_size) * self.page_size)
        return ("portions", Np, Rp, Rp, Dp, Wp), ctx_bucket

    def _small_graph_step(self, key, entries, sampled=None, extra=None) -> torch.Tensor:
        pad, ctx_bucket = key
        packed = self._pack(entries, pad=pad[1:], fixed_blocks=-(-ctx_bucket // self.page_size), extra=extra)
        logits = self._run_captured(key, packed, entries, sampled, ctx_bucket)
        return logits[:sum(len(e.want) for e in entries)]

    def _run_captured(self, key, packed, entries, sampled, ctx_bucket) -> torch.Tensor:
        """Runs the packed step through the graph of `key`: the first step of a key runs eagerly
        (kernels get built, scratch gets made), the second is captured, and from then on the graph
        is replayed on the index arrays copied into its fixed device buffer.  Returns the logits of
        all (padded) wanted rows."""
        hb, slot, o, offs, sizes, max_blocks, n_fixed, dims, counts = packed
        g = self._graphs.get(key)
        if g is None:
            dev = torch.empty(o, dtype=torch.int32, device=self.device)
            ctx = self._context(dev, hb, offs, sizes, max_blocks, n_fixed, dims, counts)
            g = {"dev": dev, "ctx": ctx, "graph": None, "logits": None, "runs": 0}
            if len(self._graphs) < self.max_graphs:
                self._graphs[key] = g                 # beyond the limit a new shape runs eagerly every time
        dev, ctx = g["dev"], g["ctx"]
        dev.copy_(slot[0][:o], non_blocking=True)
        if slot[1] is None:
            slot[1] = torch.cuda.Event()
        slot[1].record()
        self.last_h2d_bytes = o * 4
        ctx.host, ctx.n_requests = hb, len(entries)
        self.extra_dev = ctx.extra
        self._patch_tokens(entries, ctx, sampled)
        ctx.max_decode_ctx = ctx_bucket               # the split plan is fixed for the whole bucket
        ctx.max_ctx = ctx_bucket
        if g["graph"] is None:
            if g["runs"] == 0:
                g["runs"] = 1
                with ops.stream_scope():
                    return self.model.forward(ctx)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            n0 = ops.launch_count()
            # Garbage that owns device memory (an older runner's graphs and their pool) must not be
            # collected while the stream is capturing: freeing device memory invalidates the capture.
            gc.collect()
            gc_was_on = gc.isenabled()
            gc.disable()
            try:
                with torch.cuda.graph(graph, pool=self._graph_pool):
                    with ops.stream_scope():
                        g["logits"] = self.model.forward(ctx)
            finally:
                if gc_was_on:
                    gc.enable()
            g["kernels"] = ops.launch_count() - n0       # recorded, not run
            ops.add_launches(-g["kernels"])
            g["graph"] = graph
            if self._graph_pool is None:
                self._graph_pool = graph.pool()
            # the capture recorded the kernels without running them: fall through to the replay
        g["graph"].replay()
        ops.add_launches(g["kernels"])
        g["runs"] += 1
        return g["logits"]

    def captured_steps(self) -> dict:
        """{graph key: steps run through it} of the graphs that have been captured."""
        return {k: g["runs"] for k, g in self._graphs.items() if g["graph"] is not None}

    def _wanted_rows(self, logits: torch.Tensor, entries) -> torch.Tensor:
        """A captured decode step computes the logits of every row; hand out those that were asked for."""
        wanted = [r for r, e in enumerate(entries) if len(e.want)]
        if len(wanted) == len(entries):
            return logits[:len(entries)]
        if not wanted:
            return logits[:0]
        return logits[torch.tensor(wanted, dtype=torch.long, device=logits.device)]

    @torch.no_grad()
    def step(self, entries: Sequence[StepEntry], sampled: Optional[torch.Tensor] = None, extra=None) -> torch.Tensor:
        """Runs one step; returns the 32-bit logits [wanted, vocab] (a device tensor) in the order
        of the entries and of their `want`; the tensor is the caller's until the next step (a captured
        step writes its logits into the same buffer at every replay).  `sampled` (int32, device): ids sampled in the step
        before, for entries with `from_device`.  `extra` (int32 numpy array of at most EXTRA_WORDS
        words per entry): travels to the device in the step's one copy; `self.extra_dev` is its
        device copy afterwards (the engine sends the sampling parameters this way)."""
        graphs = self.use_cuda_graphs and getattr(self.model, "graph_safe", True)      # not while results are tapped
        if graphs and all(len(e.tokens) == 1 for e in entries) and len(entries) <= self.max_graph_batch:
            self._validate(entries)
            logits = self._graph_step(entries, sampled, extra)
        elif graphs and (key := self._small_step_key(entries)) is not None:
            self._validate(entries)
            logits = self._small_graph_step(key, entries, sampled, extra)
        else:
            ctx = self.prepare(entries, sampled, extra)
            self.extra_dev = ctx.extra
            with ops.stream_scope():
                logits = self.model.forward(ctx)
        for e in entries:
            self.cache.release_behind_window(e.rid)
        self.steps_run += 1
        return logits
