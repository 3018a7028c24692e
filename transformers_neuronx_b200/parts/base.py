"""Interfaces of the parts a decoder is put together from, and what a part sees of a step.

Hidden state travels between parts as two tensors of shape [tokens, hidden]: the 32-bit residual
stream, and (where a part reads its input un-normalised) a copy in the activation type.

    Norm.forward(ctx, x, out_f32=None, out_act=None, rows=None)
    Mixer.forward(ctx, h, residual)          residual += mix(h), using and updating its cache
    FeedForward.forward(ctx, h, residual)    residual += ff(h)
    PositionEncoding.table_for_embedding()   a (table, offset) added where tokens are embedded, or None
    PositionEncoding.embed(ctx, x)           any other change of the hidden state at that place
    PositionEncoding.rotate(ctx, q, k)       a change of queries and keys inside a mixer
    Block.forward(ctx, x, x_act)             one layer: its norms, mixer and feed-forward in its order

Every part lists the tensors it reads (``tensor_specs``), takes them in ``load`` and names the
kernel libraries it needs (``libraries``), so that a model compiles only what it uses.  A mixer
says what it keeps between steps with ``cache_need`` (cache/manager.py): paged keys and values,
state of fixed size per request, or nothing.  No part knows which model it is in.
"""
from __future__ import annotations

from typing import Dict, List, Sequence

import torch

from ..weights.loader import TensorSpec


class StepContext:
    """The running step, as parts see it.  All index tensors are int32 on the device."""

    def __init__(self, device, act_dtype):
        self.device = device
        self.act_dtype = act_dtype            # torch.bfloat16 or torch.float32
        self.n_tokens = 0
        self.n_requests = 0
        self.token_ids = None                 # [N]
        self.positions = None                 # [N] position of each token in its request
        self.token_request = None             # [N] index of the token's request in this batch
        self.token_source = None              # [N] row of last step's sampled ids that is this token, or -1
        self.q_start = None                   # [R] first row of each request
        self.q_len = None                     # [R] rows of each request
        self.ctx_len = None                   # [R] tokens the request had in the cache before this step
        self.logit_rows = None                # [W] rows whose logits are wanted
        self.state_slots = None               # [R] slot of each request (state of fixed size)
        self.block_tables: List[torch.Tensor] = []   # per paged group: [R, blocks]
        self.slot_mapping: List[torch.Tensor] = []   # per paged group: [N] page * page_size + row
        self.extra = None                     # the caller's own section of the step's buffer (engine/step.py)
        self.host = None                      # the same numbers as Python lists (engine/step.py: HostBatch)
        self.storage = None                   # cache/storage.py: CacheStorage
        self.cache_id = -1                    # set by the model before each mixer runs
        self.page_size = 0
        self.decode_only = False              # every request has exactly one row
        self.max_ctx = 0                      # longest context (after this step) in the batch
        self.tile_req = None                  # [tiles] request of each tile of query rows of a portion
        self.tile_q0 = None                   # [tiles] its first row within the portion
        self.decode_rows = None               # rows of requests that have exactly one row
        self.n_prefill_tiles = 0
        self.n_decode_rows = 0
        self.max_decode_ctx = 0
        self._scratch_pool = {}
        self._scratch_used = {}

    def empty(self, rows, cols, dtype=None) -> torch.Tensor:
        return torch.empty((rows, cols), dtype=dtype or self.act_dtype, device=self.device)

    def scratch(self, rows, cols, dtype=None) -> torch.Tensor:
        """A buffer that is dead when the running schedule entry ends: the next entry's requests of
        the same shape get the same memory again (an allocation per buffer and layer is what a step
        of a few tokens spends its time on).  Distinct calls within one entry get distinct buffers."""
        key = (rows, cols, dtype or self.act_dtype)
        i = self._scratch_used.get(key, 0)
        self._scratch_used[key] = i + 1
        have = self._scratch_pool.setdefault(key, [])
        if i == len(have):
            have.append(torch.empty((rows, cols), dtype=key[2], device=self.device))
        return have[i]

    def begin_entry(self) -> None:
        """Called before each schedule entry runs: the scratch buffers of the entry before are free."""
        self._scratch_used = {}

    # what the mixer of the running schedule entry owns
    def cache(self) -> torch.Tensor:
        return self.storage.tensor(self.cache_id)

    def cache_group(self) -> int:
        return self.storage.group_of(self.cache_id)


class Part:
    libraries: Sequence[str] = ()
    graph_safe = False       # True: forward launches kernels only (no host reads, no host loops over ctx.host)

    def tensor_specs(self) -> List[TensorSpec]:
        return []

    def load(self, tensors: Dict[str, torch.Tensor], device, act_dtype) -> None:
        pass

    def parameter_bytes(self) -> int:
        return 0


class Norm(Part):
    def forward(self, ctx, x, out_f32=None, out_act=None, rows=None):
        raise NotImplementedError

    def fused_params(self):
        """(gamma, beta, eps) when this norm is a LayerNorm that a following product may apply itself
        (NormedInput below), else None."""
        return None


class NormedInput:
    """A part's input that has not been normalized yet: rows of the 32-bit residual stream and the norm
    to apply.  A consumer whose first kernel can apply the norm itself does so (Linear, for one token:
    the LayerNorm kernel, its launch and its output's trip through memory are saved); anyone else
    calls tensor(), which runs the norm's own kernel once.  A block hands one out only to parts that
    say ``takes_normed_input`` (parts/block.py)."""

    def __init__(self, ctx, x, norm):
        self.ctx, self.x, self.norm = ctx, x, norm
        self._tensor = None

    @property
    def shape(self):
        return self.x.shape

    def tensor(self):
        if self._tensor is None:
            self._tensor = self.ctx.scratch(self.x.shape[0], self.x.shape[1])
            self.norm.forward(self.ctx, self.x, out_act=self._tensor)
        return self._tensor


class Mixer(Part):
    takes_normed_input = False      # True: forward's `h` may be a NormedInput (the part hands it to a Linear)

    def cache_need(self):
        return None

    def forward(self, ctx, h, residual):
        raise NotImplementedError


class FeedForward(Part):
    takes_normed_input = False

    def forward(self, ctx, h, residual):
        raise NotImplementedError


class PositionEncoding(Part):
    def table_for_embedding(self):
        return None

    def embed(self, ctx, x):
        return None

    def rotate(self, ctx, q, k):
        return None


def to_device(t: torch.Tensor, device, dtype=None) -> torch.Tensor:
    """Host tensor (possibly a view of a memory-mapped file) -> device, optionally converted."""
    if dtype is not None and t.dtype != dtype:
        t = t.to(dtype)
    return t.contiguous().to(device, non_blocking=False)


_H16 = (torch.bfloat16, torch.float16)
_rounded = {"count": 0, "example": None}


def weight_to_device(t: torch.Tensor, device, act_dtype, name: str = "") -> torch.Tensor:
    """A matrix or table goes to the device in the type it is stored in: a 32-bit tensor stays
    32-bit (it runs on the 32-bit kernels whatever the engine's type), and the 32-bit engine reads
    a 16-bit tensor of either kind as it is (its kernels widen each element exactly).  Only a
    16-bit engine that meets the other 16-bit type rounds: once, on the device, and
    rounding_report() says how many tensors lost bits that way."""
    d = t.contiguous().to(device, non_blocking=False)
    if d.dtype in _H16 and act_dtype in _H16 and d.dtype != act_dtype:
        _rounded["count"] += 1
        _rounded["example"] = _rounded["example"] or f"{name or 'a tensor'} ({d.dtype} -> {act_dtype})"
        d = d.to(act_dtype)
    return d


def rounding_report(reset: bool = True):
    """(number of tensors rounded from one 16-bit type to the other since the last report, one example)."""
    out = (_rounded["count"], _rounded["example"])
    if reset:
        _rounded["count"], _rounded["example"] = 0, None
    return out
