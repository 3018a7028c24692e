"""Multi-head attention over the paged cache.

As the reference computes it (src/transformers_neuronx/opt/model.py:388-524): q, k, v projections
with bias, q scaled by `scale` (1/sqrt(head_dim) for OPT, :458-459), scores against every earlier
key and the token's own, softmax in 32-bit, context, output projection with bias; the residual add
is fused into the output projection here.  Heads, key/value heads, head size, scale and window are
parameters.  The keys and values of this step's tokens are written into the cache's pages first (by
the append kernel, or in a step of decode tokens only by the decode attention kernel itself); the
attention kernels then read keys and values from the pages alone, whatever the cut of the batch.
"""
from __future__ import annotations

from ..cache.manager import PagedKVNeed
from ..kernels import ops
from .base import Mixer
from .linear import Linear, fuse_linears
from .registry import build_part, register_mixer
from .spec import AttentionSpec


class PagedAttention(Mixer):
    graph_safe = True
    takes_normed_input = True       # `h` only feeds the q/k/v product
    def __init__(self, spec: AttentionSpec):
        s = self.spec = spec
        if s.n_heads % s.n_kv_heads:
            raise ValueError(f"{s.n_heads} heads cannot share {s.n_kv_heads} key/value heads")
        if s.head_dim % 16 or not (16 <= s.head_dim <= 256):
            raise ValueError(f"head size {s.head_dim} is not supported: the attention kernels take "
                             "multiples of 16 from 16 to 256")
        self.q, self.k, self.v, self.out = Linear(s.q), Linear(s.k), Linear(s.v), Linear(s.out)
        self.qkv = None
        self.position = build_part("position", s.position) if s.position is not None else None

    @property
    def libraries(self):
        libs = ["gemm_simt", "gemm_tc", "gemv", "kv_cache", "attention_simt", "attention_prefill", "attention_prefill_tc", "attention_decode"]
        if self.position is not None:
            libs += list(self.position.libraries)
        return tuple(libs)

    def tensor_specs(self):
        out = []
        for p in (self.q, self.k, self.v, self.out, self.position):
            if p is not None:
                out += p.tensor_specs()
        return out

    def load(self, tensors, device, act_dtype):
        for p in (self.q, self.k, self.v, self.out):
            p.load(tensors, device, act_dtype)
        self.qkv = fuse_linears([self.q, self.k, self.v], device)
        for p in (self.q, self.k, self.v):          # the fused copy is the one that is used
            p.weight = p.bias = None
        if self.position is not None:
            self.position.load(tensors, device, act_dtype)

    def parameter_bytes(self):
        return self.qkv.parameter_bytes() + self.out.parameter_bytes()

    def cache_need(self):
        s = self.spec
        return PagedKVNeed(s.n_kv_heads, s.head_dim, s.window)

    def forward(self, ctx, h, residual):
        s = self.spec
        N = h.shape[0]
        qd, kd = s.n_heads * s.head_dim, s.n_kv_heads * s.head_dim
        qkv = ctx.scratch(N, qd + 2 * kd)
        self.qkv.forward(h, qkv)
        q, k, v = qkv[:, :qd], qkv[:, qd:qd + kd], qkv[:, qd + kd:]
        if self.position is not None:
            self.position.rotate(ctx, q, k)
        cache, g = ctx.cache(), ctx.cache_group()
        att = ctx.scratch(N, qd)
        ops.attention(ctx, g, q, cache, att, s.n_heads, s.scale, s.window or 0, new_kv=(k, v, ctx.slot_mapping[g]))
        self.out.forward(att, residual, residual=residual)


register_mixer("attention", PagedAttention)
