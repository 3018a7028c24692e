"""The two ends of the decoder: token embedding (with the optional projection to the hidden width
and the position encoding that is added there), and the head (final norm, optional projection
back, output matrix tied to the embedding table) on the rows whose logits are wanted.

Reference: host embedding src/transformers_neuronx/opt/model.py:162-166; head
src/transformers_neuronx/layers/transformer.py:148-213 (slice the wanted column, LayerNorm,
product with lm_head, no bias; logits leave in 32-bit, base.py:641-647).
"""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import Part, to_device, weight_to_device
from .linear import Linear, linear_forward
from .registry import build_part
from .spec import EmbeddingSpec, HeadSpec


class Embedding(Part):
    graph_safe = True
    def __init__(self, spec: EmbeddingSpec):
        self.spec = spec
        self.table = None
        self.project_in = Linear(spec.project_in) if spec.project_in else None
        self.position = build_part("position", spec.position) if spec.position else None

    @property
    def libraries(self):
        libs = ["embedding"]
        if self.project_in is not None:
            libs += list(self.project_in.libraries)
        if self.position is not None:
            libs += list(self.position.libraries)
        return tuple(libs)

    def tensor_specs(self):
        out = [TensorSpec(self.spec.table, (self.spec.vocab, self.spec.dim), "table")]
        for p in (self.project_in, self.position):
            if p is not None:
                out += p.tensor_specs()
        return out

    def load(self, tensors, device, act_dtype):
        self.table = weight_to_device(tensors[self.spec.table], device, act_dtype, self.spec.table)
        for p in (self.project_in, self.position):
            if p is not None:
                p.load(tensors, device, act_dtype)

    def parameter_bytes(self):
        n = self.table.numel() * self.table.element_size()
        for p in (self.project_in, self.position):
            if p is not None:
                n += p.parameter_bytes()
        return n

    def forward(self, ctx, x, x_act):
        """Fills x (32-bit) and, when given, x_act."""
        table_pos = self.position.table_for_embedding() if self.position is not None else None
        pos_table, offset = table_pos if table_pos is not None else (None, 0)
        if self.project_in is None:
            tok, pre = self.table, None
            if pos_table is not None and pos_table.dtype != tok.dtype:
                pos_table = pos_table.to(tok.dtype)
        else:
            e = ctx.empty(ctx.n_tokens, self.spec.dim)
            ops.gather_rows(self.table, ctx.token_ids, e)
            pre = ctx.empty(ctx.n_tokens, x.shape[1], torch.float32)
            self.project_in.forward(e, pre)
            tok = None
        ops.embed(tok, pre, ctx.token_ids, pos_table, ctx.positions, offset, x, x_act)
        if self.position is not None and table_pos is None:
            self.position.embed(ctx, x)
            if x_act is not None:
                ops.pick_rows(x, None, out_act=x_act)


class Head(Part):
    graph_safe = True
    def __init__(self, spec: HeadSpec):
        self.spec = spec
        self.weight = None
        self.final_norm = build_part("norm", spec.final_norm) if spec.final_norm else None
        self.project_out = Linear(spec.project_out) if spec.project_out else None

    @property
    def libraries(self):
        libs = ["layernorm", "gemm_simt", "gemm_tc", "gemv"]
        return tuple(libs)

    def tensor_specs(self):
        s = self.spec
        out = [TensorSpec(s.weight, (s.vocab, s.dim), "matrix", tied_to=s.tied_to)]
        for p in (self.final_norm, self.project_out):
            if p is not None:
                out += p.tensor_specs()
        return out

    def load(self, tensors, device, act_dtype, shared=None):
        """`shared`: {tensor name: device tensor} of tensors another part already holds (the tied table)."""
        s = self.spec
        src = tensors[s.weight]
        if shared is not None and s.tied_to in shared and src is tensors.get(s.tied_to):
            self.weight = shared[s.tied_to]
        else:
            self.weight = weight_to_device(src, device, act_dtype, s.weight)
        for p in (self.final_norm, self.project_out):
            if p is not None:
                p.load(tensors, device, act_dtype)

    def parameter_bytes(self):
        n = self.weight.numel() * self.weight.element_size()
        for p in (self.final_norm, self.project_out):
            if p is not None:
                n += p.parameter_bytes()
        return n

    def forward(self, ctx, x, rows) -> torch.Tensor:
        """32-bit logits [len(rows), vocab] of the picked rows of the residual stream."""
        R = rows.shape[0]
        y = ctx.empty(R, x.shape[1])
        if self.final_norm is not None:
            self.final_norm.forward(ctx, x, out_act=y, rows=rows)
        else:
            ops.pick_rows(x, rows, out_act=y)
        if self.project_out is not None:
            z = ctx.empty(R, self.spec.dim)
            self.project_out.forward(y, z)
            y = z
        logits = torch.empty((R, self.spec.vocab), dtype=torch.float32, device=ctx.device)
        linear_forward(y, self.weight, None, logits)
        return logits
