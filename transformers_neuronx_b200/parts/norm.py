"""LayerNorm as the reference computes it: statistics and affine in 32-bit over the hidden axis
(src/transformers_neuronx/hlo.py:84-105), with eps, scale and shift as parameters of the part."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import Norm, to_device
from .registry import register_norm
from .spec import NormSpec


class LayerNorm(Norm):
    graph_safe = True
    libraries = ("layernorm",)

    def __init__(self, spec: NormSpec):
        self.spec = spec
        self.weight = None
        self.bias = None

    def tensor_specs(self):
        s, out = self.spec, []
        if s.weight:
            out.append(TensorSpec(s.weight, (s.size,), "norm_weight"))
        if s.bias:
            out.append(TensorSpec(s.bias, (s.size,), "norm_bias"))
        return out

    def load(self, tensors, device, act_dtype):
        s = self.spec
        self.weight = to_device(tensors[s.weight], device, torch.float32) if s.weight else None
        self.bias = to_device(tensors[s.bias], device, torch.float32) if s.bias else None

    def parameter_bytes(self):
        return sum(t.numel() * 4 for t in (self.weight, self.bias) if t is not None)

    def fused_params(self):
        return self.weight, self.bias, self.spec.eps

    def forward(self, ctx, x, out_f32=None, out_act=None, rows=None):
        ops.layer_norm(x, self.weight, self.bias, self.spec.eps, out_f32=out_f32, out_act=out_act, rows=rows)


register_norm("layer_norm", LayerNorm)
