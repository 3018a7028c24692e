"""y = x W^T (+ b), with the epilogues the decoder needs (ReLU; adding into the 32-bit residual
stream), and the activation that the configuration names.  W keeps the checkpoint's [out, in]
orientation and its stored type (parts/base.py: weight_to_device): a matrix stored in 32-bit stays
32-bit (it then runs on the 32-bit kernel).  The bias is applied in 32-bit.

Kernel choice: 16-bit activations with a matrix of the same 16-bit type go to the tcgen05 tensor-core
kernel when its size rules hold (the row length in bytes a multiple of 16, for its TMA descriptors);
everything else goes to the CUDA-core kernel with 32-bit FMA accumulation.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import NormedInput, Part, to_device, weight_to_device
from .spec import LinearSpec




class Linear(Part):
    graph_safe = True
    def __init__(self, spec: LinearSpec):
        self.spec = spec
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    @property
    def libraries(self):
        return ("gemm_simt", "gemm_tc", "gemv")

    def tensor_specs(self) -> List[TensorSpec]:
        s = self.spec
        out = [TensorSpec(s.weight, (s.out_features, s.in_features), "matrix")]
        if s.bias:
            out.append(TensorSpec(s.bias, (s.out_features,), "bias"))
        return out

    def load(self, tensors: Dict[str, torch.Tensor], device, act_dtype) -> None:
        self.set_weight(weight_to_device(tensors[self.spec.weight], device, act_dtype, self.spec.weight),
                        to_device(tensors[self.spec.bias], device, torch.float32) if self.spec.bias else None)

    def set_weight(self, weight: torch.Tensor, bias: Optional[torch.Tensor]) -> None:
        self.weight, self.bias = weight, bias

    def parameter_bytes(self) -> int:
        n = self.weight.numel() * self.weight.element_size()
        if self.bias is not None:
            n += self.bias.numel() * 4
        return n

    def forward(self, a, out: torch.Tensor, residual: Optional[torch.Tensor] = None,
                activation: Optional[str] = None) -> torch.Tensor:
        """`a`: the activations, or a NormedInput (rows of the residual stream and the norm still to apply)."""
        if isinstance(a, NormedInput):
            fused = a.norm.fused_params()
            if (fused is not None and a.ctx.act_dtype == self.weight.dtype
                    and ops.gemv_layer_norm_supported(a.x, self.weight, out)):
                ops.gemv_layer_norm(a.x, fused[0], fused[1], fused[2], self.weight, out, bias=self.bias,
                                    residual=residual, activation=activation)
                return out
            a = a.tensor()
        linear_forward(a, self.weight, self.bias, out, residual, activation)
        return out


def linear_forward(a, weight, bias, out, residual=None, activation=None):
    if ops.gemm_tc_supported(a, weight, out):
        ops.gemm_tc(a, weight, out, bias=bias, residual=residual, activation=activation)
    else:
        ops.gemm_simt(a, weight, out, bias=bias, residual=residual, activation=activation)


def fuse_linears(parts: List[Linear], device) -> Linear:
    """One Linear whose output is the concatenation of the given ones' (same input): q, k and v
    become a single matrix product."""
    ws = [p.weight for p in parts]
    dtype = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
    weight = torch.cat([w.to(dtype) for w in ws], dim=0).contiguous()
    has_bias = [p.bias is not None for p in parts]
    bias = None
    if any(has_bias):
        bias = torch.cat([p.bias if p.bias is not None else
                          torch.zeros(p.weight.shape[0], dtype=torch.float32, device=device) for p in parts])
    spec = LinearSpec(parts[0].spec.in_features, sum(p.spec.out_features for p in parts), "<fused>",
                      "<fused>" if bias is not None else None)
    fused = Linear(spec)
    fused.set_weight(weight, bias)
    return fused
