"""Dense feed-forward: residual += fc2(act(fc1(h))) with biases
(src/transformers_neuronx/hlo.py:504-577); the activation is named by the configuration
(hlo.py:485-501).  The activation and the residual add run in the epilogues of the two products."""
from __future__ import annotations

from ..kernels.ops import activation_code
from .base import FeedForward
from .linear import Linear
from .registry import register_feed_forward
from .spec import DenseFeedForwardSpec


class DenseFeedForward(FeedForward):
    graph_safe = True
    takes_normed_input = True       # `h` only feeds fc1
    libraries = ("gemm_simt", "gemm_tc", "gemv")

    def __init__(self, spec: DenseFeedForwardSpec):
        self.spec = spec
        activation_code(spec.activation)          # raises on a name the epilogues do not know
        self.fc1, self.fc2 = Linear(spec.fc1), Linear(spec.fc2)

    def tensor_specs(self):
        return self.fc1.tensor_specs() + self.fc2.tensor_specs()

    def load(self, tensors, device, act_dtype):
        self.fc1.load(tensors, device, act_dtype)
        self.fc2.load(tensors, device, act_dtype)

    def parameter_bytes(self):
        return self.fc1.parameter_bytes() + self.fc2.parameter_bytes()

    def forward(self, ctx, h, residual):
        a = ctx.scratch(h.shape[0], self.spec.fc1.out_features)
        self.fc1.forward(h, a, activation=self.spec.activation)
        self.fc2.forward(a, residual, residual=residual)


register_feed_forward("dense", DenseFeedForward)
