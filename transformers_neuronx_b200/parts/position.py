"""Position encodings.  'learned': a table row per position, added where tokens are embedded, with
the row offset as a parameter (OPT's table starts at row 2:
src/transformers_neuronx/opt/model.py:232-244).  'none': nothing."""
from __future__ import annotations

from ..weights.loader import TensorSpec
from .base import PositionEncoding, weight_to_device
from .registry import register_position
from .spec import PositionSpec


class LearnedPositions(PositionEncoding):
    graph_safe = True
    libraries = ("embedding",)

    def __init__(self, spec: PositionSpec):
        self.spec = spec
        self.table = None

    def tensor_specs(self):
        return [TensorSpec(self.spec.table, (self.spec.rows, self.spec.dim), "table")]

    def load(self, tensors, device, act_dtype):
        self.table = weight_to_device(tensors[self.spec.table], device, act_dtype, self.spec.table)

    def parameter_bytes(self):
        return self.table.numel() * self.table.element_size()

    def max_position(self) -> int:
        return self.spec.rows - self.spec.offset

    def table_for_embedding(self):
        return self.table, self.spec.offset


class NoPositions(PositionEncoding):
    graph_safe = True
    def __init__(self, spec=None):
        self.spec = spec


register_position("learned", LearnedPositions)
register_position("none", NoPositions)
