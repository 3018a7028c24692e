"""Run-time settings of the engine (not properties of a model).

The reference spreads the corresponding knobs over NeuronConfig and
ContinuousBatchingConfig (src/transformers_neuronx/config.py:73-103, :148-470); only what a
one-GPU paged engine needs is kept.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

_DTYPES = {
    "f32": "float32", "fp32": "float32", "float32": "float32",
    "bf16": "bfloat16", "bfloat16": "bfloat16",
    "f16": "float16", "fp16": "float16", "float16": "float16", "half": "float16",
}


def canonical_dtype(name) -> str:
    """'f32' | 'f16' | 'bf16' (the reference's amp names, dtypes.py:18-35) or torch names -> torch name."""
    key = str(name).replace("torch.", "")
    if key not in _DTYPES:
        raise ValueError(f"unknown dtype {name!r}; expected one of f32, f16, bf16")
    return _DTYPES[key]


@dataclass
class EngineConfig:
    dtype: str = "bfloat16"            # 'bfloat16' | 'float16' (serving kernels) or 'float32' (true 32-bit path)
    page_size: int = 16                # tokens per cache page
    num_pages: Optional[int] = None    # pages per cache group; None: from max_tokens
    max_tokens: Optional[int] = None   # most tokens live requests hold at any time
    max_num_seqs: int = 64             # slots for per-request state
    max_batch_tokens: int = 2048       # token budget of one step
    max_portion: Optional[int] = None  # longest portion of one prompt in a step; None: what the budget allows
    max_model_len: Optional[int] = None  # longest request; None: the model's own limit
    use_cuda_graphs: bool = True       # capture decode-only steps and steps of a few prompt tokens
    async_scheduling: bool = True      # launch a step before the ids of the step before it are read back
    seed: int = 0

    def __post_init__(self):
        self.dtype = canonical_dtype(self.dtype)
        if self.page_size <= 0 or self.page_size % 16:
            raise ValueError(f"page_size must be a positive multiple of 16, got {self.page_size}")
        if self.max_portion is not None and self.max_portion < 1:
            raise ValueError(f"max_portion must be at least 1, got {self.max_portion}")
