"""Weights by tensor name.

A model states the tensors it reads as a list of ``TensorSpec`` (name, shape, kind); this module
reads a folder, matches names, and raises ONE error that lists every missing tensor, every
unexpected tensor and every wrong shape.  The reference resolves the same Hugging Face names
through a skeleton of modules (src/transformers_neuronx/module.py:129-279, opt/model.py:195-270),
retries without the ``model.`` prefix (module.py:161-176) and ties lm_head to embed_tokens when
the file has no lm_head.weight (module.py:142-159).

Dtype policy: a tensor keeps the type it is stored in (bfloat16, float16 or 32-bit; the reference's
three amp types, src/transformers_neuronx/dtypes.py:18-35); integer tables become int32.  What a
part does with a 16-bit tensor of another kind than the engine's is the part's business
(parts/base.py: weight_to_device): the 32-bit path widens it exactly.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .model_files import open_model_files


@dataclass(frozen=True)
class TensorSpec:
    name: str                      # name in the checkpoint
    shape: Tuple[int, ...]
    kind: str = "matrix"           # 'matrix' | 'table' | 'bias' | 'norm_weight' | 'norm_bias' | 'int_table'
    tied_to: Optional[str] = None  # when absent from the file, this other tensor is used
    optional: bool = False         # may be absent without a tie (never used by OPT)


class WeightError(ValueError):
    """Lists everything wrong with a checkpoint at once."""

    def __init__(self, where, missing, unexpected, wrong_shape, other=()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.other = list(other)
        lines = [f"weights in {where} do not fit the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, got, want in self.wrong_shape:
            lines.append(f"  wrong shape: {name} is {list(got)}, the model needs {list(want)}")
        for msg in self.other:
            lines.append("  " + msg)
        super().__init__("\n".join(lines))


def _convert(t: torch.Tensor, name: str, other: List[str]) -> torch.Tensor:
    if t.dtype in (torch.bfloat16, torch.float16, torch.float32, torch.int32):
        return t
    if t.dtype == torch.float64:
        return t.to(torch.float32)
    if t.dtype in (torch.int64, torch.int16, torch.int8, torch.uint8):
        return t.to(torch.int32)
    other.append(f"unsupported dtype: {name} is {t.dtype}")
    return t


def _strip_candidates(name: str) -> Sequence[str]:
    # A checkpoint of the bare decoder lacks the 'model.' prefix.
    if name.startswith("model."):
        return (name, name[len("model."):])
    return (name,)


def match_tensors(specs: Sequence[TensorSpec], available: Dict[str, Tuple[torch.dtype, Tuple[int, ...]]],
                  where: str) -> Dict[str, str]:
    """Returns {spec name -> name in the file} or raises WeightError.  Pure bookkeeping: works
    on (dtype, shape) alone, so tests need no tensor data."""
    missing, wrong, resolved = [], [], {}
    used = set()
    by_name = {s.name: s for s in specs}
    for s in specs:
        found = next((c for c in _strip_candidates(s.name) if c in available), None)
        if found is None:
            if s.tied_to is not None or s.optional:
                continue
            missing.append(s.name)
            continue
        used.add(found)
        resolved[s.name] = found
        got = tuple(available[found][1])
        if got != tuple(s.shape):
            wrong.append((s.name, got, s.shape))
    for s in specs:           # ties are resolved after their targets
        if s.name not in resolved and s.tied_to is not None:
            if s.tied_to in resolved:
                resolved[s.name] = resolved[s.tied_to]
                if tuple(by_name[s.tied_to].shape) != tuple(s.shape):
                    wrong.append((s.name, by_name[s.tied_to].shape, s.shape))
            elif s.tied_to not in missing:
                missing.append(s.name)
    unexpected = sorted(n for n in available if n not in used)
    if missing or unexpected or wrong:
        raise WeightError(where, missing, unexpected, wrong)
    return resolved


def load_tensors(folder: str, specs: Sequence[TensorSpec]) -> Dict[str, torch.Tensor]:
    """{spec name -> CPU tensor} for every spec; raises WeightError on any mismatch."""
    files = open_model_files(folder)
    available, owner = {}, {}
    for f in files:
        for k in f.keys():
            available[k] = f.info(k)
            owner[k] = f
    resolved = match_tensors(specs, available, folder)
    out, other = {}, []
    by_name = {s.name: s for s in specs}
    for name, src in resolved.items():
        if by_name[name].tied_to is not None and resolved.get(by_name[name].tied_to) == src:
            continue                          # filled from its tie below
        out[name] = _convert(owner[src].tensor(src), name, other)
    # A file that stores a tied tensor under both names must store the same values.
    for s in specs:
        if s.tied_to is None:
            continue
        if resolved.get(s.name) != resolved.get(s.tied_to):
            a, b = out[s.name], out[s.tied_to]
            if a.shape == b.shape and not torch.equal(a.float(), b.float()):
                other.append(f"{s.name} differs from {s.tied_to}, to which it is tied")
        out[s.name] = out[s.tied_to]          # one tensor under both names
    if other:
        raise WeightError(folder, [], [], [], other)
    for f in files:
        f.close()
    return out
