"""Descriptions of a model as data: which parts, with which sizes and constants, in which order.

An architecture (models/opt.py) turns its typed configuration into a ``ModelSpec``.  Every part
is named by a ``kind`` that the registries of parts/registry.py resolve to a class, so a model may
use different mixers and feed-forwards in different layers, and a test may register a kind of its
own.  The order in which layers run is the ``schedule``: a list of (layer, cache) pairs that may
name a layer twice, or give two entries the same cache so that one layer reads what another wrote.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional, Tuple


@dataclass(frozen=True)
class LinearSpec:
    in_features: int
    out_features: int
    weight: str                      # tensor name, [out_features, in_features]
    bias: Optional[str] = None       # tensor name, [out_features]; None: no bias


@dataclass(frozen=True)
class NormSpec:
    kind: str                        # 'layer_norm'
    size: int
    eps: float
    weight: Optional[str] = None     # None: no elementwise scale
    bias: Optional[str] = None


@dataclass(frozen=True)
class PositionSpec:
    kind: str                        # 'learned' | 'none' | a registered kind
    table: Optional[str] = None      # tensor name, [rows, dim]
    rows: int = 0
    dim: int = 0
    offset: int = 0                  # row = position + offset
    extra: Tuple = ()


@dataclass(frozen=True)
class AttentionSpec:
    kind: str                        # 'attention'
    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    scale: float
    q: LinearSpec = None
    k: LinearSpec = None
    v: LinearSpec = None
    out: LinearSpec = None
    window: Optional[int] = None     # None: every earlier position is read
    position: Optional[PositionSpec] = None   # an encoding applied to queries and keys, if any


@dataclass(frozen=True)
class DenseFeedForwardSpec:
    kind: str                        # 'dense'
    fc1: LinearSpec = None
    fc2: LinearSpec = None
    activation: str = "relu"


@dataclass(frozen=True)
class LayerSpec:
    block: str                       # 'pre_norm' | 'post_norm' | a registered kind
    norm1: Any = None
    mixer: Any = None
    norm2: Any = None
    feed_forward: Any = None


@dataclass(frozen=True)
class EmbeddingSpec:
    table: str                       # tensor name, [vocab, dim]
    vocab: int = 0
    dim: int = 0
    project_in: Optional[LinearSpec] = None
    position: Optional[PositionSpec] = None   # an encoding added to the hidden state, if any


@dataclass(frozen=True)
class HeadSpec:
    weight: str                      # tensor name of the output matrix [vocab, dim]
    vocab: int = 0
    dim: int = 0
    tied_to: Optional[str] = None    # used when the file does not store `weight`
    final_norm: Optional[NormSpec] = None
    project_out: Optional[LinearSpec] = None


@dataclass(frozen=True)
class ScheduleEntry:
    layer: int                       # index into ModelSpec.layers
    cache: int                       # which cache its mixer uses; entries may share one


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: EmbeddingSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    head: HeadSpec
    eos_token_id: Optional[int] = None
    pad_token_id: Optional[int] = None
    bos_token_id: Optional[int] = None
