"""Registries from a part's ``kind`` to the class that builds it.

A norm, mixer, feed-forward or position encoding is constructed as ``cls(spec)``; a block as
``cls(norm1, mixer, norm2, feed_forward)``; each has the interface of its family in base.py.
Registering a new kind needs no change to any file of the package: a test (or a user) calls
``register_mixer("my_kind", MyMixer)`` and names "my_kind" in a spec.
"""
from __future__ import annotations

from typing import Callable, Dict

_REG: Dict[str, Dict[str, Callable]] = {
    "mixer": {}, "feed_forward": {}, "norm": {}, "position": {}, "block": {},
}


def _register(family: str, kind: str, cls) -> None:
    _REG[family][kind] = cls


def register_mixer(kind, cls): _register("mixer", kind, cls)
def register_feed_forward(kind, cls): _register("feed_forward", kind, cls)
def register_norm(kind, cls): _register("norm", kind, cls)
def register_position(kind, cls): _register("position", kind, cls)
def register_block(kind, cls): _register("block", kind, cls)


def _lookup(family: str, kind: str):
    table = _REG[family]
    if kind not in table:
        raise KeyError(f"no {family} of kind {kind!r} is registered; known: {sorted(table)}")
    return table[kind]


def build_part(family: str, spec):
    """family in 'mixer', 'feed_forward', 'norm', 'position'; spec has a ``kind``."""
    if spec is None:
        return None
    return _lookup(family, spec.kind)(spec)


def build_block(kind: str, norm1, mixer, norm2, feed_forward):
    return _lookup("block", kind)(norm1, mixer, norm2, feed_forward)
