"""The files of a model folder, whatever layout it was saved in.

The reference reads five layouts and tries them in this order (src/transformers_neuronx/module.py:
434-460): ``model.safetensors``; the shards of ``model.safetensors.index.json``; a DIRECTORY
``pytorch_model.bin/`` holding one torch-saved tensor per file with ``key_to_filename.json``
(written by its own ``save_pretrained_split``, module.py:30-50, which is what its ``opt_demo
save`` produces); a single ``pytorch_model.bin`` state dict; and the shards of
``pytorch_model.bin.index.json``.  Every opened file offers ``keys()``, ``info(name) -> (dtype,
shape)``, ``tensor(name)`` and ``close()``; the loader sees no difference between them.

The torch-saved layouts are unpickled with ``weights_only=True``: a file that holds anything but
tensors is refused by torch itself.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Iterable, Tuple

import torch

from .safetensors_io import SafetensorsFile


class SplitTensorFolder:
    """``pytorch_model.bin/`` as a directory: key_to_filename.json names one file per tensor."""

    def __init__(self, path: str):
        self.path = path
        with open(os.path.join(path, "key_to_filename.json")) as fp:
            self._files: Dict[str, str] = json.load(fp)
        self._cache: Dict[str, torch.Tensor] = {}

    def keys(self) -> Iterable[str]:
        return self._files.keys()

    def tensor(self, name: str) -> torch.Tensor:
        t = self._cache.get(name)
        if t is None:
            t = torch.load(os.path.join(self.path, self._files[name]), map_location="cpu", weights_only=True)
            if not isinstance(t, torch.Tensor):
                raise ValueError(f"{self.path}: {self._files[name]} does not hold a tensor")
            self._cache[name] = t = t.detach()
        return t

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        t = self.tensor(name)           # the shape is inside the pickle: the piece has to be read
        return t.dtype, tuple(t.shape)

    def close(self):
        self._cache.clear()


class StateDictFile:
    """A torch-saved state dict (``pytorch_model.bin`` or one shard of it)."""

    def __init__(self, path: str):
        self.path = path
        try:
            sd = torch.load(path, map_location="cpu", weights_only=True, mmap=True)
        except (RuntimeError, ValueError):           # an old (non-zip) file cannot be mapped
            sd = torch.load(path, map_location="cpu", weights_only=True)
        if not isinstance(sd, dict) or not all(isinstance(v, torch.Tensor) for v in sd.values()):
            raise ValueError(f"{path}: not a state dict of tensors")
        self._sd = sd

    def keys(self) -> Iterable[str]:
        return self._sd.keys()

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        t = self._sd[name]
        return t.dtype, tuple(t.shape)

    def tensor(self, name: str) -> torch.Tensor:
        return self._sd[name].detach()

    def close(self):
        self._sd = {}


def open_model_files(folder: str):
    """The opened weight file(s) of a model folder, in the reference's order of preference."""
    j = lambda name: os.path.join(folder, name)
    if os.path.isfile(j("model.safetensors")):
        return [SafetensorsFile(j("model.safetensors"))]
    if os.path.isfile(j("model.safetensors.index.json")):
        with open(j("model.safetensors.index.json")) as fp:
            names = sorted(set(json.load(fp)["weight_map"].values()))
        return [SafetensorsFile(j(n)) for n in names]
    if os.path.isdir(j("pytorch_model.bin")):
        return [SplitTensorFolder(j("pytorch_model.bin"))]
    if os.path.isfile(j("pytorch_model.bin")):
        return [StateDictFile(j("pytorch_model.bin"))]
    if os.path.isfile(j("pytorch_model.bin.index.json")):
        with open(j("pytorch_model.bin.index.json")) as fp:
            names = sorted(set(json.load(fp)["weight_map"].values()))
        return [StateDictFile(j(n)) for n in names]
    raise FileNotFoundError(f"no model.safetensors, pytorch_model.bin or index of either in {folder!r}")
