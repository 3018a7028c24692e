"""Reading and writing the safetensors container with the standard library and torch only.

Layout of a file: 8 bytes little-endian header length N, N bytes of JSON
``{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}``, then the
tensors' bytes.  Tensors are returned as views of a read-only memory map, so a 13 GB checkpoint is
not copied on the host before it goes to the GPU.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from typing import Dict, Iterable, Tuple

import torch

_ST_TO_TORCH = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_TORCH_TO_ST = {v: k for k, v in _ST_TO_TORCH.items()}


class SafetensorsFile:
    """One opened file: ``keys()``, ``info(name) -> (dtype, shape)``, ``tensor(name)``."""

    def __init__(self, path: str):
        self.path = path
        self._fp = open(path, "rb")
        head = self._fp.read(8)
        if len(head) != 8:
            raise ValueError(f"{path}: too short to be a safetensors file")
        (n,) = struct.unpack("<Q", head)
        size = os.path.getsize(path)
        if n <= 0 or 8 + n > size:
            raise ValueError(f"{path}: header length {n} does not fit the file ({size} bytes)")
        self._header = json.loads(self._fp.read(n).decode("utf-8"))
        self.metadata = self._header.pop("__metadata__", {}) or {}
        self._data_start = 8 + n
        self._mm = mmap.mmap(self._fp.fileno(), 0, access=mmap.ACCESS_READ) if size else None
        for name, e in self._header.items():
            if e["dtype"] not in _ST_TO_TORCH:
                raise ValueError(f"{path}: tensor {name!r} has unsupported dtype {e['dtype']}")
            b, en = e["data_offsets"]
            if not (0 <= b <= en <= size - self._data_start):
                raise ValueError(f"{path}: tensor {name!r} lies outside the file")

    def keys(self) -> Iterable[str]:
        return self._header.keys()

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        e = self._header[name]
        return _ST_TO_TORCH[e["dtype"]], tuple(e["shape"])

    def tensor(self, name: str) -> torch.Tensor:
        e = self._header[name]
        dtype = _ST_TO_TORCH[e["dtype"]]
        shape = tuple(e["shape"])
        b, en = e["data_offsets"]
        count = 1
        for s in shape:
            count *= s
        if count == 0:
            return torch.empty(shape, dtype=dtype)
        with warnings.catch_warnings():          # the map is read-only; nothing writes through it
            warnings.simplefilter("ignore", UserWarning)
            if dtype == torch.bool:
                t = torch.frombuffer(self._mm, dtype=torch.uint8, count=count,
                                     offset=self._data_start + b).bool()
            else:
                t = torch.frombuffer(self._mm, dtype=dtype, count=count, offset=self._data_start + b)
        return t.view(shape)

    def close(self):
        # Tensors handed out are views of the map: it is closed when they are gone.
        self._fp.close()


def save_safetensors(tensors: Dict[str, torch.Tensor], path: str, metadata=None) -> None:
    header = {}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _TORCH_TO_ST:
            raise ValueError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _TORCH_TO_ST[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as fp:
        fp.write(struct.pack("<Q", len(blob)))
        fp.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu().reshape(-1)     # flat: a 0-dimensional tensor has bytes too
            if t.numel():
                fp.write(t.view(torch.uint8).numpy().tobytes() if t.dtype != torch.bool
                         else t.to(torch.uint8).numpy().tobytes())
    os.replace(tmp, path)
