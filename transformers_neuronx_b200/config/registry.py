"""One registry from an architecture's name (config.json "architectures"[0], or "model_type") to
what builds it: its typed configuration class and the function that turns a configuration into
a model specification.  The reference keeps the same map from Hugging Face names to model classes
(src/transformers_neuronx/modeling_auto.py:5-47)."""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict


@dataclass(frozen=True)
class Architecture:
    name: str                 # e.g. "OPTForCausalLM"
    model_type: str           # e.g. "opt"
    config_class: Any         # has from_dict(dict), from_pretrained(folder), save(folder), init_std
    build_spec: Callable      # config -> ModelSpec


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(arch: Architecture) -> None:
    _ARCHITECTURES[arch.name] = arch


def architectures() -> Dict[str, Architecture]:
    _ensure_builtin()
    return dict(_ARCHITECTURES)


_builtin_loaded = False


def _ensure_builtin() -> None:
    """The architectures that ship with the package register themselves when the `models` package
    is imported (models/__init__.py lists them); anything else calls register_architecture()."""
    global _builtin_loaded
    if not _builtin_loaded:
        _builtin_loaded = True
        import importlib
        importlib.import_module(__name__.rsplit(".", 2)[0] + ".models")


def resolve_architecture(config_dict: Dict[str, Any]) -> Architecture:
    _ensure_builtin()
    names = config_dict.get("architectures") or []
    for n in names:
        if n in _ARCHITECTURES:
            return _ARCHITECTURES[n]
    mt = config_dict.get("model_type")
    for a in _ARCHITECTURES.values():
        if mt is not None and a.model_type == mt:
            return a
    raise KeyError(
        f"no model registered for architectures={names!r} / model_type={mt!r}; "
        f"supported: {sorted(_ARCHITECTURES)}")


def config_from_dict(d: Dict[str, Any]):
    """(architecture, typed config) for the contents of a config.json."""
    arch = resolve_architecture(d)
    return arch, arch.config_class.from_dict(d)


def load_config(folder: str):
    """Reads folder/config.json and returns (architecture, typed config)."""
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"{path} not found: a model folder holds config.json and model.safetensors")
    with open(path) as fp:
        d = json.load(fp)
    arch = resolve_architecture(d)
    return arch, arch.config_class.from_dict(d)
