"""Typed configuration of the OPT decoder, read from the keys of its own config.json.

The reference copies the same keys from the Hugging Face config object
(src/transformers_neuronx/opt/config.py:20-40) and defines no defaults of its own; the
defaults below are those of its literal OPT-175B configuration
(src/transformers_neuronx/opt/gen_random_pretrained.py:105-140).  No model size stands
anywhere else in the package: every part receives its sizes from an instance of this class
through the architecture's specification (models/opt.py).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, fields, asdict
from typing import Any, Dict, Optional, Tuple


class ConfigError(ValueError):
    """A config.json that cannot describe a model this engine can run."""


_REQUIRED = ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
             "ffn_dim", "max_position_embeddings")


@dataclass(frozen=True)
class OPTConfig:
    # sizes: required in config.json
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    ffn_dim: int
    max_position_embeddings: int
    # optional keys
    word_embed_proj_dim: Optional[int] = None      # defaults to hidden_size
    do_layer_norm_before: bool = True
    enable_bias: bool = True
    layer_norm_elementwise_affine: bool = True
    _remove_final_layer_norm: bool = False
    activation_function: str = "relu"
    layer_norm_eps: float = 1e-5                    # the reference fixes 1e-5 in code (hlo.py:51)
    init_std: float = 0.02
    bos_token_id: int = 2
    eos_token_id: int = 2
    pad_token_id: int = 1
    torch_dtype: str = "float16"
    model_type: str = "opt"
    architectures: Tuple[str, ...] = ("OPTForCausalLM",)
    tie_word_embeddings: bool = True

    def __post_init__(self):
        if self.word_embed_proj_dim is None:
            object.__setattr__(self, "word_embed_proj_dim", self.hidden_size)
        for name in _REQUIRED + ("word_embed_proj_dim",):
            v = getattr(self, name)
            if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
                raise ConfigError(f"config key {name!r} must be a positive integer, got {v!r}")
        if self.hidden_size % self.num_attention_heads:
            raise ConfigError(
                f"hidden_size {self.hidden_size} is not a multiple of num_attention_heads "
                f"{self.num_attention_heads}")
        if not (self.layer_norm_eps > 0):
            raise ConfigError(f"layer_norm_eps must be positive, got {self.layer_norm_eps!r}")
        if not self.tie_word_embeddings:
            raise ConfigError("tie_word_embeddings=false is not supported: OPT's lm_head is tied "
                              "to embed_tokens")

    # derived sizes -----------------------------------------------------------------------
    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    @property
    def has_final_layer_norm(self) -> bool:
        return self.do_layer_norm_before and not self._remove_final_layer_norm

    @property
    def has_projection(self) -> bool:
        return self.word_embed_proj_dim != self.hidden_size

    # reading and writing -----------------------------------------------------------------
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "OPTConfig":
        missing = [k for k in _REQUIRED if k not in d]
        if missing:
            raise ConfigError("config.json lacks required key(s): " + ", ".join(missing))
        known = {f.name for f in fields(cls)}
        kw = {k: v for k, v in d.items() if k in known}          # unknown keys are ignored
        if "architectures" in kw:
            kw["architectures"] = tuple(kw["architectures"] or ())
        if kw.get("torch_dtype") is None:
            kw.pop("torch_dtype", None)
        if "dtype" in d and "torch_dtype" not in kw and isinstance(d["dtype"], str):
            kw["torch_dtype"] = d["dtype"]
        return cls(**kw)

    @classmethod
    def from_json(cls, path: str) -> "OPTConfig":
        with open(path) as fp:
            return cls.from_dict(json.load(fp))

    @classmethod
    def from_pretrained(cls, folder: str) -> "OPTConfig":
        return cls.from_json(os.path.join(folder, "config.json"))

    def to_dict(self) -> Dict[str, Any]:
        d = asdict(self)
        d["architectures"] = list(self.architectures)
        return d

    def save(self, folder: str) -> None:
        os.makedirs(folder, exist_ok=True)
        with open(os.path.join(folder, "config.json"), "w") as fp:
            json.dump(self.to_dict(), fp, indent=2)
