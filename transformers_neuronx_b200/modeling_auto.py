"""The entry-point class of a model folder, chosen by its config.json.

The reference maps `model_type` to one of its sampling classes
(src/transformers_neuronx/modeling_auto.py:5-47).  Here the table holds OPT; another architecture
registers its own entry-point class beside its registration in config/registry.py.
"""
from __future__ import annotations

import os
from typing import Dict

from .config import load_config
from .opt.model import OPTForSampling

NEURON_MODEL_FOR_CAUSAL_LM_MAPPING: Dict[str, type] = {"opt": OPTForSampling}


def register_model_class(model_type: str, cls: type) -> None:
    """The entry-point class (with from_pretrained) for folders whose config.json names `model_type`."""
    NEURON_MODEL_FOR_CAUSAL_LM_MAPPING[model_type] = cls


class NeuronAutoModelForCausalLM:
    @classmethod
    def from_pretrained(cls, pretrained_model_name_or_path, *model_args, **kwargs):
        if not os.path.isdir(pretrained_model_name_or_path):
            raise FileNotFoundError(f"{pretrained_model_name_or_path!r} is not a folder; there is no network here to "
                                    "fetch a model by name")
        arch, _ = load_config(pretrained_model_name_or_path)          # raises for an architecture nobody registered
        if arch.model_type not in NEURON_MODEL_FOR_CAUSAL_LM_MAPPING:
            raise AssertionError(f"The configuration model type '{arch.model_type}' has no entry-point class here "
                                 f"(known: {sorted(NEURON_MODEL_FOR_CAUSAL_LM_MAPPING)})")
        return NEURON_MODEL_FOR_CAUSAL_LM_MAPPING[arch.model_type].from_pretrained(pretrained_model_name_or_path,
                                                                                   *model_args, **kwargs)
