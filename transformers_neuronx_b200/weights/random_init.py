"""Seeded random weights: writes a model folder (config.json, model.safetensors) from a
configuration and a seed.

The reference's generator (src/transformers_neuronx/opt/gen_random_pretrained.py:32-102) draws
init_std * randn for matrices and embeddings and writes zeros for every bias and LayerNorm
tensor, which makes all logits equal; here biases are N(0, init_std), LayerNorm weights
1 + N(0, init_std) and LayerNorm biases N(0, init_std), so that every tensor matters in a test.
One generator stream is consumed in the order in which the model lists its tensors.
"""
from __future__ import annotations

import os
from typing import Dict, Sequence

import torch

from .loader import TensorSpec
from .safetensors_io import save_safetensors


def random_tensors(specs: Sequence[TensorSpec], seed: int, init_std: float,
                   matrix_dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    gen = torch.Generator(device="cpu")
    gen.manual_seed(int(seed))
    out = {}
    for s in specs:
        if s.tied_to is not None:
            continue                      # a tied tensor is not stored
        if s.kind == "int_table":
            out[s.name] = torch.zeros(s.shape, dtype=torch.int32)
            continue
        t = torch.randn(s.shape, generator=gen, dtype=torch.float32) * init_std
        if s.kind == "norm_weight":
            out[s.name] = (1.0 + t)       # LayerNorm tensors stay in 32-bit, as the reference's
        elif s.kind in ("norm_bias",):    # demo keeps them (opt/demo.py:23-29)
            out[s.name] = t
        else:
            out[s.name] = t.to(matrix_dtype)
    return out


def write_model_folder(folder: str, config, specs: Sequence[TensorSpec], seed: int,
                       matrix_dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    os.makedirs(folder, exist_ok=True)
    tensors = random_tensors(specs, seed, config.init_std, matrix_dtype)
    config.save(folder)
    save_safetensors(tensors, os.path.join(folder, "model.safetensors"),
                     metadata={"format": "pt", "seed": seed})
    return tensors
