"""Greedy equality of a model of this package with a reference implementation
(src/transformers_neuronx/testing/validation.py:23-101)."""
from __future__ import annotations

import torch

from ..generation_utils import HuggingFaceGenerationModelAdapter


def validate(model, neuron, config, inputs, sequence_length: int, verbose: bool = True) -> None:
    """`model`: the reference, anything with ``generate(input_ids=, attention_mask=, max_new_tokens=, ...)``
    that returns [rows, sequence_length] ids chosen greedily (a Hugging Face model on the CPU, say; nothing
    of that library is imported here).  `neuron`: the model of this package.  `inputs`: (input_ids,
    attention_mask, start_ids) as testing.data makes them.  Both ways of generating with `neuron`, the
    adapter's generate() and sample(), must give the reference's tokens; raises AssertionError naming the
    first difference otherwise."""
    neuron.to_neuron()
    input_ids, attention_mask, start_ids = inputs
    new_tokens = sequence_length - input_ids.shape[1]
    expected = torch.as_tensor(model.generate(input_ids=input_ids, attention_mask=attention_mask,
                                              max_new_tokens=new_tokens, min_new_tokens=new_tokens, top_k=1))
    adapter = HuggingFaceGenerationModelAdapter(config, neuron)
    by_generate = adapter.generate(input_ids, attention_mask=attention_mask, max_new_tokens=new_tokens)
    neuron.reset()
    by_sample = neuron.sample(input_ids, sequence_length=sequence_length, start_ids=start_ids, top_k=1)
    if verbose:
        print("reference:", expected, "generate():", by_generate, "sample():", by_sample, sep="\n")
    for name, got in (("generate()", by_generate), ("sample()", by_sample)):
        if got.shape != expected.shape or not torch.equal(got.to(expected.dtype), expected):
            bad = (got.to(expected.dtype) != expected).nonzero()[0].tolist() if got.shape == expected.shape else None
            raise AssertionError(f"{name} differs from the reference" + (f" first at row {bad[0]}, position {bad[1]}" if bad else
                                                                         f": shapes {tuple(got.shape)} and {tuple(expected.shape)}"))
