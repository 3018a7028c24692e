"""Helpers for checking a model of this package against another implementation
(src/transformers_neuronx/testing/): left-padded batches and a greedy comparison."""
from .data import batch_all_lengths, batch_full_lengths, batch_varying_lengths
from .validation import validate
