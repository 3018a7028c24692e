"""Left-padded batches for tests (src/transformers_neuronx/testing/data.py:18-77): each returns
(input_ids [rows, length], attention_mask [rows, length], start_ids [rows]) where a row attends from
its start position on; padded places hold token 0."""
from __future__ import annotations

import torch


def _seeded(seed):
    return None if seed is None else torch.Generator().manual_seed(int(seed))


def batch_varying_lengths(vocab_size: int, batch_size: int, context_length: int, seed=None):
    """Rows whose left padding has random lengths (every row keeps at least its last token)."""
    g = _seeded(seed)
    starts = torch.randint(0, context_length, (batch_size,), generator=g)
    mask = (torch.arange(context_length)[None, :] >= starts[:, None]).int()
    inputs = torch.randint(0, vocab_size, (batch_size, context_length), generator=g) * mask
    return inputs, mask, starts.int()


def batch_all_lengths(vocab_size: int, context_length: int, seed=None):
    """One row for every possible length: row i attends from position i on."""
    g = _seeded(seed)
    starts = torch.arange(context_length)
    mask = (torch.arange(context_length)[None, :] >= starts[:, None]).int()
    inputs = torch.randint(0, vocab_size, (context_length, context_length), generator=g) * mask
    return inputs, mask, starts.int()


def batch_full_lengths(vocab_size: int, batch_size: int, context_length: int, seed=None):
    """Rows without padding: a check that batching alone changes nothing."""
    g = _seeded(seed)
    inputs = torch.randint(0, vocab_size, (batch_size, context_length), generator=g)
    return inputs, torch.ones(batch_size, context_length, dtype=torch.int32), torch.zeros(batch_size, dtype=torch.int32)
