"""`generate()` with the argument names that users of Hugging Face models know, on top of this
package's model.

The reference wraps its model in a `transformers.PreTrainedModel` subclass so that the library's
own `generate` drives it (src/transformers_neuronx/generation_utils.py:15-104): the adapter turns
`attention_mask` into `start_ids` (the first attended position of each left-padded row, :70-72),
keeps the current length between calls and forwards to `model(input_ids, cache_ids, start_ids)`.
Here the same class name offers `generate` itself, for the options that map onto the engine's
sampling (greedy, sampling with temperature / top-k / top-p, eos and pad handling, `max_length` /
`max_new_tokens`, a streamer); nothing of the transformers package is imported.  Beam search and
logits processors have no counterpart in the engine and are refused by name.
"""
from __future__ import annotations

from typing import Optional, Sequence, Union

import torch

from .engine import SamplingParams


class HuggingFaceGenerationModelAdapter:
    def __init__(self, config, model):
        self.config = config
        self.model = model
        self.cur_len = 0

    def reset_generation(self) -> None:
        self.cur_len = 0
        self.model.reset()

    # ---- one forward call, as the library's loop would make it ------------------------------------
    def forward(self, input_ids, cache_ids=None, start_ids=None, attention_mask=None, return_dict=False, **unused):
        """Logits [batch, 1, vocab] of each row's last token.  cache_ids None: the rows are whole
        (left-padded) prompts; otherwise input_ids holds the next token of every row."""
        if start_ids is None and attention_mask is not None:
            start_ids = self.start_ids_of(attention_mask)
        logits = self.model(torch.as_tensor(input_ids), cache_ids, start_ids)
        logits = (logits[:, -1] if logits.dim() == 3 else logits)[:, None, :]      # all positions asked for: the last
        if cache_ids is None:
            self.cur_len = int(torch.as_tensor(input_ids).shape[1])
        else:
            self.cur_len += 1
        return {"logits": logits, "past_key_values": tuple()} if return_dict else (logits,)

    __call__ = forward

    @staticmethod
    def start_ids_of(attention_mask) -> torch.Tensor:
        """The first attended position of each row: the length of its left padding."""
        return torch.as_tensor(attention_mask).long().argmax(dim=1).int()

    # ---- generate ---------------------------------------------------------------------------------
    def generate(self, input_ids, attention_mask=None, max_length: Optional[int] = None,
                 max_new_tokens: Optional[int] = None, do_sample: bool = False, top_k: Optional[int] = 50,
                 top_p: float = 1.0, temperature: float = 1.0, eos_token_id: Union[None, int, Sequence[int]] = None,
                 pad_token_id: Optional[int] = None, streamer=None, seed: int = 0, num_beams: int = 1, **others):
        """[batch, prompt] ids (left-padded where attention_mask is 0) -> [batch, prompt + new] ids.
        A row that produced an eos id is finished; from there on it holds pad_token_id (the eos id
        when none is given), and the result ends where the last row finished."""
        if num_beams != 1:
            raise NotImplementedError("beam search is not built: the engine samples or takes the most likely token")
        if others:
            raise TypeError(f"generate() got option(s) without a counterpart in this engine: {sorted(others)}")
        self.reset_generation()
        m = self.model
        m._ready()
        input_ids = torch.as_tensor(input_ids)
        B, T0 = input_ids.shape
        if B > m.batch_size:
            raise ValueError(f"batch of {B} rows; the model was made for batch_size={m.batch_size}")
        if max_new_tokens is None:
            max_length = m.n_positions if max_length is None else int(max_length)
            max_new_tokens = max_length - T0
        if max_new_tokens <= 0:
            return input_ids
        if T0 + max_new_tokens > m.n_positions:
            raise ValueError(f"{T0} prompt tokens and {max_new_tokens} new ones exceed n_positions {m.n_positions}")
        starts = [0] * B if attention_mask is None else self.start_ids_of(attention_mask).tolist()
        rows = input_ids.tolist()
        prompts = [rows[b][starts[b]:] for b in range(B)]
        if do_sample:
            params = [SamplingParams(temperature=float(temperature), top_k=int(top_k or 0), top_p=float(top_p),
                                     seed=int(seed) + b) for b in range(B)]
        else:
            params = [SamplingParams(temperature=0.0) for _ in range(B)]
        eos = None
        if eos_token_id is not None:
            eos = (int(eos_token_id),) if isinstance(eos_token_id, int) else tuple(int(e) for e in eos_token_id)
        outs = m._generate(prompts, max_new_tokens, params, streamer, input_ids.dtype, eos=eos, pad=pad_token_id)
        self.cur_len = T0 + len(outs[0])
        return torch.cat([input_ids, torch.as_tensor(outs, dtype=input_ids.dtype)], dim=1)
