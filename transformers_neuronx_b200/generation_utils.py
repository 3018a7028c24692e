"""`generate()` with the argument names that users of Hugging Face models know, on top of this
package's model.

The reference wraps its model in a `transformers.PreTrainedModel` subclass so that the library's
own `generate` drives it (src/transformers_neuronx/generation_utils.py:15-104): the adapter turns
`attention_mask` into `start_ids` (the first attended position of each left-padded row, :70-72),
keeps the current length between calls and forwards to `model(input_ids, cache_ids, start_ids)`.
Here the same class name offers `generate` itself, for the options that map onto the engine's
sampling (greedy, sampling with temperature / top-k / top-p, eos and pad handling, `max_length` /
`max_new_tokens`, a streamer) and a beam search of its own over the model's `forward` and
`reorder_cache` (the reference gets the library's through `_reorder_cache`, :54-58); nothing of the
transformers package is imported.  Logits processors have no counterpart in the engine and are
refused by name.
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
                 pad_token_id: Optional[int] = None, streamer=None, seed: int = 0, num_beams: int = 1,
                 length_penalty: float = 1.0, early_stopping: bool = False, **others):
        """[batch, prompt] ids (left-padded where attention_mask is 0) -> [batch, prompt + new] ids.
        A row that produced an eos id is finished; from there on it holds pad_token_id (the eos id
        when none is given), and the result ends where the last row finished."""
        if others:
            raise TypeError(f"generate() got option(s) without a counterpart in this engine: {sorted(others)}")
        if num_beams != 1:
            if do_sample or streamer is not None:
                raise NotImplementedError("beam search here is the plain one: no sampling within beams, no streamer")
            return self._beam_search(torch.as_tensor(input_ids), attention_mask, int(num_beams), max_length, max_new_tokens,
                                     eos_token_id, pad_token_id, float(length_penalty), bool(early_stopping))
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

    def _reorder_cache(self, past, beam_idx):
        """The hook the library's beam search calls (generation_utils.py:54-58)."""
        self.model.reorder_cache(beam_idx)

    # ---- beam search ------------------------------------------------------------------------------
    def _beam_search(self, input_ids, attention_mask, num_beams, max_length, max_new_tokens, eos_token_id, pad_token_id,
                     length_penalty, early_stopping):
        """Every prompt keeps the `num_beams` most likely continuations so far (sum of the tokens'
        log-probabilities).  A continuation that ends with an eos id is finished and scored by its sum
        divided by (its number of new tokens) ** length_penalty; a prompt is done when it has num_beams
        finished continuations and (early_stopping, or) no running beam can still beat the worst of
        them at its present length.  Returns each prompt's best continuation, padded with pad_token_id
        (the eos id when none is given) to the longest."""
        m = self.model
        m._ready()
        B, T0 = input_ids.shape
        nb = num_beams
        if nb < 1 or B * nb > m.batch_size:
            raise ValueError(f"{B} prompts x {nb} beams need batch_size >= {B * nb}; the model was made for {m.batch_size}")
        if max_new_tokens is None:
            max_new_tokens = (m.n_positions if max_length is None else int(max_length)) - T0
        if max_new_tokens <= 0:
            return input_ids
        if T0 + max_new_tokens > m.n_positions:
            raise ValueError(f"{T0} prompt tokens and {max_new_tokens} new ones exceed n_positions {m.n_positions}")
        eos = set()
        if eos_token_id is not None:
            eos = {int(eos_token_id)} if isinstance(eos_token_id, int) else {int(e) for e in eos_token_id}
        fill = int(pad_token_id) if pad_token_id is not None else (min(eos) if eos else 0)
        starts = torch.zeros(B, dtype=torch.int32) if attention_mask is None else self.start_ids_of(attention_mask)
        self.reset_generation()
        rows = input_ids.repeat_interleave(nb, dim=0)                    # the beams of a prompt are neighbours
        row_starts = starts.repeat_interleave(nb)
        last = lambda t: t[:, -1] if t.dim() == 3 else t                 # (a model asked for all positions' logits)
        logits = last(m(rows, None, row_starts))                         # [B * nb, vocab], 32-bit, on the host
        V = logits.shape[-1]
        scores = torch.full((B, nb), float("-inf"))
        scores[:, 0] = 0.0                                               # the beams start out identical: one counts
        tokens = [[[] for _ in range(nb)] for _ in range(B)]             # new tokens of every running beam
        finished = [[] for _ in range(B)]                                # (score, tokens) of ended continuations
        done = [False] * B
        cur = T0
        for step in range(max_new_tokens):
            logp = torch.log_softmax(logits.float(), dim=-1).view(B, nb, V) + scores[:, :, None]
            vals, idx = torch.topk(logp.view(B, nb * V), min(2 * nb, nb * V), dim=1)
            src = list(range(B * nb))
            nxt = [fill] * (B * nb)
            for b in range(B):
                if done[b]:
                    continue
                keep = []
                for rank, (v, i) in enumerate(zip(vals[b].tolist(), idx[b].tolist())):
                    beam, tok = divmod(i, V)
                    if v == float("-inf"):
                        break
                    if tok in eos:
                        if rank < nb:                                    # only if it would have been kept as a beam
                            seq = tokens[b][beam] + [tok]
                            finished[b].append((v / (len(seq) ** length_penalty), seq))
                        continue
                    keep.append((v, beam, tok))
                    if len(keep) == nb:
                        break
                if len(finished[b]) >= nb:
                    finished[b] = sorted(finished[b], key=lambda h: -h[0])[:nb]
                    best_running = max((k[0] for k in keep), default=float("-inf")) / ((step + 1) ** length_penalty)
                    if early_stopping or not keep or best_running <= finished[b][-1][0]:
                        done[b] = True
                        continue
                if not keep:                                             # every candidate ended: nothing left to run
                    done[b] = True
                    continue
                new_tokens = []
                for j in range(nb):
                    v, beam, tok = keep[j] if j < len(keep) else (float("-inf"), keep[0][1], keep[0][2])
                    scores[b, j] = v
                    src[b * nb + j] = b * nb + beam
                    nxt[b * nb + j] = tok
                    new_tokens.append(tokens[b][beam] + [tok])
                tokens[b] = new_tokens
            if all(done) or step == max_new_tokens - 1:
                break
            m.reorder_cache(src)
            logits = last(m(torch.tensor(nxt, dtype=input_ids.dtype)[:, None], torch.tensor([cur], dtype=torch.int32), row_starts))
            cur += 1
        outs = []
        for b in range(B):
            cands = list(finished[b])
            if not done[b] or not cands:                                 # ran to the limit: the running beams count too
                for j in range(nb):
                    if scores[b, j] > float("-inf") and tokens[b][j]:
                        cands.append((float(scores[b, j]) / (len(tokens[b][j]) ** length_penalty), tokens[b][j]))
            outs.append(max(cands, key=lambda h: h[0])[1])
        length = max(len(o) for o in outs)
        outs = [o + [fill] * (length - len(o)) for o in outs]
        self.reset_generation()
        self.cur_len = T0 + length
        return torch.cat([input_ids, torch.as_tensor(outs, dtype=input_ids.dtype)], dim=1)

