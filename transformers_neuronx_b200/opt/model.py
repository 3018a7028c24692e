"""The Python entry point in the reference's manner:

    model = OPTForSampling.from_pretrained(path, batch_size=4, amp='bf16', n_positions=2048)
    model.to_neuron()
    tokens = model.sample(input_ids, sequence_length=2048)

Names and meanings follow src/transformers_neuronx/opt/model.py:34-192: ``sequence_length`` is the
total length (prompt included); ``sample`` draws from the top_k (default 50) most likely tokens and
never draws the end-of-sequence token (sampling.py:26-30, :131-180); ``top_k=1`` is greedy, as in
the reference's own validation (testing/validation.py:68-101); ``forward(input_ids, cache_ids,
start_ids)`` returns the 32-bit logits [batch, vocab] of each row's last token (of every position of
the prompts with ``NeuronConfig(output_all_logits=True)``); ``start_ids`` marks left padding;
``save`` / ``load`` keep the compiled kernels in a folder between processes.  With ``neuron_config=NeuronConfig(on_device_generation=GenerationConfig(...))``
``sample`` chooses tokens as that configuration says (opt/model.py:187-189, sampling.py:34-105).
``tp_degree``, ``unroll`` and ``context_length_estimate`` have no meaning on one GPU and are accepted
and ignored with a warning.  ``to_neuron`` loads the weights onto the GPU and compiles the kernels
that the model needs.
"""
from __future__ import annotations

import os
import warnings
from typing import List, Optional

import torch

from ..config import EngineConfig, GenerationConfig, NeuronConfig, OPTConfig, canonical_dtype, load_config
from ..engine import LLMEngine, SamplingParams, StepEntry, load_model
from ..kernels import ops


class OPTForSampling:
    def __init__(self, folder: str, config: OPTConfig, batch_size=1, amp=None, tp_degree=None, n_positions=2048,
                 unroll=None, context_length_estimate=None, context_unroll=None, neuron_config=None, **kwargs):
        for name, val in (("tp_degree", tp_degree), ("unroll", unroll), ("context_unroll", context_unroll),
                          ("context_length_estimate", context_length_estimate)):
            if val is not None:
                warnings.warn(f"{name}={val!r} has no meaning for the one-GPU engine and is ignored")
        if neuron_config is not None and not isinstance(neuron_config, NeuronConfig):
            raise TypeError("neuron_config must be a NeuronConfig of this package")
        self.neuron_config = neuron_config or NeuronConfig()
        if kwargs:
            raise KeyError(f"unknown argument(s): {sorted(kwargs)}")
        if amp is None:                  # the checkpoint's own type (opt/model.py:38-41, dtypes.py:29-35)
            amp = {"float16": "f16", "bfloat16": "bf16"}.get(str(config.torch_dtype).replace("torch.", ""), "f32")
        self.amp = amp
        self.dtype = canonical_dtype(amp)
        max_bucket = max(n_positions) if isinstance(n_positions, (list, tuple)) else n_positions
        if max_bucket > config.max_position_embeddings:     # opt/model.py:51-57
            raise ValueError(f"Sequence length ({max_bucket}) cannot be larger than position embedding's "
                             f"context size ({config.max_position_embeddings})!")
        self.folder = folder
        self.config = config
        self.batch_size = max(batch_size) if isinstance(batch_size, (list, tuple)) else int(batch_size)
        if self.neuron_config.continuous_batching is not None:      # as many cache lines as sequences may be alive
            self.batch_size = max(self.batch_size, self.neuron_config.continuous_batching.max_num_seqs)
        self.n_positions = int(max_bucket)
        self.engine: Optional[LLMEngine] = None
        self.model = None
        self._rows: List[str] = []
        self._seqs = set()              # sequence ids alive under continuous batching

    # ---- loading ------------------------------------------------------------------------------------
    @classmethod
    def from_pretrained(cls, pretrained_model_path, *model_args, **kwargs):
        if not os.path.isdir(pretrained_model_path):
            raise FileNotFoundError(f"{pretrained_model_path!r} is not a folder; there is no network here to "
                                    "fetch a model by name")
        arch, config = load_config(pretrained_model_path)
        if arch.name != "OPTForCausalLM":
            raise ValueError(f"{pretrained_model_path} holds a {arch.name}, not an OPT model")
        return cls(pretrained_model_path, config, *model_args, **kwargs)

    def to_neuron(self):
        """Weights to the GPU, kernels compiled, cache made.  Kept under the reference's name."""
        if self.engine is not None:
            return self
        self.model, _ = load_model(self.folder, self.dtype, spec_hook=self._spec_hook())
        ec = EngineConfig(dtype=self.dtype, max_num_seqs=max(self.batch_size, 1), max_model_len=self.n_positions,
                          max_tokens=self.batch_size * (-(-self.n_positions // 16) * 16),
                          max_batch_tokens=max(2048, self.batch_size))
        self.engine = LLMEngine(self.model, ec, eos_token_id=self.config.eos_token_id)
        return self

    to_gpu = to_neuron

    def _spec_hook(self):
        """NeuronConfig(sparse_attn=...) of the sliding-window kind: every attention layer gets the window."""
        sa = self.neuron_config.sparse_attn
        if sa is None:
            return None
        import dataclasses

        def with_window(spec):
            layers = tuple(dataclasses.replace(l, mixer=dataclasses.replace(l.mixer, window=sa.keys_attended))
                           if hasattr(l.mixer, "window") else l for l in spec.layers)
            return dataclasses.replace(spec, layers=layers)
        return with_window

    # ---- compiled kernels kept between processes (base.py:110-190: save / load of compiled artifacts) ----
    def save(self, directory: str) -> None:
        """Writes the compiled kernel libraries this model uses into `directory`."""
        from ..kernels import build as kbuild
        self._ready()
        kbuild.export_libraries(self.model.libraries(self.model.act_dtype), directory)

    def load(self, directory: str) -> None:
        """Call before to_neuron(): kernels compiled earlier (by save) from the same sources are
        taken from `directory` instead of being compiled again."""
        from ..kernels import build as kbuild
        kbuild.import_libraries(directory)

    def is_compiled(self) -> bool:
        """Whether every kernel library this model needs is built already (base.py:143-151 asks the same of
        its compiled kernels)."""
        from ..kernels import build as kbuild
        from ..models.decoder import DecoderModel
        import torch as _torch
        act = {"float32": _torch.float32, "bfloat16": _torch.bfloat16, "float16": _torch.float16}[self.dtype]
        if self.model is not None:
            libs = self.model.libraries(self.model.act_dtype)
        else:
            arch, cfg = load_config(self.folder)
            libs = DecoderModel(arch.build_spec(cfg)).libraries(act)
        return all(os.path.isfile(kbuild.library_path(n)) for n in kbuild.with_flavour(libs, act))

    def profile(self, profile_dir: str, ntff_count_limit=None) -> str:
        """Where the time of a prompt step and a few decode steps goes, kernel family by kernel family
        (CUDA events around every kernel call, graphs off meanwhile), written to
        `profile_dir`/kernel_profile.txt and returned.  The reference runs each compiled kernel under the
        Neuron profiler here (base.py:754-759); `ntff_count_limit` is its option and has no meaning here."""
        from ..kernels.profile import kernel_profile
        self._ready()
        self.reset()
        runner = self.engine.runner
        n_prompt = max(1, min(64, self.n_positions // 2))
        n_decode = max(0, min(8, self.n_positions - n_prompt - 1))
        ids = [[self.config.bos_token_id] + [3 + (7 * i + b) % (self.config.vocab_size - 3) for i in range(1, n_prompt)]
               for b in range(self.batch_size)]
        graphs, runner.use_cuda_graphs = runner.use_cuda_graphs, False
        try:
            with kernel_profile() as prof:
                self.forward(torch.tensor(ids))
                for t in range(n_decode):
                    self.forward(torch.full((self.batch_size, 1), 5, dtype=torch.long), torch.tensor([n_prompt + t]))
            report = (f"{self.batch_size} rows: one step of {n_prompt}-token prompts and {n_decode} decode steps, "
                      f"{self.dtype}\n" + prof.report() + "\n")
        finally:
            runner.use_cuda_graphs = graphs
            self.reset()
        os.makedirs(profile_dir, exist_ok=True)
        with open(os.path.join(profile_dir, "kernel_profile.txt"), "w") as fp:
            fp.write(report)
        return report

    def update_generation_config(self, generation_config: GenerationConfig) -> None:
        """Replaces the on-device generation settings; the next sample() call uses them (base.py:761-762)."""
        if not isinstance(generation_config, GenerationConfig):
            raise TypeError("generation_config must be a GenerationConfig of this package")
        self.neuron_config.on_device_generation = generation_config

    def _ready(self):
        if self.engine is None:
            self.to_neuron()

    # ---- generation ---------------------------------------------------------------------------------
    def sample(self, input_ids, sequence_length, start_ids=None, top_k=50, streamer=None, temperature=1.0,
               top_p=1.0, seed=0):
        """[batch, prompt] ids -> [batch, sequence_length] ids (prompt included).  With an
        on_device_generation configuration the tokens are chosen as it says and top_k, temperature
        and top_p of this call are not used."""
        self._ready()
        input_ids = torch.as_tensor(input_ids)
        B, T0 = input_ids.shape
        if self.neuron_config.on_device_generation is not None:
            return self._sample_tokens(input_ids, sequence_length, start_ids, self.neuron_config.on_device_generation,
                                       streamer, seed)
        if B > self.batch_size:
            raise ValueError(f"batch of {B} rows; the model was made for batch_size={self.batch_size}")
        if sequence_length > self.n_positions:
            raise ValueError(f"sequence_length {sequence_length} exceeds n_positions {self.n_positions}")
        starts = [0] * B if start_ids is None else [int(s) for s in torch.as_tensor(start_ids).tolist()]
        rows = input_ids.tolist()
        prompts = [rows[b][starts[b]:] for b in range(B)]
        n_new = sequence_length - T0
        if n_new <= 0:
            return input_ids[:, :sequence_length]
        greedy = top_k == 1
        params = [SamplingParams(temperature=0.0 if greedy else float(temperature), top_k=0 if greedy else int(top_k or 0),
                                 top_p=float(top_p), seed=int(seed) + b, suppress_eos=True) for b in range(B)]
        outs = self._generate(prompts, n_new, params, streamer, input_ids.dtype)
        return torch.cat([input_ids, torch.as_tensor(outs, dtype=input_ids.dtype)], dim=1)

    def _generate(self, prompts, n_new, params, streamer, dtype, eos=None, pad=None):
        """Runs the rows to the end.  With a streamer every new column of tokens is handed to it
        (`put` of a [batch, 1] tensor) as soon as all its ids are known, and `end` is called last
        (sampling.py:159-160, :172-173); rows that are finished are filled with `pad` (the first eos
        id when none is given)."""
        eng = self.engine
        stop = eos is not None
        fill = (eos[0] if pad is None else int(pad)) if stop else None
        if streamer is None:
            outs = eng.generate(prompts, n_new, params, stop_on_eos=stop, eos_token_id=eos)
        else:
            rids = [eng.add_request(p, n_new, q, stop_on_eos=stop, eos_token_id=eos) for p, q in zip(prompts, params)]
            reqs = [eng.requests[r] for r in rids]
            sent = 0
            while eng.has_work():
                eng.step()
                while True:
                    col = []
                    for r in reqs:
                        if sent < len(r.output) and r.output[sent] != eng.PENDING:
                            col.append(r.output[sent])
                        elif r.finished and sent >= len(r.output) and stop and any(sent < len(o.output) for o in reqs):
                            col.append(fill)
                        else:
                            col = None
                            break
                    if col is None:
                        break
                    streamer.put(torch.tensor(col, dtype=dtype)[:, None])
                    sent += 1
            streamer.end()
            outs = [r.output for r in reqs]
            for rid in rids:
                del eng.requests[rid]
        if stop:
            length = max(len(o) for o in outs)
            outs = [o + [fill] * (length - len(o)) for o in outs]
        return outs

    def _sample_tokens(self, input_ids, sequence_length, start_ids, gen: GenerationConfig, streamer, seed):
        """The reference's loop for a model that chooses its tokens itself (sampling.py:34-105):
        without eos_token_id every row runs to sequence_length; with it, a row that produced the id
        is filled with it from there on and the result ends where the last row finished."""
        B, T0 = input_ids.shape
        if B > self.batch_size:
            raise ValueError(f"batch of {B} rows; the model was made for batch_size={self.batch_size}")
        limit = self.n_positions if gen.max_length is None else min(self.n_positions, int(gen.max_length))
        if sequence_length > limit:
            raise ValueError(f"sequence_length {sequence_length} exceeds the longest sequence {limit}")
        starts = [0] * B if start_ids is None else [int(s) for s in torch.as_tensor(start_ids).tolist()]
        rows = input_ids.tolist()
        prompts = [rows[b][starts[b]:] for b in range(B)]
        n_new = sequence_length - T0
        if n_new <= 0:
            return input_ids[:, :sequence_length]
        params = []
        for b in range(B):
            k, p, t, n_min = gen.for_row(b)
            if gen.is_greedy():
                params.append(SamplingParams(temperature=0.0))
            else:
                params.append(SamplingParams(temperature=t, top_k=k, top_p=p, seed=int(seed) + b, top_p_min_tokens=n_min,
                                             deterministic=gen.deterministic))
        eos = gen.eos_ids()
        outs = self._generate(prompts, n_new, params, streamer, input_ids.dtype, eos=tuple(eos) if eos else None)
        return torch.cat([input_ids, torch.as_tensor(outs, dtype=input_ids.dtype)], dim=1)

    # ---- the static-batch forward of the reference ---------------------------------------------------------
    def reset(self):
        if self.engine is not None:
            for rid in self._rows + [("seq", s) for s in self._seqs]:
                if rid in self.engine.runner.cache:
                    self.engine.runner.finish(rid)
        self._rows = []
        self._seqs = set()

    def forward(self, input_ids, cache_ids=None, start_ids=None):
        """cache_ids None: the rows are whole prompts (a new batch).  Otherwise input_ids holds the
        next token(s) of every row at positions cache_ids.  Returns 32-bit logits [batch, vocab] of
        the last token of each row, on the host."""
        self._ready()
        input_ids = torch.as_tensor(input_ids)
        B, T = input_ids.shape
        runner = self.engine.runner
        if self.neuron_config.continuous_batching is not None and start_ids is not None and cache_ids is not None:
            return self._forward_sequences(input_ids, torch.as_tensor(cache_ids), torch.as_tensor(start_ids))
        starts = [0] * B if start_ids is None else [int(s) for s in torch.as_tensor(start_ids).tolist()]
        if cache_ids is None:
            self.reset()
            self._rows = [f"row{b}" for b in range(B)]
            for rid in self._rows:
                runner.add_request(rid)
            toks = [input_ids[b, starts[b]:].tolist() for b in range(B)]
        else:
            first = int(torch.as_tensor(cache_ids).flatten()[0])
            toks = [input_ids[b].tolist() for b in range(B)]
            for b, rid in enumerate(self._rows):
                have = runner.cache.length(rid)
                if have != first - starts[b]:
                    raise ValueError(f"row {b} holds {have} tokens; cache_ids says {first - starts[b]}")
        if self.neuron_config.output_all_logits and cache_ids is None:
            # logits of every position [batch, tokens, vocab] (base.py:716-717); left padding holds zeros
            entries = [StepEntry(rid, t, list(range(len(t)))) for rid, t in zip(self._rows, toks)]
            flat = runner.step(entries).to("cpu", torch.float32)
            ops.raise_on_device_error()
            out = torch.zeros(B, T, flat.shape[1])
            row = 0
            for b, t in enumerate(toks):
                out[b, T - len(t):] = flat[row:row + len(t)]
                row += len(t)
            return self._cast_logits(out)
        entries = [StepEntry(rid, t, [len(t) - 1]) for rid, t in zip(self._rows, toks)]
        logits = runner.step(entries).to("cpu", torch.float32)
        ops.raise_on_device_error()           # a bounded wait that ran out inside a kernel: the logits are invalid
        return self._cast_logits(logits)

    def _cast_logits(self, logits):
        """The logits in NeuronConfig.cast_logits_dtype (32-bit unless asked otherwise; base.py:641-647)."""
        return logits.to(getattr(torch, self.neuron_config.cast_logits_dtype))

    __call__ = forward

    def _forward_sequences(self, input_ids, cache_ids, seq_ids):
        """forward() under NeuronConfig(continuous_batching=...), as a serving loop outside the model drives
        the reference (base.py:492-587, :613-639): row i belongs to sequence seq_ids[i], which owns a cache
        line; cache_ids [rows, tokens] holds the positions of the row's tokens, a shorter row padded on the
        right with zeros.  A row that starts at position 0 begins its sequence anew (what the line held is
        given back); any other row goes on where its sequence ends, with one token or with a further
        portion.  Rows of different kinds may share a call.  Returns the logits [rows, vocab] of each row's
        last token, 32-bit, on the host."""
        runner = self.engine.runner
        B, T = input_ids.shape
        cache_ids = cache_ids.reshape(B, -1)
        if cache_ids.shape[1] != T or seq_ids.numel() != B:
            raise ValueError("cache_ids must be [rows, tokens] like input_ids, with one sequence id per row")
        lines = self.neuron_config.continuous_batching.max_num_seqs
        entries, seen = [], set()
        for b in range(B):
            sid = int(seq_ids.flatten()[b])
            if not 0 <= sid < lines or sid in seen:
                raise ValueError(f"row {b}: sequence id {sid} (ids are 0..{lines - 1}, each at most once a call)")
            seen.add(sid)
            rid = ("seq", sid)
            pos = cache_ids[b].tolist()
            count = 1 if T == 1 else max(pos) - pos[0] + 1
            if pos[:count] != list(range(pos[0], pos[0] + count)):
                raise ValueError(f"row {b}: positions {pos[:count]} are not consecutive")
            if pos[0] == 0:
                if rid in runner.cache:
                    runner.finish(rid)
                runner.add_request(rid)
                self._seqs.add(sid)
            elif rid not in runner.cache or runner.cache.length(rid) != pos[0]:
                have = runner.cache.length(rid) if rid in runner.cache else 0
                raise ValueError(f"row {b}: sequence {sid} holds {have} tokens; cache_ids says {pos[0]}")
            entries.append(StepEntry(rid, input_ids[b, :count].tolist(), [count - 1]))
        logits = runner.step(entries).to("cpu", torch.float32)
        ops.raise_on_device_error()
        return self._cast_logits(logits)

    def reorder_cache(self, reorder_ids) -> None:
        """Row i of the running batch goes on from what row reorder_ids[i] holds: the cache side of beam
        search (src/transformers_neuronx/base.py:153-154, decoder.py:2303-2320, which gather whole cache
        lines).  Here the rows' pages change hands, and only a row that a second beam also goes on from
        is copied.  Rows may only go on from rows that hold as many tokens (the beams of one prompt)."""
        self._ready()
        ids = [int(i) for i in torch.as_tensor(reorder_ids).flatten().tolist()]
        if len(ids) != len(self._rows):
            raise ValueError(f"reorder_cache got {len(ids)} indices for {len(self._rows)} rows")
        runner = self.engine.runner
        by_length = {}
        for i, rid in enumerate(self._rows):
            by_length.setdefault(runner.cache.length(rid), []).append(i)
        for length, members in by_length.items():
            local = {i: j for j, i in enumerate(members)}
            if any(ids[i] not in local for i in members):
                raise ValueError("a row can only go on from a row that holds as many tokens")
            runner.reorder([self._rows[i] for i in members], [local[ids[i]] for i in members])

    def setup_reorder_cache(self) -> None:
        """The reference compiles its reorder kernel on request (base.py:156-160); nothing to prepare here."""


class OPTForGreedySearch(OPTForSampling):
    """Greedy search with the choice made on the device (opt/model.py:534-570)."""

    def sample(self, input_ids, sequence_length, start_ids=None, **_):
        return super().sample(input_ids, sequence_length, start_ids=start_ids, top_k=1)
