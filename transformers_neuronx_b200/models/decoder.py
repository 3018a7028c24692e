"""A decoder put together from parts according to a ModelSpec: embedding, the scheduled layers,
head.  It knows no architecture: models/opt.py (or a test) supplies the specification."""
from __future__ import annotations

import contextlib
from typing import Dict, List, Optional

import torch

from ..kernels import build as kbuild
from ..kernels import ops
from ..parts import Embedding, Head, build_block, build_part
from ..parts.spec import ModelSpec
from ..weights.loader import TensorSpec


class DecoderModel:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.embedding = Embedding(spec.embedding)
        self.blocks = []
        for ls in spec.layers:
            self.blocks.append(build_block(ls.block, build_part("norm", ls.norm1), build_part("mixer", ls.mixer),
                                           build_part("norm", ls.norm2),
                                           build_part("feed_forward", ls.feed_forward)))
        self.head = Head(spec.head)
        for e in spec.schedule:
            if not (0 <= e.layer < len(self.blocks)):
                raise ValueError(f"schedule names layer {e.layer}, the model has {len(self.blocks)}")
        self.device = None
        self.act_dtype = None
        self._taps: Optional[Dict[str, torch.Tensor]] = None

    # ---- taps -----------------------------------------------------------------------------------
    @contextlib.contextmanager
    def tap_hidden_states(self):
        """Inside the block every step leaves copies of its intermediate results in the dictionary
        that is yielded: "embedding", "entry<i>" (the 32-bit residual stream [tokens, hidden] after
        the i-th schedule entry) and "logits"; a later step overwrites them.  Steps run eagerly
        meanwhile (a captured graph would write into buffers of its own).  The counterpart of the
        reference's named debug tensors (src/transformers_neuronx/global_debugger.py:27-91)."""
        taps: Dict[str, torch.Tensor] = {}
        prev, self._taps = self._taps, taps
        try:
            yield taps
        finally:
            self._taps = prev

    # ---- parts, tensors, kernels --------------------------------------------------------------
    def all_parts(self):
        out = [self.embedding]
        for b in self.blocks:
            out += b.parts()
        out.append(self.head)
        return out

    def tensor_specs(self) -> List[TensorSpec]:
        seen, out = set(), []
        for p in self.all_parts():
            for s in p.tensor_specs():
                if s.name not in seen:
                    seen.add(s.name)
                    out.append(s)
        return out

    def libraries(self, act_dtype=None) -> List[str]:
        """Kernel libraries worth compiling before the first step (the rest are compiled when first used)."""
        libs = []
        for p in self.all_parts():
            libs += [l for l in p.libraries if l in kbuild.SOURCES]
        if act_dtype == torch.float32:
            libs = [l for l in libs if l not in ("gemm_tc", "gemv", "attention_prefill", "attention_prefill_tc", "attention_decode")]
        return list(dict.fromkeys(libs))

    @property
    def graph_safe(self) -> bool:
        """Whether a step of this model can be captured in a CUDA graph now (every part says so,
        and nobody is tapping intermediate results)."""
        return self._taps is None and all(getattr(p, "graph_safe", False) for p in self.all_parts())

    def cache_needs(self) -> Dict[int, object]:
        """{cache id -> what the mixer(s) using it keep}; entries sharing a cache must agree."""
        needs: Dict[int, object] = {}
        for e in self.spec.schedule:
            need = self.blocks[e.layer].mixer.cache_need()
            if e.cache in needs and needs[e.cache] != need:
                raise ValueError(f"cache {e.cache} is shared by mixers with different needs: "
                                 f"{needs[e.cache]} and {need}")
            needs[e.cache] = need
        return needs

    def load(self, tensors: Dict[str, torch.Tensor], device, act_dtype) -> None:
        self.device, self.act_dtype = device, act_dtype
        self.embedding.load(tensors, device, act_dtype)
        for b in self.blocks:
            for p in b.parts():
                p.load(tensors, device, act_dtype)
        self.head.load(tensors, device, act_dtype, shared={self.spec.embedding.table: self.embedding.table})

    def parameter_bytes(self) -> int:
        """Bytes of every weight one step reads once (a tied table counted once)."""
        n, seen = 0, set()
        for p in self.all_parts():
            n += p.parameter_bytes()
        if self.head.weight is self.embedding.table:
            n -= self.head.weight.numel() * self.head.weight.element_size()
        return n

    # ---- one step -------------------------------------------------------------------------------
    def forward(self, ctx) -> torch.Tensor:
        """Runs the tokens of ctx through the scheduled layers; returns 32-bit logits of ctx.logit_rows
        ([0, vocab] when none is wanted)."""
        N, H = ctx.n_tokens, self.spec.hidden_size
        x = ctx.empty(N, H, torch.float32)
        first = self.blocks[self.spec.schedule[0].layer] if self.spec.schedule else None
        want_act = any(self.blocks[e.layer].needs_act_input for e in self.spec.schedule)
        x_act = ctx.empty(N, H) if want_act else None
        self.embedding.forward(ctx, x, x_act if (first is not None and first.needs_act_input) else None)
        act_current = first is not None and first.needs_act_input
        taps = self._taps
        if taps is not None:
            taps.clear()
            taps["embedding"] = x.clone()
        for i, e in enumerate(self.spec.schedule):
            block = self.blocks[e.layer]
            if block.needs_act_input and not act_current:
                ops.pick_rows(x, None, out_act=x_act)
            ctx.cache_id = e.cache
            ctx.begin_entry()
            block.forward(ctx, x, x_act)
            act_current = block.keeps_act_current
            if taps is not None:
                taps[f"entry{i}"] = x.clone()
        if ctx.logit_rows is None or ctx.logit_rows.shape[0] == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=ctx.device)
        logits = self.head.forward(ctx, x, ctx.logit_rows)
        if taps is not None:
            taps["logits"] = logits.clone()
        return logits
