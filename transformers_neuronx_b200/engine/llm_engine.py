"""Requests in, tokens out: the scheduler, the step function and the sampler in one loop."""
from __future__ import annotations

import itertools
from typing import Dict, Hashable, List, Optional, Sequence

import torch

from ..config import EngineConfig
from ..sampling import Sampler
from .scheduler import Request, SamplingParams, Scheduler, StepPlan
from .step import StepEntry, StepRunner


class LLMEngine:
    def __init__(self, model, engine_config: EngineConfig, eos_token_id: Optional[int] = None):
        self.model = model
        self.config = engine_config
        ec = engine_config
        max_len = min(ec.max_model_len or model.spec.max_positions, model.spec.max_positions)
        if ec.num_pages is not None:
            num_pages = ec.num_pages
        else:
            tokens = ec.max_tokens if ec.max_tokens is not None else ec.max_num_seqs * max_len
            num_pages = -(-tokens // ec.page_size)
        self.runner = StepRunner(model, ec.page_size, num_pages, ec.max_num_seqs, max_len,
                                 use_cuda_graphs=ec.use_cuda_graphs)
        self.scheduler = Scheduler(self.runner.cache, ec.max_batch_tokens, ec.max_num_seqs, max_len)
        self.sampler = Sampler(model.device)
        self.eos_token_id = model.spec.eos_token_id if eos_token_id is None else eos_token_id
        self._ids = itertools.count()
        self.requests: Dict[Hashable, Request] = {}
        self.stats = {"steps": 0, "tokens_run": 0, "tokens_sampled": 0, "preemptions": 0}

    def add_request(self, prompt: Sequence[int], max_new_tokens: int, params: Optional[SamplingParams] = None,
                    rid: Optional[Hashable] = None, stop_on_eos: bool = True) -> Hashable:
        rid = next(self._ids) if rid is None else rid
        if rid in self.requests and not self.requests[rid].finished:
            raise ValueError(f"request {rid!r} is still running")
        req = Request(rid, [int(t) for t in prompt], int(max_new_tokens), params or SamplingParams(),
                      stop_on_eos=stop_on_eos, eos_token_id=self.eos_token_id)
        self.scheduler.add(req)
        self.requests[rid] = req
        return rid

    def has_work(self) -> bool:
        return self.scheduler.has_work()

    @torch.no_grad()
    def step(self) -> List[Request]:
        """One scheduler decision, one model step, one sampling call.  Returns finished requests."""
        plan: StepPlan = self.scheduler.schedule()
        entries, rows = [], []
        for it in plan.items:
            all_tokens = it.request.tokens
            toks = all_tokens[it.start:it.start + it.count] if it.count > 1 else [all_tokens[it.start]]
            entries.append(StepEntry(it.request.rid, toks, [it.count - 1] if it.sample else []))
            if it.sample:
                rows.append(it.request)
        logits = self.runner.step(entries)
        sampled: Dict[Hashable, int] = {}
        if rows:
            suppress = self.eos_token_id if (self.eos_token_id is not None and
                                             all(r.params.suppress_eos for r in rows)) else -1
            if suppress < 0 and any(r.params.suppress_eos for r in rows):
                raise ValueError("suppress_eos must be set for all requests of a step or for none")
            ids = self.sampler.sample(
                logits, [r.params.temperature for r in rows], [r.params.top_k for r in rows],
                [r.params.top_p for r in rows], [r.params.seed for r in rows],
                [len(r.output) for r in rows], suppress_id=suppress)
            host = ids.tolist()                       # the step's one device-to-host read
            sampled = {r.rid: t for r, t in zip(rows, host)}
        done = self.scheduler.commit(plan, sampled)
        for r in done:
            self.runner.forget(r.rid)
        for r in plan.preempted:
            self.runner.forget(r.rid)
        self.stats["steps"] += 1
        self.stats["tokens_run"] += plan.n_tokens
        self.stats["tokens_sampled"] += len(rows)
        self.stats["preemptions"] = self.scheduler.num_preemptions
        return done

    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens, params=None,
                 stop_on_eos: bool = True) -> List[List[int]]:
        """Runs the given prompts to the end; returns the new tokens of each."""
        n = len(prompts)
        mnt = max_new_tokens if isinstance(max_new_tokens, (list, tuple)) else [max_new_tokens] * n
        ps = params if isinstance(params, (list, tuple)) else [params] * n
        rids = [self.add_request(p, m, q, stop_on_eos=stop_on_eos) for p, m, q in zip(prompts, mnt, ps)]
        while self.has_work():
            self.step()
        out = [self.requests[r].output for r in rids]
        for r in rids:
            del self.requests[r]
        return out
