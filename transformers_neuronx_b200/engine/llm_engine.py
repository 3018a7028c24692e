"""Requests in, tokens out: the scheduler, the step function and the sampler in one loop."""
from __future__ import annotations

import itertools
from typing import Dict, Hashable, List, Optional, Sequence

import torch

from ..config import EngineConfig
from ..kernels import ops
from ..sampling import MAX_SUPPRESSED, Sampler, needs_top_p, pack_rows
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
        self.scheduler = Scheduler(self.runner.cache, ec.max_batch_tokens, ec.max_num_seqs, max_len,
                                   max_portion=ec.max_portion)
        self.sampler = Sampler(model.device)
        self.eos_token_id = model.spec.eos_token_id if eos_token_id is None else eos_token_id
        self._ids = itertools.count()
        self.requests: Dict[Hashable, Request] = {}
        # the ids sampled in a step, and after them the kernels' error word (one more entry)
        n_ids = max(64, 2 * ec.max_num_seqs) + 1
        self._ids_dev = [torch.zeros(n_ids, dtype=torch.int32, device=model.device) for _ in range(2)]
        self._ids_host = [torch.zeros(n_ids, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._err_word = ops.error_word(model.device)
        self._events = [torch.cuda.Event() for _ in range(2)]
        self._parity = 0
        self._inflight = None          # the last step's sampled ids, not yet read back
        self._awaiting: List[Request] = []   # finished requests whose last ids are still on their way
        self.stats = {"steps": 0, "tokens_run": 0, "tokens_sampled": 0, "preemptions": 0}

    def add_request(self, prompt: Sequence[int], max_new_tokens: int, params: Optional[SamplingParams] = None,
                    rid: Optional[Hashable] = None, stop_on_eos: bool = True, eos_token_id=None,
                    max_time: Optional[float] = None) -> Hashable:
        rid = next(self._ids) if rid is None else rid
        if rid in self.requests and not self.requests[rid].finished:
            raise ValueError(f"request {rid!r} is still running")
        req = Request(rid, [int(t) for t in prompt], int(max_new_tokens), params or SamplingParams(),
                      stop_on_eos=stop_on_eos, eos_token_id=self.eos_token_id if eos_token_id is None else eos_token_id,
                      max_time=max_time)
        if req.params.suppress_eos and len(req.eos_ids()) > MAX_SUPPRESSED:
            raise ValueError(f"request {rid!r}: suppress_eos takes at most {MAX_SUPPRESSED} end-of-sequence ids, "
                             f"got {len(req.eos_ids())}")
        self.scheduler.add(req)
        self.requests[rid] = req
        return rid

    def has_work(self) -> bool:
        return self.scheduler.has_work() or self._inflight is not None

    # A sampled id is needed by the host for three things: as the next input of its request, to
    # notice the end-of-sequence token, and to hand it to the caller.  Only the first is urgent,
    # and it does not need the host: the next step takes the id from where the sampling kernel
    # left it on the device.  So a step is launched before the ids of the step before it have
    # been read back; the request's output holds -1 at that place meanwhile.  A request that
    # produced the end-of-sequence token is noticed one step late: the step that was already
    # launched for it is wasted and its token dropped.
    PENDING = -1

    @torch.no_grad()
    def step(self) -> List[Request]:
        """One scheduler decision, one model step, one sampling call.  Returns the requests that
        finished and whose tokens are all known."""
        if not self.scheduler.has_work():
            finished = self._resolve(self._inflight)
            self._inflight = None
            return finished
        plan: StepPlan = self.scheduler.schedule()
        for r in plan.preempted:
            self.runner.forget(r.rid)
        entries, rows = [], []
        any_from_device = False
        for it in plan.items:
            req = it.request
            all_tokens = req.tokens
            src = None
            if it.count == 1:
                tok = all_tokens[it.start]
                if tok == self.PENDING:
                    src, tok = req._dev_row, 0
                    any_from_device = True
                toks = [tok]
            else:
                toks = all_tokens[it.start:it.start + it.count]
                if self.PENDING in toks[-2:]:
                    raise AssertionError(f"request {req.rid!r}: a portion holds a token that is not known yet")
            entries.append(StepEntry(req.rid, toks, [it.count - 1] if it.sample else [], from_device=src))
            if it.sample:
                rows.append(req)
        prev_ids = self._ids_dev[self._parity ^ 1] if any_from_device else None
        # The rows to sample, with every row's own parameters (temperature, top-k, top-p, seed and
        # counter, the fixed draw, the ids it must not draw), packed into the step's own staging buffer.
        extra = None
        if rows:
            ps = [r.params for r in rows]
            extra = pack_rows([p.temperature for p in ps], [p.top_k for p in ps], [p.top_p for p in ps],
                              [p.seed for p in ps], [len(r.output) for r in rows], [p.top_p_min_tokens for p in ps],
                              [p.deterministic for p in ps], [r.eos_ids() if r.params.suppress_eos else () for r in rows])
        logits = self.runner.step(entries, prev_ids, extra)
        cur = None
        if rows:
            R = len(rows)
            if self._ids_dev[self._parity].shape[0] < R + 1:
                if any_from_device:
                    raise AssertionError("the batch outgrew the id buffers while ids were still on the device")
                self._ids_dev = [torch.zeros(2 * R + 1, dtype=torch.int32, device=self.model.device) for _ in range(2)]
                self._ids_host = [torch.zeros(2 * R + 1, dtype=torch.int32).pin_memory() for _ in range(2)]
            out = self._ids_dev[self._parity]
            self.sampler.sample_packed(logits, self.runner.extra_dev, needs_top_p([p.top_p for p in ps],
                                                                                 [p.deterministic for p in ps]),
                                       out, err_word=self._err_word)
            host = self._ids_host[self._parity]
            host[:R + 1].copy_(out[:R + 1], non_blocking=True)    # the step's device-to-host read, waited for later
            ev = self._events[self._parity]
            ev.record()
            for i, r in enumerate(rows):
                r._dev_row = i
            cur = (rows, [len(r.output) for r in rows], host, ev, R, self.stats["steps"])
        done_by_count = self.scheduler.commit(plan, {r.rid: self.PENDING for r in rows})
        for r in done_by_count:
            self.runner.forget(r.rid)
        self._awaiting.extend(done_by_count)
        self.stats["steps"] += 1
        self.stats["tokens_run"] += plan.n_tokens
        self.stats["tokens_sampled"] += len(rows)
        self.stats["preemptions"] = self.scheduler.num_preemptions
        if self.config.async_scheduling:
            finished = self._resolve(self._inflight)      # the step before this one
            self._inflight = cur
        else:
            finished = self._resolve(self._inflight) + self._resolve(cur)
            self._inflight = None
        self._parity ^= 1
        return finished

    def _resolve(self, inflight) -> List[Request]:
        """Waits for a step's sampled ids, writes them over the placeholders, and ends requests
        that produced the end-of-sequence token.  Returns requests that are finished with all
        their tokens known."""
        if inflight is not None:
            rows, places, host, ev, R, step_no = inflight
            ev.synchronize()
            ids = host[:R + 1].tolist()
            ops.raise_if_error_code(ids.pop(), f" during or before step {step_no}")
            for req, place, tok in zip(rows, places, ids):
                if place >= len(req.output):
                    continue                                   # cut off by an earlier end-of-sequence token
                req.output[place] = tok
                req._all[len(req.prompt) + place] = tok
                if req.stop_on_eos and req.is_eos(tok):
                    del req.output[place + 1:]
                    del req._all[len(req.prompt) + place + 1:]
                    req.finish_reason = "eos"
                    if not req.finished:
                        req.finished = True
                        if req in self.scheduler.running:
                            self.scheduler.running.remove(req)
                            self.runner.cache.free_request(req.rid)
                            self.runner.forget(req.rid)
                        elif req in self.scheduler.waiting:    # preempted meanwhile
                            self.scheduler.waiting.remove(req)
                        self._awaiting.append(req)
        ready = [r for r in self._awaiting if not r.output or r.output[-1] != self.PENDING]
        self._awaiting = [r for r in self._awaiting if r.output and r.output[-1] == self.PENDING]
        return ready

    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens, params=None,
                 stop_on_eos: bool = True, eos_token_id=None) -> List[List[int]]:
        """Runs the given prompts to the end; returns the new tokens of each."""
        n = len(prompts)
        mnt = max_new_tokens if isinstance(max_new_tokens, (list, tuple)) else [max_new_tokens] * n
        ps = params if isinstance(params, (list, tuple)) else [params] * n
        rids = [self.add_request(p, m, q, stop_on_eos=stop_on_eos, eos_token_id=eos_token_id)
                for p, m, q in zip(prompts, mnt, ps)]
        while self.has_work():
            self.step()
        out = [self.requests[r].output for r in rids]
        for r in rids:
            del self.requests[r]
        return out
