"""The scheduler: which requests run in the next step, and with how many tokens.

The reference has none: a static batch runs in lock-step (src/transformers_neuronx/sampling.py:131-180)
and continuous batching is left to an external server (base.py:492-587).  The decisions here:

* admission: first come, first served, while a slot is free, the step's token budget is not spent
  and the pages for the request's first portion are free.  A request that could never fit (its
  prompt and new tokens exceed the model's length or the whole page pool) is refused when it is
  submitted.
* budget: every running request that is decoding gets its one token first; what is left of
  ``max_batch_tokens`` goes to portions of prompts, oldest request first; a portion is cut to the
  budget (and to ``max_portion`` when set), down to one token.
* pages run out: a decoding request that needs a page when none is free makes the scheduler
  preempt the most recently admitted running request: everything it holds is given back and it
  returns to the head of the waiting queue with the tokens it has so far, to be computed again
  later.  Prompt portions are simply cut to the pages that are free (or wait).
* finish: the requested number of new tokens is reached, the end-of-sequence token was
  produced and the request stops on it, or the request's ``max_time`` has passed (checked after a
  token, stopping_criteria.py:15-33); its pages and slot are given back at once, and
  ``finish_reason`` says which.

The scheduler only decides; it takes pages through the cache manager when the step is prepared.
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional

from ..cache import CacheManager


@dataclass
class SamplingParams:
    temperature: float = 0.0        # 0: greedy
    top_k: int = 0                  # 0: off
    top_p: float = 1.0              # 1: off
    seed: int = 0
    suppress_eos: bool = False      # never sample the end-of-sequence token (sampling.py:144)
    top_p_min_tokens: int = 1       # the fewest tokens top-p keeps (config.py:113, hlo.py:2349-2361)
    deterministic: bool = False     # the draw's uniform number is one half (config.py:118, hlo.py:2452-2453)


@dataclass
class Request:
    rid: Hashable
    prompt: List[int]
    max_new_tokens: int
    params: SamplingParams = field(default_factory=SamplingParams)
    stop_on_eos: bool = True
    eos_token_id: Optional[object] = None      # one id, or several (any of them ends the request)
    max_time: Optional[float] = None           # seconds after `started` beyond which no further token is asked for
    started: float = field(default_factory=time.monotonic)
    # progress
    finish_reason: Optional[str] = None        # "length", "eos" or "time" once finished
    output: List[int] = field(default_factory=list)
    computed: int = 0               # tokens of prompt+output whose keys/values are in the cache
    finished: bool = False
    preemptions: int = 0
    arrival: int = 0

    def eos_ids(self):
        e = self.eos_token_id
        if e is None:
            return ()
        return tuple(e) if isinstance(e, (list, tuple, set, frozenset)) else (e,)

    def is_eos(self, tok: int) -> bool:
        e = self.eos_token_id
        if e is None:
            return False
        return tok in e if isinstance(e, (list, tuple, set, frozenset)) else tok == e

    def __post_init__(self):
        self._all = list(self.prompt) + list(self.output)      # prompt and output as one list, kept in step
        self._dev_row = -1          # row of this request in the ids the sampling kernel wrote last

    @property
    def tokens(self) -> List[int]:
        return self._all

    @property
    def total(self) -> int:
        return len(self._all)

    def append_output(self, tok: int) -> None:
        self.output.append(tok)
        self._all.append(tok)


@dataclass
class Scheduled:
    request: Request
    start: int                      # first token (index into request.tokens) run in this step
    count: int                      # how many
    sample: bool                    # the last of them is the request's newest token: sample after it


@dataclass
class StepPlan:
    items: List[Scheduled] = field(default_factory=list)
    preempted: List[Request] = field(default_factory=list)
    admitted: List[Request] = field(default_factory=list)

    @property
    def n_tokens(self) -> int:
        return sum(i.count for i in self.items)


class Scheduler:
    def __init__(self, cache: CacheManager, max_batch_tokens: int, max_num_seqs: int, max_model_len: int,
                 max_portion: Optional[int] = None):
        self.cache = cache
        self.max_batch_tokens = int(max_batch_tokens)
        self.max_num_seqs = int(max_num_seqs)
        self.max_model_len = int(max_model_len)
        self.max_portion = max_portion
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []          # in order of admission
        self._arrivals = 0
        self.num_preemptions = 0

    # ---- submit -----------------------------------------------------------------------------------
    def add(self, req: Request) -> None:
        if not req.prompt:
            raise ValueError(f"request {req.rid!r}: empty prompt")
        if req.max_new_tokens < 1:
            raise ValueError(f"request {req.rid!r}: max_new_tokens must be at least 1 (a request that asks for "
                             "no token has nothing to run)")
        need = len(req.prompt) + req.max_new_tokens
        if need > self.max_model_len:
            raise ValueError(f"request {req.rid!r} needs {need} positions; the limit is {self.max_model_len}")
        pool = min(p.num_pages for p in self.cache.pools) if self.cache.pools else None
        # the last new token is sampled but never fed back, so need - 1 tokens are cached at most
        if pool is not None and self.cache.pages_for_tokens(max(1, need - 1)) > pool:
            raise ValueError(f"request {req.rid!r} needs {self.cache.pages_for_tokens(need - 1)} pages; "
                             f"the whole pool has {pool}")
        req.arrival = self._arrivals
        self._arrivals += 1
        self.waiting.append(req)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ---- decide the next step ------------------------------------------------------------------------
    def _preempt(self, plan: StepPlan, keep: Request) -> bool:
        """Gives back everything the most recently admitted running request holds (never `keep`
        unless it is the only one).  Returns False when nothing can be preempted."""
        victims = [r for r in self.running if r is not keep]
        if not victims:
            return False
        victim = max(victims, key=lambda r: r.arrival)
        self.running.remove(victim)
        plan.items = [i for i in plan.items if i.request is not victim]
        self.cache.free_request(victim.rid)
        victim.computed = 0
        victim.preemptions += 1
        self.num_preemptions += 1
        self.waiting.appendleft(victim)
        plan.preempted.append(victim)
        return True

    def _pages_free_after(self, plan: StepPlan) -> List[int]:
        """Free pages of every group once the items planned so far have taken theirs."""
        cached = getattr(plan, "_free", None)
        if cached is not None and cached[0] == len(plan.items) and cached[2] == self.num_preemptions:
            return list(cached[1])
        free = self.cache.free_pages()
        for it in plan.items:
            for g, n in enumerate(self.cache.pages_needed(it.request.rid, it.count)):
                free[g] -= n
        plan._free = (len(plan.items), list(free), self.num_preemptions)
        return free

    def _take(self, plan: StepPlan, item: "Scheduled") -> None:
        """Adds an item to the plan and keeps the running count of free pages current."""
        free = self._pages_free_after(plan)
        for g, n in enumerate(self.cache.pages_needed(item.request.rid, item.count)):
            free[g] -= n
        plan.items.append(item)
        plan._free = (len(plan.items), free, self.num_preemptions)

    def _fits(self, plan: StepPlan, rid, count: int) -> bool:
        free = self._pages_free_after(plan)
        return all(n <= f for n, f in zip(self.cache.pages_needed(rid, count), free))

    def _largest_fitting(self, plan: StepPlan, rid, count: int) -> int:
        """Largest portion <= count whose pages are free."""
        free = self._pages_free_after(plan)
        ps = self.cache.page_size
        have = self.cache.length(rid)
        best = count
        for g, f in enumerate(free):
            blocks_now = len(self.cache.block_table(rid, g))
            room = (blocks_now + f) * ps - have
            best = min(best, room)
        return max(0, best)

    def schedule(self) -> StepPlan:
        plan = StepPlan()
        budget = self.max_batch_tokens
        # 1. one token for every running request that is decoding
        for req in list(self.running):
            if req not in self.running:          # preempted while serving an older request
                continue
            if req.computed < req.total - 1:
                continue                         # still in its prompt: served below
            if budget <= 0:
                break
            while not self._fits(plan, req.rid, 1):
                if not self._preempt(plan, keep=req):
                    raise RuntimeError(f"request {req.rid!r} cannot get a page although it runs alone")
            if req in self.running:
                self._take(plan, Scheduled(req, req.total - 1, 1, True))
                budget -= 1
        # 2. portions of prompts of running requests, oldest first
        planned = {id(i.request) for i in plan.items}
        for req in self.running:
            if budget <= 0:
                break
            remaining = req.total - req.computed
            if id(req) in planned:
                continue
            n = min(remaining, budget, self.max_portion or remaining)
            n = self._largest_fitting(plan, req.rid, n)
            if n <= 0:
                continue
            self._take(plan, Scheduled(req, req.computed, n, req.computed + n == req.total))
            budget -= n
        # 3. admit waiting requests, first come first served
        while self.waiting and budget > 0 and len(self.running) < self.max_num_seqs and not plan.preempted:
            req = self.waiting[0]
            if self.cache.slots.num_free <= 0:
                break
            remaining = req.total - req.computed
            n = min(remaining, budget, self.max_portion or remaining)
            # pages for the first portion must be free now
            free = self._pages_free_after(plan)
            need = self.cache.pages_for_tokens(n)
            if any(need > f for f in free):
                fit = min(free) * self.cache.page_size if free else n
                n = min(n, fit)
                if n <= 0:
                    break
            self.waiting.popleft()
            self.cache.add_request(req.rid)
            self.running.append(req)
            plan.admitted.append(req)
            self._take(plan, Scheduled(req, req.computed, n, req.computed + n == req.total))
            budget -= n
        if not plan.items and self.has_work():
            raise RuntimeError("the scheduler found nothing to run although requests are pending "
                               "(no page is free and nothing can be preempted)")
        return plan

    # ---- after the step ------------------------------------------------------------------------------
    def commit(self, plan: StepPlan, sampled: Dict[Hashable, int], now: Optional[float] = None) -> List[Request]:
        """Records the step's progress and the sampled tokens; returns the requests that finished
        (their pages and slots are already given back).  A request with `max_time` ends with the
        first token sampled after that many seconds, as the reference's MaxTimeCriteria ends a
        generation (src/transformers_neuronx/stopping_criteria.py:15-33): the check comes after a
        token, so at least one is produced."""
        done = []
        now = time.monotonic() if now is None else now
        for it in plan.items:
            req = it.request
            req.computed = it.start + it.count
            if not it.sample:
                continue
            tok = int(sampled[req.rid])
            req.append_output(tok)
            hit_eos = req.stop_on_eos and req.is_eos(tok)
            timed_out = req.max_time is not None and now - req.started > req.max_time
            if len(req.output) >= req.max_new_tokens or hit_eos or timed_out:
                req.finished = True
                req.finish_reason = "eos" if hit_eos else ("length" if len(req.output) >= req.max_new_tokens else "time")
                self.running.remove(req)
                self.cache.free_request(req.rid)
                done.append(req)
        return done
