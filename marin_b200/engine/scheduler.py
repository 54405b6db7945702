"""The scheduler: which requests run in the next step, and with how many tokens.

Policy (host bookkeeping only).  Each step has a token budget.  Requests that are decoding
come first with one token each; what is left of the budget goes to prompt portions, running
requests before newly admitted ones, first come first served; a portion is
``min(rest of the prompt, budget left)`` and may be as small as one token.  A request is
admitted while fewer than ``max_batch`` run and its first portion's pages are free.

When pages run out for a request that is already running, the most recently admitted running
request is preempted: its pages go back, it returns to the front of the waiting queue and later
recomputes its prompt plus the tokens it had generated.  A request that does not fit the pool
even when it runs alone ends with ``StopReason.OUT_OF_PAGES``.  (The reference never runs two
Qwen3 requests at once and makes a starved request wait for another to finish,
crates/cli/src/server/sched.rs:30-51,150-162; its stop reasons are
crates/runtime/src/generate.rs:38-44.)
"""
from __future__ import annotations

import enum
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional, Sequence

from ..cache.manager import CacheManager
from ..sampling.sampler import SamplingParams


class StopReason(enum.Enum):
    MAX_TOKENS = "max_tokens"
    END_OF_TEXT = "end_of_text"
    CONTEXT_FULL = "context_full"
    CANCELLED = "cancelled"
    OUT_OF_PAGES = "out_of_pages"


class RequestError(ValueError):
    """A request that cannot be admitted at all: empty prompt, prompt longer than the context."""


@dataclass
class Request:
    req_id: Hashable
    prompt: List[int]
    params: SamplingParams
    output: List[int] = field(default_factory=list)
    computed: int = 0               # tokens of prompt+output whose keys/values are in the cache
    stop: Optional[StopReason] = None
    preemptions: int = 0
    admitted_at: int = -1

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output

    @property
    def num_tokens(self) -> int:
        return len(self.prompt) + len(self.output)

    def tokens_from(self, start: int, count: int) -> List[int]:
        """``tokens[start:start + count]`` without building the whole list."""
        p = len(self.prompt)
        end = start + count
        if end <= p:
            return self.prompt[start:end]
        if start >= p:
            return self.output[start - p:end - p]
        return self.prompt[start:] + self.output[:end - p]

    @property
    def finished(self) -> bool:
        return self.stop is not None


@dataclass
class Planned:
    """One request's share of the next step."""

    request: Request
    tokens: List[int]
    sample: bool                    # the portion ends the known tokens: sample the next one from its last logits
    missing: List[int] = field(default_factory=list)   # pages per cache group this portion still needs


class Scheduler:
    def __init__(self, cache: CacheManager, max_batch: int, token_budget: int, max_seq_len: int):
        if token_budget < 1 or max_batch < 1:
            raise ValueError("token_budget and max_batch must be at least 1")
        self.cache, self.max_batch, self.token_budget, self.max_seq_len = cache, max_batch, token_budget, max_seq_len
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.finished: List[Request] = []
        self._clock = 0

    # ---- admission ------------------------------------------------------------------------------------
    def add(self, request: Request) -> None:
        request.params.validate()
        if not request.prompt:
            raise RequestError("the prompt is empty")
        if len(request.prompt) > self.max_seq_len:
            raise RequestError(f"the prompt has {len(request.prompt)} tokens, the context holds {self.max_seq_len}")
        if request.params.max_tokens == 0:
            request.stop = StopReason.MAX_TOKENS
            self.finished.append(request)
            return
        self.waiting.append(request)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def cancel(self, req_id: Hashable) -> None:
        for r in list(self.running):
            if r.req_id == req_id:
                self._finish(r, StopReason.CANCELLED)
        for r in list(self.waiting):
            if r.req_id == req_id:
                self.waiting.remove(r)
                r.stop = StopReason.CANCELLED
                self.finished.append(r)

    # ---- one step's plan --------------------------------------------------------------------------------
    def _pages_fit(self, planned: Sequence[Planned], extra: Optional[Planned] = None) -> bool:
        """Whether the pages the planned portions (and ``extra``) need are free, in every group."""
        need = self._need_of(planned)
        if extra is not None:
            for g, n in enumerate(self.cache.pages_missing(extra.request.req_id, extra.request.computed + len(extra.tokens))):
                need[g] += n
        return all(n <= free for n, free in zip(need, self.cache.free_pages()))

    def _need_of(self, planned: Sequence[Planned]) -> List[int]:
        need = [0] * len(self.cache.groups)
        for p in planned:
            for g, n in enumerate(p.missing):
                need[g] += n
        return need

    def _portion(self, request: Request, budget: int) -> Planned:
        rest = request.num_tokens - request.computed
        count = min(rest, budget)
        return Planned(request, request.tokens_from(request.computed, count), sample=rest <= budget)

    def _preempt(self, victim: Request) -> None:
        self.cache.release(victim.req_id)
        self.running.remove(victim)
        victim.computed = 0
        victim.preemptions += 1
        self.waiting.appendleft(victim)

    def _finish(self, request: Request, reason: StopReason) -> None:
        request.stop = reason
        if request in self.running:
            self.running.remove(request)
            self.cache.release(request.req_id)
        self.finished.append(request)

    def _plan_without_contest(self) -> Optional[List[Planned]]:
        """The common step: nobody can be admitted (no one waits, or every place is taken) and the running requests'
        portions all find their pages.  One question to the cache instead of one per request; None if it does not
        apply, and the careful path below decides."""
        if not self.running or (self.waiting and len(self.running) < self.max_batch):
            return None
        budget = self.token_budget
        plan: List[Planned] = []
        for request in sorted(self.running, key=lambda r: r.admitted_at):
            if budget == 0:
                break
            portion = self._portion(request, budget)
            plan.append(portion)
            budget -= len(portion.tokens)
        if not self.cache.can_reserve([(p.request.req_id, p.request.computed + len(p.tokens)) for p in plan]):
            return None
        return plan

    def schedule(self) -> List[Planned]:
        plan = self._plan_without_contest()
        if plan is not None:
            return plan
        budget = self.token_budget
        plan = []
        # 1. running requests, oldest first: decodes take one token, prompts a portion
        for request in sorted(self.running, key=lambda r: r.admitted_at):
            if request not in self.running:      # preempted while making room for an older one
                continue
            if budget == 0:
                break
            portion = self._portion(request, budget)
            while not self._pages_fit(plan, portion):
                victims = [r for r in self.running if r is not request and all(p.request is not r for p in plan)]
                if not victims:
                    break
                self._preempt(max(victims, key=lambda r: r.admitted_at))
            if not self._pages_fit(plan, portion):
                if not plan and len(self.running) == 1:
                    self._finish(request, StopReason.OUT_OF_PAGES)
                continue
            portion.missing = self.cache.pages_missing(request.req_id, request.computed + len(portion.tokens))
            plan.append(portion)
            budget -= len(portion.tokens)
        # 2. admit waiting requests while there is room
        while self.waiting and budget > 0 and len(self.running) < self.max_batch:
            request = self.waiting[0]
            portion = self._portion(request, budget)
            self.cache.admit(request.req_id)
            if not self._pages_fit(plan, portion):
                self.cache.release(request.req_id)
                if not self.running:
                    # alone and still too large for the pool: it can never run
                    self.waiting.popleft()
                    request.stop = StopReason.OUT_OF_PAGES
                    self.finished.append(request)
                    continue
                break
            self.waiting.popleft()
            self._clock += 1
            request.admitted_at = self._clock
            self.running.append(request)
            portion.missing = self.cache.pages_missing(request.req_id, request.computed + len(portion.tokens))
            plan.append(portion)
            budget -= len(portion.tokens)
        return plan

    # ---- after the step ----------------------------------------------------------------------------------
    def update(self, plan: Sequence[Planned], sampled: Dict[Hashable, int]) -> List[tuple]:
        """Records what ran and the tokens sampled for the requests whose portion ended their known
        tokens; returns ``[(req_id, token)]`` for the tokens that were emitted (a stop token is not)."""
        emitted: List[tuple] = []
        for p in plan:
            r = p.request
            r.computed += len(p.tokens)
            if not p.sample:
                continue
            token = sampled[r.req_id]
            if token in r.params.stop_tokens:
                self._finish(r, StopReason.END_OF_TEXT)      # the stop token is not emitted
                continue
            r.output.append(token)
            emitted.append((r.req_id, token))
            if len(r.output) >= r.params.max_tokens:
                self._finish(r, StopReason.MAX_TOKENS)
            elif r.computed >= self.max_seq_len:
                # the cache is full: the token just emitted cannot be fed (generate.rs:217-221)
                self._finish(r, StopReason.CONTEXT_FULL)
        return emitted
