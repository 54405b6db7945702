"""The scheduler: which requests run in the next step, and with how many tokens.  The decisions are made in C++
(``csrc/host/scheduler.cpp``); this module holds its Python face.

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

import ctypes
import enum
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np

from ..cache.manager import CacheManager
from ..sampling.sampler import SamplingParams


class StopReason(enum.Enum):
    MAX_TOKENS = "max_tokens"
    END_OF_TEXT = "end_of_text"
    CONTEXT_FULL = "context_full"
    CANCELLED = "cancelled"
    OUT_OF_PAGES = "out_of_pages"
    NON_FINITE_LOGITS = "non_finite_logits"      # the model produced NaN or infinity for this request: it was ended


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
    """The handle of the C++ scheduler (``csrc/host/scheduler.cpp``), which holds the queues, the requests' tokens
    and counters and decides every step; the ``Request`` objects here mirror what it says about them."""

    _STOPS = [StopReason.MAX_TOKENS, StopReason.END_OF_TEXT, StopReason.CONTEXT_FULL, StopReason.CANCELLED, StopReason.OUT_OF_PAGES,
              StopReason.NON_FINITE_LOGITS]

    def __init__(self, cache: CacheManager, max_batch: int, token_budget: int, max_seq_len: int):
        if token_budget < 1 or max_batch < 1:
            raise ValueError("token_budget and max_batch must be at least 1")
        self.cache, self.max_batch, self.token_budget, self.max_seq_len = cache, max_batch, token_budget, max_seq_len
        self._lib = cache._lib
        self._core = self._lib.mbs_create(cache._core(), int(max_batch), int(token_budget), int(max_seq_len))
        if not self._core:
            raise ValueError("the scheduler core refused these sizes")
        self._by_sid: Dict[int, Request] = {}
        self._sid_of: Dict[Hashable, int] = {}
        self._in_cache: Dict[Hashable, int] = {}                  # requests this scheduler has put into cache.requests
        self._items = np.zeros((max_batch + 1, 6), np.int64)
        self._tokens = np.zeros(token_budget, np.int32)
        self._emitted_ids = np.zeros(max_batch + 1, np.int64)
        self._emitted_tokens = np.zeros(max_batch + 1, np.int32)

    def __del__(self):
        core, self._core = getattr(self, "_core", None), None
        if core:
            self._lib.mbs_destroy(core)

    # ---- what the core says about the requests -----------------------------------------------------------
    def _refresh(self, requests: Sequence[Request]) -> None:
        """Brings the mirrors of these requests up to date, and ``cache.requests`` with who is running."""
        requests = [r for r in requests if r.req_id in self._sid_of]
        if not requests:
            return
        ids = np.fromiter((self._sid_of[r.req_id] for r in requests), np.int64, len(requests))
        out = np.zeros((len(requests), 8), np.int64)
        if self._lib.mbs_states(self._core, len(requests), ids.ctypes.data, out.ctypes.data) != 0:
            raise KeyError("the scheduler core does not know one of its requests")
        for r, (computed, n_out, stop, preemptions, admitted_at, where, handle, slot) in zip(requests, out.tolist()):
            r.computed, r.preemptions, r.admitted_at = computed, preemptions, admitted_at
            r.stop = None if stop < 0 else self._STOPS[stop]
            if n_out != len(r.output):
                buf = np.zeros(max(n_out, 1), np.int32)
                self._lib.mbs_output(self._core, self._sid_of[r.req_id], buf.ctypes.data, n_out)
                r.output[:] = buf[:n_out].tolist()
            known = self._in_cache.get(r.req_id)
            if where == 1 and known != handle:
                self._enter_cache(r.req_id, handle, slot)
            elif where != 1 and known is not None:
                self.cache.requests.pop(r.req_id, None)
                del self._in_cache[r.req_id]

    def _enter_cache(self, req_id: Hashable, handle: int, slot: int) -> None:
        from ..cache.manager import RequestCache

        self.cache.requests[req_id] = RequestCache(self.cache, handle, slot)
        self._in_cache[req_id] = handle
        for tensor in self.cache.state.values():
            tensor[slot].zero_()

    def _listed(self, which: int) -> List[Request]:
        n = self._lib.mbs_list(self._core, which, None, 0)
        buf = np.zeros(max(n, 1), np.int64)
        self._lib.mbs_list(self._core, which, buf.ctypes.data, n)
        return [self._by_sid[i] for i in buf[:n].tolist() if i in self._by_sid]

    @property
    def waiting(self) -> List[Request]:
        return self._listed(0)

    @property
    def running(self) -> List[Request]:
        return self._listed(1)

    @property
    def finished(self) -> List[Request]:
        return self._listed(2)

    # ---- admission ------------------------------------------------------------------------------------
    def add(self, request: Request) -> None:
        request.params.validate()
        prompt = np.asarray(request.prompt, np.int32).reshape(-1)
        stops = np.asarray(list(request.params.stop_tokens), np.int32).reshape(-1)
        sid = ctypes.c_int64()
        rc = self._lib.mbs_add(self._core, prompt.ctypes.data, int(prompt.size), int(request.params.max_tokens),
                               stops.ctypes.data, int(stops.size), ctypes.byref(sid))
        if rc == 20:
            raise RequestError("the prompt is empty")
        if rc == 21:
            raise RequestError(f"the prompt has {len(request.prompt)} tokens, the context holds {self.max_seq_len}")
        if rc != 0:
            raise RequestError(f"the scheduler refused the request (code {rc})")
        self._by_sid[sid.value] = request
        self._sid_of[request.req_id] = sid.value
        self._refresh([request])

    def has_work(self) -> bool:
        return self._lib.mbs_has_work(self._core) == 1

    def cancel(self, req_id: Hashable) -> None:
        sid = self._sid_of.get(req_id)
        if sid is None:
            return
        self._lib.mbs_cancel(self._core, sid)
        self._refresh([self._by_sid[sid]])

    def forget(self, req_id: Hashable) -> None:
        """Drops a finished request from the scheduler's memory."""
        sid = self._sid_of.get(req_id)
        if sid is not None and self._lib.mbs_forget(self._core, sid) == 0:
            del self._sid_of[req_id]
            del self._by_sid[sid]

    # ---- one step's plan --------------------------------------------------------------------------------
    def schedule(self) -> List[Planned]:
        changed = ctypes.c_int(0)
        n = self._lib.mbs_schedule(self._core, self._items.ctypes.data, len(self._items), self._tokens.ctypes.data,
                                   len(self._tokens), ctypes.byref(changed))
        if n < 0:
            raise RuntimeError(f"the scheduler core failed (code {n})")
        if changed.value:
            self._refresh(list(self._by_sid.values()))
        plan: List[Planned] = []
        at = 0
        flat = self._tokens[: int(self._items[:n, 2].sum())].tolist()
        for sid, start, count, sample, handle, slot in self._items[:n].tolist():
            request = self._by_sid[sid]
            request.computed = start
            plan.append(Planned(request, flat[at:at + count], bool(sample)))
            at += count
        return plan

    def schedule_running(self) -> List[Planned]:
        """The plan of a step that is already running: the engine launched it before it had read the tokens of the step
        before, supposing that the same requests decode on (``Engine.step``).  Requests that ended or were cancelled
        since are not in it; nobody is admitted or preempted."""
        n = self._lib.mbs_schedule_running(self._core, self._items.ctypes.data, len(self._items), self._tokens.ctypes.data, len(self._tokens))
        if n < 0:
            raise RuntimeError(f"the step that was launched ahead does not fit the scheduler's state (code {n})")
        plan: List[Planned] = []
        flat = self._tokens[:n].tolist()
        for (sid, start, count, sample, handle, slot), token in zip(self._items[:n].tolist(), flat):
            request = self._by_sid[sid]
            request.computed = start
            plan.append(Planned(request, [token], bool(sample)))
        return plan

    def has_waiting(self) -> bool:
        return self._lib.mbs_list(self._core, 0, None, 0) > 0

    # ---- after the step ----------------------------------------------------------------------------------
    def update(self, plan: Sequence[Planned], sampled: Dict[Hashable, int]) -> List[tuple]:
        """Records what ran and the tokens sampled for the requests whose portion ended their known
        tokens; returns ``[(req_id, token)]`` for the tokens that were emitted (a stop token is not).  A negative token says the request's logits were not finite:
        it ends with ``StopReason.NON_FINITE_LOGITS``."""
        tokens = np.asarray([sampled[p.request.req_id] for p in plan if p.sample], np.int32).reshape(-1)
        changed = ctypes.c_int(0)
        n = self._lib.mbs_update(self._core, tokens.ctypes.data, int(tokens.size), self._emitted_ids.ctypes.data,
                                 self._emitted_tokens.ctypes.data, ctypes.byref(changed))
        if n < 0:
            raise RuntimeError(f"the scheduler core failed (code {n})")
        emitted: List[tuple] = []
        for sid, token in zip(self._emitted_ids[:n].tolist(), self._emitted_tokens[:n].tolist()):
            request = self._by_sid[sid]
            request.output.append(token)
            emitted.append((request.req_id, token))
        for p in plan:
            p.request.computed += len(p.tokens)
        if changed.value:
            self._refresh([p.request for p in plan])
        return emitted
