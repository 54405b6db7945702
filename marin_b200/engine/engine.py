"""The Python entry point: a model folder (or a configuration and a seed) in, tokens out.

``Engine`` loads the model the folder's config.json names, sizes the page pool, and runs
requests through the scheduler and the step function.  Option names follow ``marin-run``'s
(crates/cli/src/args.rs:352-389): ``ctx`` is the context window (prompt + reply, default
``min(2048, max_position_embeddings)`` as crates/cli/src/memory.rs:27-39), sampling options live
in :class:`SamplingParams` (``temperature`` = ``--temp``, ``top_k``, ``top_p``, ``seed``,
``max_tokens``).
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Union

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..config.base import ModelConfig, load_config
from ..kernels import ops
from ..models import Model, architecture_of
from ..parts.base import Runtime
from ..sampling.sampler import Sampler, SamplingParams
from ..weights.loader import load_tensors
from ..weights.random_init import random_tensor
from .scheduler import Planned, Request, Scheduler, StopReason
from .step import Runner, StepEntry

DEFAULT_CTX = 2048
_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           "f32": torch.float32, torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def parse_dtype(dtype) -> torch.dtype:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise ValueError(f"dtype must be bfloat16 or float32, got {dtype!r}") from None


def require_cuda(device) -> torch.device:
    device = torch.device(device)
    if device.type != "cuda" or not torch.cuda.is_available():
        raise RuntimeError("marin_b200 runs on a CUDA GPU (sm_100a) only; there is no CPU path")
    return device


def build_model(config: ModelConfig) -> Model:
    return Model(architecture_of(config).build_spec(config))


def load_model(model_dir: str, rt: Runtime) -> (ModelConfig, Model):
    """config.json chooses the model class; safetensors are read by name and checked as a whole."""
    config = load_config(model_dir)
    model = build_model(config)
    tensors = load_tensors(model_dir, model.tensor_specs(), model.spec.ignorable)
    model.load(tensors, rt)
    return config, model


def random_model(config: ModelConfig, seed: int, rt: Runtime) -> Model:
    """Random weights made directly on the device (no folder is written)."""
    model = build_model(config)
    dev = rt.device if rt.device.type == "cuda" else "cpu"
    tensors = {}
    for spec in model.tensor_specs():
        tensors[spec.name] = random_tensor(spec, seed, rt.dtype if spec.role != "norm" else torch.float32, dev)
    model.load(tensors, rt)
    return model


@dataclass
class Generation:
    req_id: Hashable
    prompt_tokens: int
    tokens: List[int]
    stop: StopReason
    preemptions: int = 0


class Engine:
    def __init__(self, model: Union[str, None] = None, *, config: Optional[ModelConfig] = None, seed: int = 0,
                 dtype="bfloat16", ctx: Optional[int] = None, page_size: int = 16, num_pages: Optional[int] = None,
                 max_batch: int = 64, token_budget: int = 2048, device="cuda:0", cuda_graphs: bool = True,
                 device_sampling: bool = True, _rt: Optional[Runtime] = None):
        """``model``: a folder with config.json and model.safetensors; or ``config`` + ``seed`` for
        random weights.  ``num_pages``: pages per cache group (default: enough for ``max_batch``
        sequences of ``ctx`` positions)."""
        self.rt = _rt or Runtime(require_cuda(device), parse_dtype(dtype))
        if model is not None:
            self.config, self.model = load_model(model, self.rt)
        elif config is not None:
            self.config, self.model = config, random_model(config, seed, self.rt)
        else:
            raise ValueError("give a model folder or a configuration")
        if self.rt.device.type == "cuda":
            from ..kernels import build
            build.build_for(self.model, self.rt.dtype, verbose=True)
        limit = self.config.max_position_embeddings
        self.ctx = min(DEFAULT_CTX, limit) if ctx is None else int(ctx)
        if self.ctx <= 0 or self.ctx > limit:
            raise ValueError(f"ctx {self.ctx} is outside 1..{limit} (max_position_embeddings)")
        pages_per_seq = -(-self.ctx // page_size)
        self.num_pages = int(num_pages) if num_pages is not None else pages_per_seq * max_batch
        needs = self.model.cache_needs()
        self.cache = CacheManager(needs, [e.cache_of for e in self.model.spec.schedule], page_size,
                                  self.num_pages, max_requests=max_batch)
        self.cache.allocate(self.rt.device, self.rt.dtype)
        self.runner = Runner(self.model, self.cache, self.rt, self.ctx)
        if cuda_graphs and self.rt.device.type == "cuda":
            sizes = [b for b in (1, 2, 4, 8, 16, 32, 64, 128, 256) if b < max_batch] + [max_batch]
            self.runner.enable_graphs(sizes)
        self.max_batch, self.token_budget = max_batch, token_budget
        #: False: logits go to the host and the host sampler (the reference's algorithm line by line) picks the token
        self.device_sampling = device_sampling and self.rt.device.type == "cuda"
        #: pack the next decode step's inputs while the GPU runs the current one (Runner.prepare_next)
        self.prepare_ahead = True
        self.scheduler = Scheduler(self.cache, max_batch, token_budget, self.ctx)
        self._requests: Dict[Hashable, Request] = {}
        self._samplers: Dict[Hashable, Sampler] = {}
        self._next_id = 0
        self._steps_unchecked = 0

    # ---- requests, one step at a time ------------------------------------------------------------------
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None,
                    req_id: Optional[Hashable] = None) -> Hashable:
        """Queues a request (token ids); returns its id.  ``step`` runs it with the others."""
        params = params or SamplingParams()
        if req_id is None:
            req_id = self._next_id
            self._next_id += 1
        request = Request(req_id, [int(t) for t in prompt], params)
        self.scheduler.add(request)
        self._requests[req_id] = request
        self._samplers[req_id] = Sampler(params)
        return req_id

    def has_work(self) -> bool:
        return self.scheduler.has_work()

    def step(self) -> List[tuple]:
        """One scheduler decision and one model step.  Returns ``[(req_id, token)]`` for the requests
        that produced a token in this step (host ints)."""
        plan = self.scheduler.schedule()
        if not plan:
            return []
        entries = [StepEntry(p.request.req_id, p.tokens, [len(p.tokens) - 1] if p.sample else []) for p in plan]
        logits = self.runner.step(entries)
        if self.prepare_ahead and all(p.sample and len(p.tokens) == 1 and len(p.request.output) + 1 < p.request.params.max_tokens
                                      for p in plan):
            # every request decodes and none reaches its length limit: most likely the next step is this one over
            # again, one position on; its inputs are packed now, while the GPU is busy, instead of after the wait below
            self.runner.prepare_next(entries)
        sampled = self._sample(plan, logits, self._samplers, self.config.vocab_size)
        self._steps_unchecked += 1
        if self._steps_unchecked >= self.CHECK_EVERY:
            self.check_device()
        return self.scheduler.update(plan, sampled)

    #: a kernel whose bounded wait gave up leaves a code on the device; it is read every so many steps (one small copy)
    #: and when a generation ends, and raises ``KernelError``
    CHECK_EVERY = 32

    def check_device(self) -> None:
        self._steps_unchecked = 0
        if self.rt.device.type == "cuda":
            ops.check_device_errors()

    def result(self, req_id: Hashable) -> Generation:
        r = self._requests[req_id]
        return Generation(r.req_id, len(r.prompt), list(r.output), r.stop, r.preemptions)

    def forget(self, req_id: Hashable) -> None:
        self.scheduler.forget(req_id)
        self._requests.pop(req_id, None)
        self._samplers.pop(req_id, None)

    # ---- generation -------------------------------------------------------------------------------------
    def generate(self, prompts: Sequence[Sequence[int]],
                 params: Union[SamplingParams, Sequence[SamplingParams], None] = None,
                 on_token=None) -> List[Generation]:
        """Generates for every prompt (token ids in, token ids out), all requests sharing the steps."""
        if params is None:
            params = SamplingParams()
        plist = list(params) if isinstance(params, (list, tuple)) else [params] * len(prompts)
        if len(plist) != len(prompts):
            raise ValueError("one SamplingParams per prompt, or one for all")
        ids = [self.add_request(prompt, p) for prompt, p in zip(prompts, plist)]
        idle = 0
        while self.scheduler.has_work():
            emitted = self.step()
            idle = 0 if emitted or self.scheduler.running else idle + 1
            if idle > 2:
                raise RuntimeError("the scheduler made no progress")
            if on_token is not None:
                for rid, token in emitted:
                    on_token(rid, token)
        self.check_device()
        out = [self.result(i) for i in ids]
        for i in ids:
            self.forget(i)
        return out

    def _sample(self, plan: Sequence[Planned], logits: torch.Tensor, samplers: Dict[Hashable, Sampler],
                vocab: int) -> Dict[Hashable, int]:
        rows = [p for p in plan if p.sample]
        if not rows:
            return {}
        out: Dict[Hashable, int] = {}
        if all(p.request.params.greedy and p.request.params.usable_vocab in (None, vocab) for p in rows):
            ids = self.runner.greedy_ids if len(rows) == len(plan) else None
            if ids is None or ids.numel() != len(rows):
                ids = torch.empty(len(rows), device=logits.device, dtype=torch.int32)
                ops.argmax(logits, vocab, ids)
            for p, token in zip(rows, ids.tolist()):
                out[p.request.req_id] = int(token)
            return out
        if self.device_sampling:
            # the kept set and the draw are computed on the device; each request's own splitmix64 stream gives its u
            n = len(rows)
            host = torch.empty(5, n, dtype=torch.float32)
            ints = host.view(torch.int32)
            for i, p in enumerate(rows):
                prm = p.request.params
                ints[0, i] = prm.usable_vocab or vocab
                host[1, i] = prm.temperature
                ints[2, i] = prm.top_k
                host[3, i] = prm.top_p
                host[4, i] = 0.0 if prm.greedy else samplers[p.request.req_id].next_unit()
            dev = host.pin_memory().to(logits.device, non_blocking=True)
            dint = dev.view(torch.int32)
            ids = torch.empty(n, device=logits.device, dtype=torch.int32)
            ops.sample(logits, dint[0], dev[1], dint[2], dev[3], dev[4], ids)
            for p, token in zip(rows, ids.tolist()):
                out[p.request.req_id] = int(token)
            return out
        host = logits.float().cpu().numpy()
        for i, p in enumerate(rows):
            usable = p.request.params.usable_vocab or vocab
            out[p.request.req_id] = samplers[p.request.req_id].sample(host[i], usable)
        return out
