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
from ..parts.spec import TensorSpec
from ..sampling.sampler import Sampler, SamplerError, SamplingParams
from ..weights.loader import load_tensors
from ..weights.random_init import random_tensor
from .memory import Footprint, OutOfDeviceMemory, plan as plan_memory
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


def load_model(model_dir: str, rt: Runtime, extra_tensors: str = "error") -> (ModelConfig, Model):
    """config.json chooses the model class; safetensors are read by name and checked as a whole."""
    config = load_config(model_dir)
    model = build_model(config)
    tensors = load_tensors(model_dir, model.tensor_specs(), model.spec.ignorable, extra_tensors)
    model.load(tensors, rt)
    return config, model


def load_random(model: Model, seed: int, rt: Runtime) -> None:
    """Random weights made directly on the device (no folder is written)."""
    dev = rt.device if rt.device.type == "cuda" else "cpu"

    class Drawn(dict):
        """The tensors by name, each drawn when a part takes it: at no time are all of them there twice (once as drawn,
        once as the parts keep them, fused and laid out for the kernels)."""

        def pop(self, name, *default):
            spec = super().pop(name, *default)
            if not isinstance(spec, TensorSpec):
                return spec
            return random_tensor(spec, seed, rt.dtype if spec.role != "norm" else torch.float32, dev)

    model.load(Drawn({spec.name: spec for spec in model.tensor_specs()}), rt)
    if rt.device.type == "cuda":
        torch.cuda.empty_cache()


def random_model(config: ModelConfig, seed: int, rt: Runtime) -> Model:
    model = build_model(config)
    load_random(model, seed, rt)
    return model


class GenerationError(RuntimeError):
    """A request whose logits were not finite: it has ended with ``StopReason.NON_FINITE_LOGITS`` (its pages are free
    again); ``req_id`` names it."""

    def __init__(self, req_id, message: str):
        super().__init__(message)
        self.req_id = req_id


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
                 device_sampling: bool = True, extra_tensors: str = "error", _rt: Optional[Runtime] = None,
                 _free_bytes: Optional[int] = None):
        """``model``: a folder with config.json and model.safetensors; or ``config`` + ``seed`` for
        random weights.  ``num_pages``: pages per cache group (default: enough for ``max_batch``
        sequences of ``ctx`` positions, or as many as the device has room for if that is fewer).
        ``extra_tensors``: ``"error"`` lists tensors of the folder that the model does not know in the one
        error with everything else that is wrong; ``"warn"`` loads without them and keeps their names in
        ``self.ignored_tensors`` (the reference ignores extras: crates/model/src/qwen3/weight_bytes.rs:9-10).

        Before anything is loaded the weights, the page pool and the working memory are added up from the
        parts' own figures and compared with the device's free memory (``self.footprint``,
        ``engine/memory.py``); what does not fit raises ``OutOfDeviceMemory`` with the numbers."""
        self.rt = _rt or Runtime(require_cuda(device), parse_dtype(dtype))
        if model is not None:
            self.config = load_config(model)
        elif config is not None:
            self.config = config
        else:
            raise ValueError("give a model folder or a configuration")
        self.model = build_model(self.config)
        limit = self.config.max_position_embeddings
        self.ctx = min(DEFAULT_CTX, limit) if ctx is None else int(ctx)
        if self.ctx <= 0 or self.ctx > limit:
            raise ValueError(f"ctx {self.ctx} is outside 1..{limit} (max_position_embeddings)")
        on_gpu = self.rt.device.type == "cuda"
        graph_sizes = []
        if cuda_graphs and on_gpu and self.model.capturable():
            graph_sizes = [b for b in (1, 2, 4, 8, 16, 32, 64, 128, 256) if b < max_batch] + [max_batch]
        free = _free_bytes
        if free is None and on_gpu:
            free = int(torch.cuda.mem_get_info(self.rt.device)[0])
        self.footprint = plan_memory(self.model, self.rt.dtype, page_size, self.ctx, max_batch, token_budget, num_pages,
                                     graph_sizes, free)
        self.num_pages = self.footprint.num_pages
        # The pool first, while the device is still empty: what loading holds for a moment (a float32 draw of a random
        # table, staging copies) then fits in the room planned for working memory, and no fragment of it is left
        # standing between the weights when the largest allocation of all is made.
        needs = self.model.cache_needs()
        self.cache = CacheManager(needs, [e.cache_of for e in self.model.spec.schedule], page_size,
                                  self.num_pages, max_requests=max_batch)
        self.cache.allocate(self.rt.device, self.rt.dtype)
        self.ignored_tensors: List[str] = []
        if model is not None:
            tensors = load_tensors(model, self.model.tensor_specs(), self.model.spec.ignorable, extra_tensors, self.ignored_tensors)
            self.model.load(tensors, self.rt)
            del tensors
        else:
            load_random(self.model, seed, self.rt)
        if on_gpu:
            from ..kernels import build
            build.build_for(self.model, self.rt.dtype, verbose=True)
            torch.cuda.empty_cache()
        self.runner = Runner(self.model, self.cache, self.rt, self.ctx)
        if graph_sizes:
            self.runner.enable_graphs(graph_sizes)
        self.max_batch, self.token_budget = max_batch, token_budget
        #: False: logits go to the host and the host sampler (the reference's algorithm line by line) picks the token
        self.device_sampling = device_sampling and on_gpu
        #: pack the next decode step's inputs while the GPU runs the current one (Runner.prepare_next)
        self.prepare_ahead = True
        #: launch the next decode step before the current one's tokens have reached the host (see ``step``)
        self.run_ahead = True
        self._ahead: Optional[dict] = None
        self.scheduler = Scheduler(self.cache, max_batch, token_budget, self.ctx)
        self._requests: Dict[Hashable, Request] = {}
        self._samplers: Dict[Hashable, Sampler] = {}
        self._next_id = 0

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
        that produced a token in this step (host ints).

        Every step learns, with the sampled ids it reads anyway, whether a kernel's bounded wait gave up
        (``KernelError``).  A request whose logits are NaN or infinite is ended, the others' tokens are
        recorded, and ``GenerationError`` is raised naming it (the reference fails such a pass:
        crates/model/src/qwen3/model.rs:128, crates/sampler/src/lib.rs:135-137).

        **Running ahead.**  While every request decodes greedily and nobody waits to be admitted, the step after
        the current one is launched before the current one's tokens have reached the host: its token ids are fed on
        the device (``Runner.launch_ahead``).  The GPU then goes from step to step without waiting for the host, and
        a call of ``step`` returns the tokens of the older of the two steps in flight.  A request that turns out to
        have ended (a stop token) has computed one token for nothing; its row of the step that ran ahead is dropped."""
        ahead, self._ahead = self._ahead, None
        if ahead is not None:
            plan = self.scheduler.schedule_running()          # the step that is running already: who of it goes on
            if not plan:
                return self.step()                            # everybody ended: nothing of it counts
            self.runner.commit_ahead(ahead, {p.request.req_id for p in plan})
            entries = [StepEntry(p.request.req_id, p.tokens, [0]) for p in plan]
            rows = {rid: i for i, rid in enumerate(ahead["req_ids"])}
            if [p.request.req_id for p in plan] == list(ahead["req_ids"]) and self._may_run_ahead(plan):
                self._ahead = self.runner.launch_ahead(entries)
            if self._ahead is not None:
                ids = self.runner.read_ahead(self._ahead)     # the ids of the step that ran ahead; the next one runs meanwhile
            else:
                ids = self.runner.read_graph_ids(ahead["rows"], ahead["which"])
            sampled = {p.request.req_id: int(ids[rows[p.request.req_id]]) for p in plan}
            return self._record(plan, sampled)
        plan = self.scheduler.schedule()
        if not plan:
            return []
        entries = [StepEntry(p.request.req_id, p.tokens, [len(p.tokens) - 1] if p.sample else []) for p in plan]
        logits = self.runner.step(entries)
        decoding = all(p.sample and len(p.tokens) == 1 for p in plan)
        if decoding and self.run_ahead and self.runner.greedy_ids is not None and self._may_run_ahead(plan):
            self._ahead = self.runner.launch_ahead(entries)
            if self._ahead is not None:
                ids = self.runner.read_ahead(self._ahead)
                return self._record(plan, {p.request.req_id: int(t) for p, t in zip(plan, ids)})
        if self.prepare_ahead and decoding and all(len(p.request.output) + 1 < p.request.params.max_tokens for p in plan):
            # every request decodes and none reaches its length limit: most likely the next step is this one over
            # again, one position on; its inputs are packed now, while the GPU is busy, instead of after the wait below
            self.runner.prepare_next(entries)
        sampled = self._sample(plan, logits, self._samplers, self.config.vocab_size)
        return self._record(plan, sampled)

    def _may_run_ahead(self, plan: Sequence[Planned]) -> bool:
        """Whether the step after the one that runs may be launched before its tokens are known: all requests decode
        greedily over the whole vocabulary, each has room for the token being made and one more, and nobody waits to
        be admitted (a newcomer would have to wait a step longer)."""
        if not (self.run_ahead and self.device_sampling) or self.scheduler.has_waiting():
            return False
        vocab = self.config.vocab_size
        for p in plan:
            prm = p.request.params
            if not (prm.greedy and prm.usable_vocab in (None, vocab)) or len(p.request.output) + 2 > prm.max_tokens:
                return False
        return True

    def _record(self, plan: Sequence[Planned], sampled: Dict[Hashable, int]) -> List[tuple]:
        emitted = self.scheduler.update(plan, sampled)          # a negative id ends its request (NON_FINITE_LOGITS)
        bad = [rid for rid, token in sampled.items() if token < 0]
        if bad:
            raise GenerationError(bad[0], f"request {bad[0]!r}: the logits hold a value that is not finite"
                                  + (f" (and those of {len(bad) - 1} more requests)" if len(bad) > 1 else "")
                                  + "; ended, the other requests' tokens of this step are recorded")
        return emitted

    def check_device(self) -> None:
        """Raises ``KernelError`` if a kernel's bounded wait gave up since the last look (one small copy, one wait).
        ``step`` learns of it by itself when it samples; this is for callers that drive ``runner`` directly."""
        if self.runner.scratch is not None:
            self.runner.scratch.check()

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
            try:
                emitted = self.step()
            except Exception:
                for i in ids:                                  # a failed generation leaves nothing behind
                    self.scheduler.cancel(i)
                    self.forget(i)
                raise
            idle = 0 if emitted or self.scheduler.running else idle + 1
            if idle > 2:
                raise RuntimeError("the scheduler made no progress")
            if on_token is not None:
                for rid, token in emitted:
                    on_token(rid, token)
        out = [self.result(i) for i in ids]
        for i in ids:
            self.forget(i)
        return out

    def _sample(self, plan: Sequence[Planned], logits: torch.Tensor, samplers: Dict[Hashable, Sampler],
                vocab: int) -> Dict[Hashable, int]:
        """The next token of every request of the plan that wants one; -1 where the logits were not finite."""
        rows = [p for p in plan if p.sample]
        if not rows:
            return {}
        out: Dict[Hashable, int] = {}
        scratch = self.runner.scratch
        n = len(rows)
        if self.device_sampling and all(p.request.params.greedy and p.request.params.usable_vocab in (None, vocab) for p in rows):
            if self.runner.greedy_ids is not None and len(rows) == len(plan) and self.runner.greedy_ids.numel() == n:
                ids = self.runner.read_graph_ids(n)           # a replayed graph has found the largest logits already
            else:
                with ops.using(scratch):
                    ops.argmax(logits, vocab, scratch.ids(n))
                ids = scratch.read(n)
            for p, token in zip(rows, ids):
                out[p.request.req_id] = int(token)
            return out
        if self.device_sampling:
            # the kept set and the draw are computed on the device; each request's own splitmix64 stream gives its u
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
            with ops.using(scratch):
                ops.sample(logits, dint[0], dev[1], dint[2], dev[3], dev[4], scratch.ids(n))
            for p, token in zip(rows, scratch.read(n)):
                out[p.request.req_id] = int(token)
            return out
        host = logits.float().cpu().numpy()
        if scratch is not None:
            scratch.check()
        for i, p in enumerate(rows):
            usable = p.request.params.usable_vocab or vocab
            try:
                out[p.request.req_id] = samplers[p.request.req_id].sample(host[i], usable)
            except SamplerError as err:
                if "NaN" not in str(err):
                    raise
                out[p.request.req_id] = -1
        return out
