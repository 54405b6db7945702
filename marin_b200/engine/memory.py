"""Memory planning: will the weights, the cache and the working memory fit the GPU, decided before anything is loaded.

The reference checks its start-up bytes (weights + first cache slab) and its whole window against free
memory with 512 MiB of slack for activations and kernel code (crates/model/src/qwen3/fit.rs:2-22), counting
the bytes it really loads (crates/model/src/qwen3/weight_bytes.rs:11-69) and reporting a footprint
(crates/cli/src/memory.rs:27-59).  Here the whole page pool is allocated at start-up, so one comparison
decides: weights + pool + working memory + slack against what the device has free.  Every figure comes from
the parts' own answers (``Part.weight_bytes``, the cache needs' ``bytes_per_token``), so another architecture
is planned without a change here.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch

#: kept free for kernel code, the CUDA context's own allocations and fragmentation (the reference's figure) ...
SLACK_BYTES = 512 * 1024 * 1024
#: ... and on top of it this fraction of what is free: an allocator that hands out memory in segments of megabytes
#: leaves more unusable the more it manages (measured on a 180 GB device filled to the brim: 0.7 GiB held in part-used
#: segments and as much again in kernel modules loaded after the plan was made)
SLACK_FRACTION = 1.0 / 64


class OutOfDeviceMemory(RuntimeError):
    """The model, its cache and its working memory do not fit the device."""


@dataclass
class Footprint:
    weights: int            # bytes of the tensors as the device keeps them
    page: int               # bytes of one page over all cache groups
    num_pages: int          # pages per group
    state: int              # fixed-size per-request state
    workspace: int          # activations of the largest step, logits, graphs' buffers, kernel scratch
    slack: int
    free: Optional[int]     # what the device had free when the plan was made (None: not asked)
    pages_wanted: int       # pages that max_batch sequences of ctx positions would need
    pages_that_fit: Optional[int]

    @property
    def cache(self) -> int:
        return self.page * self.num_pages

    @property
    def needed(self) -> int:
        return self.weights + self.cache + self.state + self.workspace + self.slack

    def lines(self) -> str:
        gib = 1 << 30
        free = "unknown" if self.free is None else f"{self.free / gib:.2f} GiB"
        return (f"weights {self.weights / gib:.2f} GiB + cache {self.cache / gib:.2f} GiB ({self.num_pages} pages of "
                f"{self.page / 1024:.0f} KiB) + per-request state {self.state / gib:.3f} GiB + working memory "
                f"{self.workspace / gib:.2f} GiB + slack {self.slack / gib:.2f} GiB = {self.needed / gib:.2f} GiB; free {free}")


def workspace_bytes(model, dtype: torch.dtype, token_budget: int, max_batch: int, graph_sizes: Sequence[int]) -> int:
    """An upper estimate of what steps allocate besides weights and cache: per token of the largest step the
    float32 residual stream and the widest activations of a layer (each part's matrices name their widths), the
    float32 logits of ``max_batch`` rows, the same again for every captured batch size, and the kernels' scratch."""
    from ..parts.base import element_size

    size = element_size(dtype)
    widest = 0
    for part in model.parts():
        width = sum(int(s.shape[0]) for s in part.tensor_specs() if s.role == "matrix" and len(s.shape) == 2)
        widest = max(widest, width)
    hidden, vocab = model.spec.hidden_size, model.spec.vocab_size
    per_token = 4 * hidden * 2 + size * (2 * hidden + 2 * widest)
    logits = 4 * vocab * max_batch
    graphs = sum(b * (4 * vocab + per_token) for b in graph_sizes)
    scratch = 96 << 20
    return token_budget * per_token + logits + graphs + scratch


def plan(model, dtype: torch.dtype, page_size: int, ctx: int, max_batch: int, token_budget: int,
         num_pages: Optional[int], graph_sizes: Sequence[int] = (), free_bytes: Optional[int] = None,
         slack: Optional[int] = None) -> Footprint:
    """The footprint of an engine with these options.  ``num_pages`` None: as many pages as ``max_batch`` sequences
    of ``ctx`` positions need, or as many as fit if that is fewer (at least one sequence's worth, else an error).
    Raises ``OutOfDeviceMemory`` naming weights, cache, working memory and the largest pool that would fit."""
    from ..cache.manager import CacheManager

    if slack is None:
        slack = SLACK_BYTES + (int(free_bytes * SLACK_FRACTION) if free_bytes is not None else 0)
    needs = model.cache_needs()
    probe = CacheManager(needs, [e.cache_of for e in model.spec.schedule], page_size, 1, max_batch)
    page, state = probe.bytes_per_page(dtype), probe.state_bytes()
    per_seq = -(-ctx // page_size)
    wanted = per_seq * max_batch
    weights = model.weight_bytes(dtype)
    work = workspace_bytes(model, dtype, token_budget, max_batch, graph_sizes)
    fit = None
    if free_bytes is not None:
        left = free_bytes - weights - state - work - slack
        fit = max(0, left // page) if page > 0 else wanted
    chosen = num_pages if num_pages is not None else (wanted if fit is None else min(wanted, fit))
    fp = Footprint(weights, page, int(chosen), state, work, slack, free_bytes, wanted, fit)
    if free_bytes is not None and page > 0:
        if num_pages is not None and num_pages > fit:
            raise OutOfDeviceMemory(f"num_pages={num_pages} does not fit the device: {fp.lines()}; at most {fit} pages would fit")
        if num_pages is None and fit < per_seq:
            raise OutOfDeviceMemory(f"not even one sequence of ctx={ctx} positions ({per_seq} pages) fits beside the weights: "
                               f"{fp.lines()}; at most {fit} pages would fit")
    elif free_bytes is not None and fp.needed > free_bytes:
        raise OutOfDeviceMemory(f"the model does not fit the device: {fp.lines()}")
    return fp
