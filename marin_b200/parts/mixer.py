"""Mixers: the parts that let tokens see other tokens.

Interface every mixer has (a test can register its own):

``cache_need()`` → what it keeps between steps: a :class:`PagedKV` (keys and values
in pages, all of them or a window), a :class:`StateNeed` (fixed-size per-request
state), or None.

``forward(x, ctx, cache, residual)`` → reads ``x`` ``[T, hidden]`` (activation dtype),
mixes over each request's tokens and what ``cache`` holds, and **adds** its output
into ``residual`` (float32 ``[T, hidden]``).  ``ctx`` is the step's
:class:`marin_b200.engine.context.StepContext`; ``cache`` is this run's view of the
cache (:class:`marin_b200.cache.manager.PagedView` or ``StateView``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from ..kernels import ops
from .base import Part, Runtime, element_size
from .registry import lookup, register_mixer
from .spec import PartSpec, TensorSpec


@dataclass(frozen=True)
class PagedKV:
    """Keys and values of ``kv_heads`` heads of ``head_dim`` per position, kept in pages.
    ``window`` = how many of the latest positions are ever read again (None: all)."""

    kv_heads: int
    head_dim: int
    window: Optional[int] = None

    def bytes_per_token(self, dtype: torch.dtype) -> int:
        """Bytes one position of one layer holds in the cache (keys and values)."""
        return 2 * self.kv_heads * self.head_dim * element_size(dtype)

    def bytes_read(self, context: int, dtype: torch.dtype) -> int:
        """Bytes one decoded token reads of a sequence of ``context`` positions."""
        kept = context if self.window is None else min(context, self.window)
        return kept * self.bytes_per_token(dtype)


@dataclass(frozen=True)
class StateNeed:
    """A fixed-size state per request: ``shape`` elements of ``dtype``, zeroed when a request starts."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32

    def bytes(self) -> int:
        count = 1
        for s in self.shape:
            count *= int(s)
        return count * element_size(self.dtype)

    def bytes_read(self, context: int, dtype: torch.dtype) -> int:
        return self.bytes()


class Mixer(Part):
    #: True if ``forward`` takes ``x`` as ``ops.NormedRows`` too, and a keyword ``then_norm`` (an ``ops.NormOut``:
    #: the norm wanted of the updated residual), returning ``ops.NormedRows`` if its last product carried that norm
    #: and None otherwise.  A block couples norms only between parts that both say so.
    couples_norm = False
    #: True if a step in which every request brings one token may be captured in a CUDA graph and replayed for other
    #: requests of the same number: ``forward`` then launches the same kernels whatever the lengths and slots are,
    #: reads them from ``ctx``'s device tensors only (never ``ctx.spans`` or another host value), and waits for
    #: nothing on the host.  The step function captures graphs only for models whose parts all say so.  Rows that
    #: pad a captured batch stand for empty requests: length 0, the spare state slot (see ``CacheManager``).
    capturable = True

    def cache_need(self):
        return None

    def decode_plan_key(self):
        """Mixers that answer the same (hashable) key share one decode plan per captured graph; None: no plan."""
        return None

    def decode_plan(self, requests: int, span: int, rt: Runtime):
        """What this mixer fixes ahead for single-token steps of ``requests`` requests whose sequences are at most
        ``span`` long: how it splits the work and the scratch memory it then needs.  A captured graph owns the plan;
        ``forward`` finds it as ``ctx.decode_plans[self.decode_plan_key()]``."""
        return None

    def forward(self, x: torch.Tensor, ctx, cache, residual: torch.Tensor) -> None:
        raise NotImplementedError


@register_mixer("gqa_attention")
class GQAttention(Mixer):
    """Causal grouped-query attention over the paged cache.

    ``q,k,v = x W^T`` (no bias); optional per-head RMSNorm of q and k over ``head_dim``
    *before* the rotation; keys (normed, rotated) and values (raw) go to the cache; query
    head ``h`` reads kv head ``h // (heads // kv_heads)``; scores scaled by
    ``1/sqrt(head_dim)``; softmax in float32 over positions ``0..=pos`` (or the last
    ``window``); output through ``o_proj`` added to the residual
    (crates/model/src/qwen3/layer.rs:59-88, crates/tensor/src/attention.rs:148-169).
    """

    def __init__(self, hidden: int, heads: int, kv_heads: int, head_dim: int, name: str,
                 position: PartSpec, qk_norm: bool = True, norm_eps: float = 1e-6,
                 window: Optional[int] = None, scale: Optional[float] = None):
        self.hidden, self.heads, self.kv_heads, self.head_dim = int(hidden), int(heads), int(kv_heads), int(head_dim)
        if self.heads % self.kv_heads != 0:
            raise ValueError(f"{heads} heads cannot share {kv_heads} kv heads evenly")
        self.name, self.qk_norm, self.norm_eps = name, bool(qk_norm), float(norm_eps)
        self.window = int(window) if window else None
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        self.position = lookup("position", position.kind)(**position.params)
        self.q_dim, self.kv_dim = self.heads * self.head_dim, self.kv_heads * self.head_dim
        self.w_qkv = self.w_o = self.q_weight = self.k_weight = None

    def cache_need(self):
        return PagedKV(self.kv_heads, self.head_dim, self.window)

    def tensor_specs(self) -> List[TensorSpec]:
        n, h, d = self.name, self.hidden, self.head_dim
        specs = [
            TensorSpec(f"{n}.q_proj.weight", (self.q_dim, h)),
            TensorSpec(f"{n}.k_proj.weight", (self.kv_dim, h)),
            TensorSpec(f"{n}.v_proj.weight", (self.kv_dim, h)),
            TensorSpec(f"{n}.o_proj.weight", (h, self.q_dim)),
        ]
        if self.qk_norm:
            specs += [TensorSpec(f"{n}.q_norm.weight", (d,), "norm"), TensorSpec(f"{n}.k_norm.weight", (d,), "norm")]
        return specs

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        n = self.name
        q, k, v = (tensors.pop(f"{n}.{p}_proj.weight") for p in "qkv")
        # One matrix for the three projections: one pass over x instead of three.
        self.w_qkv = rt.matrix(torch.cat([q, k, v], dim=0))
        self.w_o = rt.matrix(tensors.pop(f"{n}.o_proj.weight"))
        if self.qk_norm:
            self.q_weight = rt.f32(tensors.pop(f"{n}.q_norm.weight"))
            self.k_weight = rt.f32(tensors.pop(f"{n}.k_norm.weight"))
        self.position.load(tensors, rt)
        self.rt = rt

    couples_norm = True

    def flops(self, tokens: int, pairs: int = 0) -> float:
        """The four projections, and per (query, key) pair a score and a weighted value of ``head_dim`` each."""
        return super().flops(tokens, pairs) + 4.0 * pairs * self.heads * self.head_dim

    def kernel_jobs(self, dtype) -> Dict[str, tuple]:
        return ops.attention_jobs(dtype, self.heads, self.kv_heads, self.head_dim)

    def decode_plan_key(self):
        return ("paged_attention", self.heads, self.kv_heads, self.head_dim)

    def decode_plan(self, requests: int, span: int, rt: Runtime):
        return ops.decode_plan(rt.device, rt.dtype, requests, self.heads, self.kv_heads, self.head_dim, span)

    def forward(self, x, ctx, cache, residual: torch.Tensor, then_norm=None):
        T = x.shape[0]
        ws = ctx.workspace
        writes = cache.owner
        pos = self.position
        q = ws.get("q", (T, self.q_dim), x.dtype)
        # A run that reads another run's cache computes only the queries.
        w = self.w_qkv if writes else self.w_qkv[: self.q_dim]
        ops.stage_name = "q|k|v, heads"
        if not ops.gemm_qkv_heads(x, w, q, self.q_weight, self.k_weight, self.norm_eps, ctx.positions, pos.inv_freq,
                                  pos.rotary_dim, pos.interleaved, cache.slot_mapping, cache.k, cache.v, self.heads,
                                  self.kv_heads, self.head_dim, writes, ctx):
            qkv = ws.get("qkv", (T, w.shape[0]), x.dtype)
            ops.gemm(x, w, qkv)
            ops.qk_norm_rope_write(
                qkv, q, self.q_weight, self.k_weight, self.norm_eps, ctx.positions,
                pos.inv_freq, pos.rotary_dim, pos.interleaved, cache.slot_mapping,
                cache.k, cache.v, self.heads, self.kv_heads, self.head_dim, writes,
            )
        out = ws.get("attn_out", (T, self.q_dim), x.dtype)
        ops.stage_name = "attention"
        plans = ctx.decode_plans
        ops.attention(q, cache.k, cache.v, out, ctx, cache.block_table, self.heads, self.kv_heads,
                      self.head_dim, self.scale, self.window or 0, plans.get(self.decode_plan_key()) if plans else None)
        ops.stage_name = "o"
        return ops.gemm(out, self.w_o, residual, accumulate=True, then_norm=then_norm)
