"""A model assembled from a :class:`ModelSpec`: embedding, blocks run in schedule order,
final norm and head.  It owns weights only; caches and batches come from outside."""
from __future__ import annotations

from typing import Dict, List

import torch

from ..kernels import ops
from ..parts.base import Runtime
from ..parts.registry import lookup
from ..parts.spec import ModelSpec, TensorSpec


class Model:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.embedding = lookup("embedding", spec.embedding.kind)(**spec.embedding.params)
        self.blocks = [lookup("block", layer.block)(layer) for layer in spec.layers]
        self.final_norm = lookup("norm", spec.final_norm.kind)(**spec.final_norm.params)
        self.head = lookup("head", spec.head.kind)(**spec.head.params)
        for i, entry in enumerate(spec.schedule):
            if not 0 <= entry.layer < len(self.blocks):
                raise ValueError(f"schedule entry {i} names layer {entry.layer}, the model has {len(self.blocks)}")
            if entry.cache_of is not None:
                if not 0 <= entry.cache_of < i or spec.schedule[entry.cache_of].cache_of is not None:
                    raise ValueError(f"schedule entry {i} must read the cache of an earlier entry that owns one")
        self.rt: Runtime | None = None

    def tensor_specs(self) -> List[TensorSpec]:
        specs = list(self.embedding.tensor_specs())
        for block in self.blocks:
            specs += block.tensor_specs()
        specs += self.final_norm.tensor_specs()
        specs += self.head.tensor_specs()
        return specs

    def cache_needs(self) -> List[object]:
        """What each schedule entry keeps between steps (None for entries that read another's cache)."""
        needs = []
        for entry in self.spec.schedule:
            need = self.blocks[entry.layer].mixer.cache_need()
            needs.append(need if entry.cache_of is None else None)
        return needs

    # ---- what the code around the model asks of it: every answer is the sum of the parts' own answers ----------------
    def parts(self) -> List[object]:
        """Every part of the model once: embedding, the blocks' parts in layer order, final norm, head."""
        out = [self.embedding]
        for block in self.blocks:
            out += block.parts() if hasattr(block, "parts") else [block]
        return out + [self.final_norm, self.head]

    def weight_bytes(self, dtype: torch.dtype) -> int:
        """Bytes the weights hold on the device (a tied head holds none of its own)."""
        return sum(p.weight_bytes(dtype) for p in self.parts())

    def bytes_read(self, tokens: int, dtype: torch.dtype) -> int:
        """Bytes of weights a step over ``tokens`` tokens has to read: every layer run as often as the schedule names
        it, the embedding's rows, the whole head."""
        total = self.embedding.bytes_read(tokens, dtype) + self.final_norm.bytes_read(tokens, dtype) + self.head.bytes_read(tokens, dtype)
        for entry in self.spec.schedule:
            total += self.blocks[entry.layer].bytes_read(tokens, dtype)
        return total

    def flops(self, tokens: int, pairs: int, logit_rows: int) -> float:
        """Floating-point operations of a step over ``tokens`` tokens in which every mixer looks at ``pairs``
        (query, key) pairs and ``logit_rows`` rows go through the head."""
        total = self.head.flops(logit_rows)
        for entry in self.spec.schedule:
            total += self.blocks[entry.layer].flops(tokens, pairs)
        return total

    def cache_bytes_read(self, context: int, dtype: torch.dtype) -> int:
        """Bytes of the cache one decoded token of a sequence of ``context`` positions reads, over all schedule entries."""
        total = 0
        for entry in self.spec.schedule:
            need = self.blocks[entry.layer].mixer.cache_need()
            if need is not None:
                total += need.bytes_read(context, dtype)
        return total

    def kernel_jobs(self, dtype: torch.dtype) -> Dict[str, tuple]:
        """``{library: (sources, defines)}`` of the kernels specialised for this model's parts."""
        jobs: Dict[str, tuple] = {}
        for p in self.parts():
            jobs.update(p.kernel_jobs(dtype))
        return jobs

    def capturable(self) -> bool:
        """Whether single-token steps of this model may be captured in CUDA graphs: every mixer and feed-forward says so."""
        return all(getattr(p, "capturable", True) for p in self.parts())

    def decode_plans(self, requests: int, span: int) -> Dict[object, object]:
        """One decode plan per kind of mixer (``Mixer.decode_plan_key``), for a captured graph of ``requests`` rows
        over sequences of up to ``span`` positions."""
        plans: Dict[object, object] = {}
        for p in self.parts():
            key = p.decode_plan_key() if hasattr(p, "decode_plan_key") else None
            if key is not None and key not in plans:
                plan = p.decode_plan(requests, span, self.rt)
                if plan is not None:
                    plans[key] = plan
        return plans

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        self.embedding.load(tensors, rt)
        for block in self.blocks:
            block.load(tensors, rt)
        self.final_norm.load(tensors, rt)
        self.head.load(tensors, rt)
        if getattr(self.head, "tied", False):
            self.head.tie(self.embedding.table)

    def forward(self, ctx, caches, observe=None) -> torch.Tensor:
        """Runs the step's tokens through every schedule entry; returns float32 logits
        ``[len(ctx.logit_rows), vocab]`` at the rows asked for.  ``observe(i, hidden)`` is called with the
        residual stream (float32 ``[T, hidden]``) before the first entry (i = 0) and after entry i - 1."""
        rt, ws = self.rt, ctx.workspace
        T = ctx.num_tokens
        hidden = ws.get("hidden", (T, self.spec.hidden_size), torch.float32)
        ops.stage_name = "embedding"
        self.embedding.forward(ctx.token_ids, hidden)
        if observe is not None:
            observe(0, hidden)
        carried = None            # the next block's first norm, if the block before could carry it on its last product
        schedule = self.spec.schedule
        for i, entry in enumerate(schedule):
            block = self.blocks[entry.layer]
            if getattr(block, "chains_norm", False):
                following = self.blocks[schedule[i + 1].layer] if i + 1 < len(schedule) else None
                carried = block.forward(hidden, ctx, caches.view(i, ctx), x_in=carried, next_block=following)
            else:
                block.forward(hidden, ctx, caches.view(i, ctx))
                carried = None
            if observe is not None:
                observe(i + 1, hidden)
        W = ctx.num_logit_rows
        if W == 0:
            return torch.empty(0, self.spec.vocab_size, device=rt.device, dtype=torch.float32)
        ops.stage_name = "final norm"
        rows = ws.get("logit_hidden", (W, self.spec.hidden_size), torch.float32)
        ops.gather_rows(hidden, ctx.logit_rows, rows)
        normed = ws.get("logit_normed", (W, self.spec.hidden_size), rt.dtype)
        self.final_norm.forward(rows, normed)
        ops.stage_name = "head"
        logits = ws.get("logits", (W, self.spec.vocab_size), torch.float32)
        self.head.forward(normed, logits)
        return logits
