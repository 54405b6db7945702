"""How a layer's parts are arranged around the residual stream."""
from __future__ import annotations

from typing import Dict, List

import torch

from ..kernels import ops
from .base import Part, Runtime
from .registry import lookup, register_block
from .spec import LayerSpec, TensorSpec


@register_block("prenorm")
class PreNormBlock(Part):
    """``h += mixer(norm1(h)); h += feedforward(norm2(h))`` — the residual stream ``h`` stays
    float32 and both parts add into it (crates/model/src/qwen3/layer.rs:56-103)."""

    def __init__(self, spec: LayerSpec):
        names = spec.names
        norm_cls = lookup("norm", spec.norm.kind)
        self.norm1 = norm_cls(name=f"{spec.prefix}.{names['norm1']}", **spec.norm.params)
        self.norm2 = norm_cls(name=f"{spec.prefix}.{names['norm2']}", **spec.norm.params)
        self.mixer = lookup("mixer", spec.mixer.kind)(name=f"{spec.prefix}.{names['mixer']}", **spec.mixer.params)
        self.feedforward = lookup("feedforward", spec.feedforward.kind)(
            name=f"{spec.prefix}.{names['feedforward']}", **spec.feedforward.params)

    def parts(self) -> List[Part]:
        return [self.norm1, self.mixer, self.norm2, self.feedforward]

    def tensor_specs(self) -> List[TensorSpec]:
        return [s for p in self.parts() for s in p.tensor_specs()]

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        for p in self.parts():
            p.load(tensors, rt)
        self.rt = rt

    def weight_bytes(self, dtype) -> int:
        return sum(p.weight_bytes(dtype) for p in self.parts())

    def bytes_read(self, tokens: int, dtype) -> int:
        return sum(p.bytes_read(tokens, dtype) for p in self.parts())

    def flops(self, tokens: int, pairs: int = 0) -> float:
        return sum(p.flops(tokens, pairs) for p in self.parts())

    def kernel_jobs(self, dtype) -> Dict[str, tuple]:
        jobs: Dict[str, tuple] = {}
        for p in self.parts():
            jobs.update(p.kernel_jobs(dtype))
        return jobs

    #: ``forward`` takes ``x_in`` / ``next_block`` and returns the next block's input (see there)
    chains_norm = True

    def _rider(self, norm, producer, consumer, out):
        """``norm`` as a rider on ``producer``'s last product, if both parts around it can couple."""
        if getattr(producer, "couples_norm", False) and getattr(consumer, "couples_norm", False) and hasattr(norm, "coupling"):
            return norm.coupling(out)
        return None

    def forward(self, hidden: torch.Tensor, ctx, cache, x_in=None, next_block=None):
        """``x_in``: this block's first norm of ``hidden``, already there or carried by the block before (what that
        block returned).  ``next_block``: the block that runs next; if its first norm can ride on this block's last
        product, its input is returned, else None."""
        ws = ctx.workspace
        normed = ws.get("normed", tuple(hidden.shape), self.rt.dtype)
        if x_in is None:
            ops.stage_name = "norm"
        x = x_in if x_in is not None else self.norm1.forward(hidden, normed)
        rider = self._rider(self.norm2, self.mixer, self.feedforward, normed)
        x = self.mixer.forward(x, ctx, cache, hidden, then_norm=rider) if rider is not None else self.mixer.forward(x, ctx, cache, hidden)
        if x is None:
            ops.stage_name = "norm"
            x = self.norm2.forward(hidden, normed)
        rider = None
        if next_block is not None and getattr(next_block, "chains_norm", False):
            rider = self._rider(next_block.norm1, self.feedforward, next_block.mixer, normed)
        if rider is not None:
            return self.feedforward.forward(x, ctx, hidden, then_norm=rider)
        self.feedforward.forward(x, ctx, hidden)
        return None
