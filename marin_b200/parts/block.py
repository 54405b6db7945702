"""How a layer's parts are arranged around the residual stream."""
from __future__ import annotations

from typing import Dict, List

import torch

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

    def forward(self, hidden: torch.Tensor, ctx, cache) -> None:
        ws = ctx.workspace
        normed = ws.get("normed", tuple(hidden.shape), self.rt.dtype)
        self.norm1.forward(hidden, normed)
        self.mixer.forward(normed, ctx, cache, hidden)
        self.norm2.forward(hidden, normed)
        self.feedforward.forward(normed, ctx, hidden)
