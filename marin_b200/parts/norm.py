"""Normalisation parts."""
from __future__ import annotations

from typing import Dict, List

import torch

from ..kernels import ops
from .base import Part, Runtime
from .registry import register_norm
from .spec import TensorSpec


@register_norm("rmsnorm")
class RMSNorm(Part):
    """``y_i = x_i / sqrt(mean(x^2) + eps) * w_i`` over the last axis, sums in float32.

    The weight multiplies directly (no ``1 + w``), as the reference computes it
    (crates/tensor/src/norm.rs:16-22, crates/cuda/src/kernels.cu:51-58); ``unit_offset``
    selects the ``1 + w`` form other architectures use.
    """

    def __init__(self, dim: int, eps: float, name: str, unit_offset: bool = False):
        self.dim, self.eps, self.name, self.unit_offset = int(dim), float(eps), name, bool(unit_offset)
        self.weight: torch.Tensor | None = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(f"{self.name}.weight", (self.dim,), "norm")]

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.weight = rt.f32(tensors.pop(f"{self.name}.weight"))

    def forward(self, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """``x`` float32 ``[rows, dim]`` → ``out`` (float32 or bfloat16) ``[rows, dim]``."""
        ops.rmsnorm(x, self.weight, self.eps, out, self.unit_offset)
        return out

    def coupling(self, out: torch.Tensor) -> "ops.NormOut":
        """This norm as a rider on the product that last updates its input (``ops.gemm(..., then_norm=...)``)."""
        return ops.NormOut(self.weight, self.unit_offset, self.eps, out)
