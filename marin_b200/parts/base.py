"""What every part has in common: the tensors it expects and how it takes them.

``Runtime`` carries what a part needs to know about where it runs: the device and the
activation dtype (``torch.bfloat16`` for the serving path, ``torch.float32`` for the
true 32-bit path).  The residual stream is float32 in both.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List

import torch

from .spec import TensorSpec


@dataclass
class Runtime:
    device: torch.device
    dtype: torch.dtype  # activations and matrices: torch.bfloat16 or torch.float32

    def matrix(self, t: torch.Tensor) -> torch.Tensor:
        """A weight matrix as the kernels of this runtime read it."""
        return t.to(device=self.device, dtype=self.dtype).contiguous()

    def f32(self, t: torch.Tensor) -> torch.Tensor:
        """Norm weights and other small vectors are kept in float32 (bf16 to f32 is exact)."""
        return t.to(device=self.device, dtype=torch.float32).contiguous()

    def empty(self, *shape, dtype=None) -> torch.Tensor:
        return torch.empty(*shape, device=self.device, dtype=dtype or self.dtype)


class Part:
    """Base of every part: names its tensors, takes them, frees nothing else."""

    def tensor_specs(self) -> List[TensorSpec]:
        return []

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        """Takes this part's tensors out of ``tensors`` (CPU, stored dtype) onto the device."""
