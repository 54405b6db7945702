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


def element_size(dtype: torch.dtype) -> int:
    return torch.empty(0, dtype=dtype).element_size()


def spec_bytes(spec: TensorSpec, dtype: torch.dtype) -> int:
    """Bytes of one tensor as it is kept on the device: matrices and tables in the runtime's dtype, norm weights
    in float32, integer tables in int32."""
    count = 1
    for s in spec.shape:
        count *= int(s)
    return count * (4 if spec.role in ("norm", "int_table") else element_size(dtype))


class Part:
    """Base of every part: names its tensors, takes them, frees nothing else.

    Besides computing, a part answers the questions the code around the model asks, so that memory planning, the
    build step and the measurements know nothing about any particular part:

    ``weight_bytes(dtype)``      bytes its tensors hold on the device;
    ``bytes_read(tokens, dtype)`` bytes of them a step over ``tokens`` tokens has to read (all of them unless the
                                 part says otherwise: an embedding table gives only the rows asked for);
    ``flops(tokens, pairs)``     floating-point operations of such a step; ``pairs`` counts the (query, key) pairs
                                 a mixer looks at (only mixers use it);
    ``kernel_jobs(dtype)``       ``{library name: (sources, defines)}`` of kernels specialised for this part's
                                 sizes, to be compiled before the model first runs.
    """

    def tensor_specs(self) -> List[TensorSpec]:
        return []

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        """Takes this part's tensors out of ``tensors`` (CPU, stored dtype) onto the device."""

    def weight_bytes(self, dtype: torch.dtype) -> int:
        return sum(spec_bytes(s, dtype) for s in self.tensor_specs())

    def bytes_read(self, tokens: int, dtype: torch.dtype) -> int:
        return self.weight_bytes(dtype)

    def flops(self, tokens: int, pairs: int = 0) -> float:
        """Two operations per token and element of every weight matrix; parts that do more add it."""
        total = 0
        for s in self.tensor_specs():
            if s.role == "matrix" and len(s.shape) >= 2:
                count = 1
                for n in s.shape:
                    count *= int(n)
                total += count
        return 2.0 * tokens * total

    def kernel_jobs(self, dtype: torch.dtype) -> Dict[str, tuple]:
        return {}
