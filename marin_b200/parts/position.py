"""Position encodings.

A rotary encoding hands the attention mixer a table of inverse frequencies and says how
pairs are formed; the fused norm + rotation + cache-write kernel takes both as
parameters.  ``NoPosition`` hands over nothing and the mixer skips the rotation.
"""
from __future__ import annotations

from typing import Optional

import torch

from .base import Part, Runtime
from .registry import register_position


class PositionEncoding(Part):
    #: float32 ``[rotary_dim // 2]`` on the device, or None when nothing rotates
    inv_freq: Optional[torch.Tensor] = None
    rotary_dim: int = 0
    #: False: element i pairs with i + rotary_dim/2 ("rotate half"); True: (2i, 2i+1)
    interleaved: bool = False


@register_position("rope")
class Rotary(PositionEncoding):
    """Rotary embedding with half-split pairing.

    ``f_i = theta^(-(2i/d))`` in float32 and ``angle = float(pos) * f_i``; the pair
    ``(a, b) = (x[i], x[i + d/2])`` becomes ``(a cos - b sin, b cos + a sin)``
    (crates/tensor/src/ops.rs:52-95, crates/cuda/src/kernels.cu:147-162).
    """

    def __init__(self, head_dim: int, theta: float, rotary_dim: Optional[int] = None, interleaved: bool = False):
        self.head_dim = int(head_dim)
        self.theta = float(theta)
        self.rotary_dim = int(rotary_dim) if rotary_dim is not None else self.head_dim
        self.interleaved = bool(interleaved)
        if self.rotary_dim % 2 != 0 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and within head_dim {self.head_dim}")

    def load(self, tensors, rt: Runtime) -> None:
        half = self.rotary_dim // 2
        i = torch.arange(half, dtype=torch.float32)
        exponent = -(i * 2.0 / float(self.rotary_dim))
        self.inv_freq = torch.pow(torch.tensor(self.theta, dtype=torch.float32), exponent).to(rt.device)


@register_position("none")
class NoPosition(PositionEncoding):
    def __init__(self, **_ignored):
        self.inv_freq, self.rotary_dim = None, 0
