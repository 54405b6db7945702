"""Feed-forward parts.

Interface: ``forward(x, ctx, residual)`` reads ``x`` ``[T, hidden]`` (activation dtype) and
**adds** its output into ``residual`` (float32 ``[T, hidden]``).  A routed feed-forward
(experts) has the same interface; what it routes on is its own business.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..kernels import ops
from .base import Part, Runtime
from .registry import register_feedforward
from .spec import TensorSpec


class FeedForward(Part):
    #: True if ``forward`` takes ``x`` as ``ops.NormedRows`` too, and a keyword ``then_norm`` (an ``ops.NormOut``),
    #: returning ``ops.NormedRows`` if its last product carried that norm and None otherwise (see ``Mixer``).
    couples_norm = False
    #: as ``Mixer.capturable``: single-token steps launch the same kernels whatever the batch holds, without a wait
    #: on the host (a routed feed-forward that reads its routing back to the host says False)
    capturable = True

    def forward(self, x: torch.Tensor, ctx, residual: torch.Tensor) -> None:
        raise NotImplementedError


@register_feedforward("swiglu")
class SwiGLU(FeedForward):
    """``down( g / (1 + exp(-g)) * u )`` with ``g = x W_gate^T`` and ``u = x W_up^T``, no bias
    (crates/model/src/qwen3/mlp.rs:22-37, crates/tensor/src/silu.rs:18)."""

    def __init__(self, hidden: int, intermediate: int, name: str):
        self.hidden, self.intermediate, self.name = int(hidden), int(intermediate), name
        self.w_gate_up = self.w_down = None

    def tensor_specs(self) -> List[TensorSpec]:
        n, h, i = self.name, self.hidden, self.intermediate
        return [
            TensorSpec(f"{n}.gate_proj.weight", (i, h)),
            TensorSpec(f"{n}.up_proj.weight", (i, h)),
            TensorSpec(f"{n}.down_proj.weight", (h, i)),
        ]

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        n = self.name
        gate, up = tensors.pop(f"{n}.gate_proj.weight"), tensors.pop(f"{n}.up_proj.weight")
        # One matrix for both projections.  Where the tensor-core kernel can apply the activation in its epilogue
        # the rows are interleaved in blocks of 16 (gate, up, gate, ...) so that a gate value and its up value
        # meet in one warp; otherwise gate rows come first, then up rows.
        self.fused = ops.can_fuse_swiglu(rt.dtype, self.hidden, self.intermediate)
        if self.fused:
            self.w_gate_up = rt.matrix(ops.interleave_gate_up(gate, up))
        else:
            self.w_gate_up = rt.matrix(torch.cat([gate, up], dim=0))
        self.w_down = rt.matrix(tensors.pop(f"{n}.down_proj.weight"))

    couples_norm = True

    def forward(self, x, ctx, residual: torch.Tensor, then_norm=None):
        T = x.shape[0]
        ws = ctx.workspace
        act = ws.get("ffn_act", (T, self.intermediate), x.dtype)
        ops.stage_name = "gate|up, SwiGLU"
        if self.fused:
            ops.gemm_swiglu(x, self.w_gate_up, act, ws)
        else:
            gate_up = ws.get("gate_up", (T, 2 * self.intermediate), x.dtype)
            ops.gemm(x, self.w_gate_up, gate_up)
            ops.swiglu(gate_up, act)
        ops.stage_name = "down"
        return ops.gemm(act, self.w_down, residual, accumulate=True, then_norm=then_norm)
