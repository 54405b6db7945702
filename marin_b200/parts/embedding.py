"""Token embedding and output head."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .base import Part, Runtime, element_size
from .registry import register_embedding, register_head
from .spec import TensorSpec


@register_embedding("token_table")
class TokenEmbedding(Part):
    """``hidden[t] = float32(table[ids[t]])`` — no scaling, no position term
    (crates/model/src/qwen3/model.rs:133-153)."""

    def __init__(self, vocab: int, hidden: int, name: str):
        self.vocab, self.hidden, self.name = int(vocab), int(hidden), name
        self.table: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(f"{self.name}.weight", (self.vocab, self.hidden), "table")]

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.table = rt.matrix(tensors.pop(f"{self.name}.weight"))

    def bytes_read(self, tokens: int, dtype: torch.dtype) -> int:
        return tokens * self.hidden * element_size(dtype)          # only the rows asked for leave memory

    def forward(self, ids: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        ops.embed(ids, self.table, out)
        return out


@register_head("linear")
class LinearHead(Part):
    """``logits = rows W^T`` in float32; ``tied_to`` names the embedding whose table is the
    head matrix when the checkpoint has no ``lm_head`` (model.rs:125-127)."""

    def __init__(self, vocab: int, hidden: int, name: str, tied: bool = False):
        self.vocab, self.hidden, self.name, self.tied = int(vocab), int(hidden), name, bool(tied)
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [] if self.tied else [TensorSpec(f"{self.name}.weight", (self.vocab, self.hidden), "table")]

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        if not self.tied:
            self.weight = rt.matrix(tensors.pop(f"{self.name}.weight"))

    def tie(self, table: torch.Tensor) -> None:
        self.weight = table

    def bytes_read(self, tokens: int, dtype: torch.dtype) -> int:
        return self.vocab * self.hidden * element_size(dtype)      # tied or not, the whole matrix is read

    def flops(self, tokens: int, pairs: int = 0) -> float:
        """``tokens`` counts the rows whose logits are wanted."""
        return 2.0 * tokens * self.vocab * self.hidden

    def forward(self, rows: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        ops.gemm(rows, self.weight, out)
        return out
