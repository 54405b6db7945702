"""What one step hands to the parts: the batch, flattened, as device tensors."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Tuple

import torch


class Workspace:
    """Activation buffers by name, kept between steps so that a step allocates nothing once warm."""

    def __init__(self, device):
        self.device = device
        self._buffers: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}

    def get(self, name: str, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        count = 1
        for s in shape:
            count *= int(s)
        key = (name, dtype)
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < count:
            buf = torch.empty(max(count, 1), device=self.device, dtype=dtype)
            self._buffers[key] = buf
        return buf[:count].view(*shape)


@dataclass
class Span:
    """One request's part in the step, on the host: where its tokens lie in the flat batch."""

    row: int          # index among the step's requests
    req_id: object
    start: int        # first flat token index
    count: int        # tokens in this step
    pos0: int         # position of its first token (= cached length before the step)
    slot: int         # per-request state slot


@dataclass
class StepContext:
    num_tokens: int
    num_requests: int
    num_decode: int            # the first `num_decode` requests bring exactly one token each
    num_logit_rows: int
    max_query_len: int
    max_seq_len: int           # longest sequence (after this step) in the batch
    token_ids: torch.Tensor    # int32 [T]
    positions: torch.Tensor    # int32 [T]
    req_index: torch.Tensor    # int32 [T]: row of the request each token belongs to
    cu_tokens: torch.Tensor    # int32 [R+1]: where each request's tokens start in the flat batch
    seq_lens: torch.Tensor     # int32 [R]: length of each request after this step
    state_slots: torch.Tensor  # int32 [R]
    logit_rows: torch.Tensor   # int32 [W]: flat token indices whose logits are wanted
    group_block_tables: List[torch.Tensor]   # per cache group: int32 [R, max_pages]
    group_slot_mappings: List[torch.Tensor]  # per cache group: int32 [T]
    spans: List[Span]
    workspace: Workspace
    extras: Dict[str, object] = field(default_factory=dict)
    #: set for captured single-token steps: what each kind of mixer fixed ahead for them (``Mixer.decode_plan``), by
    #: the mixers' ``decode_plan_key()``; the capture owns the plans' scratch memory
    decode_plans: Dict[object, object] = field(default_factory=dict)
