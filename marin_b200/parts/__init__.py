"""The parts models are put together from, and the registries that name them."""
from . import block, embedding, feedforward, mixer, norm, position  # noqa: F401  (registration)
from .base import Part, Runtime
from .mixer import Mixer, PagedKV, StateNeed
from .feedforward import FeedForward
from .position import PositionEncoding
from .registry import (lookup, register_block, register_embedding, register_feedforward, register_head,
                       register_mixer, register_norm, register_position)
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorSpec

__all__ = [
    "Part", "Runtime", "Mixer", "PagedKV", "StateNeed", "FeedForward", "PositionEncoding", "lookup",
    "register_block", "register_embedding", "register_feedforward", "register_head", "register_mixer",
    "register_norm", "register_position", "LayerSpec", "ModelSpec", "PartSpec", "ScheduleEntry", "TensorSpec",
]
