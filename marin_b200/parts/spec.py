"""Plain data that describes a model: which parts each layer is made of, and the order layers run in.

A model is data before it is code.  An architecture's builder turns its typed
configuration into a :class:`ModelSpec`; :class:`marin_b200.models.model.Model` turns the
spec into parts by looking every ``kind`` up in the part registries.  Nothing in
a part knows which model it is in: it sees only its own parameters.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass(frozen=True)
class TensorSpec:
    """One tensor a part expects in the checkpoint.

    ``role`` decides storage and random initialisation: ``matrix`` (bf16 or f32,
    N(0, 0.02)), ``norm`` (kept f32 on the device, 1 + N(0, 0.05)), ``table``
    (an embedding table, treated like a matrix), ``int_table`` (int32).
    """

    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"


@dataclass
class PartSpec:
    """A part chosen by name from a registry, with the parameters it is built from."""

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass
class LayerSpec:
    """One layer: how its parts are arranged (``block``) and which parts they are."""

    block: str
    norm: PartSpec
    mixer: PartSpec
    feedforward: PartSpec
    prefix: str
    #: names inside ``prefix`` of the sub-modules, so that parts find their tensors
    names: Dict[str, str] = field(default_factory=dict)


@dataclass
class ScheduleEntry:
    """One run of a layer.  ``cache_of`` names an earlier entry whose cache this run reads
    instead of keeping one of its own (it then writes nothing)."""

    layer: int
    cache_of: Optional[int] = None


@dataclass
class ModelSpec:
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    final_norm: PartSpec
    head: PartSpec
    layers: List[LayerSpec]
    schedule: List[ScheduleEntry]
    #: tensors that may be present in a checkpoint and are ignored (e.g. an unused head when tied)
    ignorable: Tuple[str, ...] = ()
