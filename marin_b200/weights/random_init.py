"""Random-weights mode: a model folder (config.json, model.safetensors) from a configuration and a seed.

Matrices and tables are N(0, 0.02), norm weights 1 + N(0, 0.05).  Every tensor is drawn
from a generator seeded by (seed, tensor name), so a tensor's values do not depend on
which other tensors exist or in which order they are made.  The reference has no such
mode in its engine; its fixture script draws a random Qwen3 the same way
(scripts/gen_reference.py:82-118).
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Iterator, Tuple

import torch

from ..config.base import ModelConfig
from ..parts.spec import TensorSpec
from .safetensors_io import write_safetensors

MATRIX_STD = 0.02
NORM_STD = 0.05
#: most elements drawn in one go (tensors above this are drawn in runs of rows: same seed, same values every time, but
#: not the values one draw of the whole tensor would give)
DRAW_AT_ONCE = 1 << 26


def _seed_for(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(digest[:8], "little") & ((1 << 63) - 1)


def random_tensor(spec: TensorSpec, seed: int, dtype: torch.dtype, device="cpu",
                  matrix_std: float = MATRIX_STD, norm_std: float = NORM_STD) -> torch.Tensor:
    gen = torch.Generator(device=device)
    gen.manual_seed(_seed_for(seed, spec.name))
    if spec.role == "int_table":
        return torch.randint(0, 2 ** 15, spec.shape, generator=gen, device=device, dtype=torch.int32)
    count = 1
    for n in spec.shape:
        count *= int(n)
    if count > DRAW_AT_ONCE and dtype != torch.float32 and len(spec.shape) >= 1:
        # a large table is drawn in runs of rows, so that the float32 draw never holds more than a fraction of it
        out = torch.empty(spec.shape, device=device, dtype=dtype)
        rows = max(1, DRAW_AT_ONCE // max(1, count // int(spec.shape[0])))
        for at in range(0, int(spec.shape[0]), rows):
            part = torch.randn((min(rows, int(spec.shape[0]) - at), *spec.shape[1:]), generator=gen, device=device, dtype=torch.float32)
            out[at:at + rows] = ((1.0 + norm_std * part) if spec.role == "norm" else matrix_std * part).to(dtype)
        return out
    values = torch.randn(spec.shape, generator=gen, device=device, dtype=torch.float32)
    if spec.role == "norm":
        values = 1.0 + norm_std * values
    else:
        values = matrix_std * values
    return values.to(dtype)


def random_tensors(config: ModelConfig, seed: int, dtype: torch.dtype = torch.bfloat16, device="cpu",
                   **scales) -> Iterator[Tuple[str, torch.Tensor]]:
    from ..models import Model, architecture_of

    model = Model(architecture_of(config).build_spec(config))
    for spec in model.tensor_specs():
        yield spec.name, random_tensor(spec, seed, dtype, device, **scales)


def write_random_model(model_dir: str, config: ModelConfig, seed: int,
                       dtype: torch.dtype = torch.bfloat16, **scales) -> str:
    """Writes ``config.json`` and ``model.safetensors`` for ``config`` into ``model_dir``."""
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as fh:
        json.dump(config.to_json_dict(), fh, indent=2)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), random_tensors(config, seed, dtype, **scales))
    return model_dir
