"""Typed model configuration: the base class and the reading of ``config.json``.

Every size and constant of a model comes from the keys of its own ``config.json``;
nothing in this package hard-codes one.  A configuration class per architecture
turns the raw keys into typed fields and refuses variants the engine does not
implement, the way the reference's ``Qwen3Config::parse`` does
(crates/model/src/qwen3/config.rs:79-123, refusals :198-222).
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


class ConfigError(ValueError):
    """A config.json that is malformed, incomplete or names an unsupported variant."""


@dataclass
class ModelConfig:
    """Fields every architecture's configuration exposes to the engine."""

    architecture: str = ""
    model_type: str = ""
    vocab_size: int = 0
    hidden_size: int = 0
    max_position_embeddings: int = 0
    eos_token_ids: List[int] = field(default_factory=list)
    raw: Dict[str, Any] = field(default_factory=dict, repr=False, compare=False)

    def to_json_dict(self) -> Dict[str, Any]:
        """The config.json this configuration would be read back from."""
        raise NotImplementedError


def read_json(path: str) -> Dict[str, Any]:
    try:
        with open(path, "r", encoding="utf-8") as fh:
            value = json.load(fh)
    except FileNotFoundError as err:
        raise ConfigError(f"{path} does not exist") from err
    except json.JSONDecodeError as err:
        raise ConfigError(f"{path} is not valid JSON: {err}") from err
    if not isinstance(value, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    return value


def require(raw: Dict[str, Any], key: str, kind) -> Any:
    if key not in raw or raw[key] is None:
        raise ConfigError(f"config.json: `{key}` is missing")
    value = raw[key]
    if kind is int:
        if isinstance(value, bool) or not isinstance(value, int):
            raise ConfigError(f"config.json: `{key}` must be an integer, got {value!r}")
    elif kind is float:
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise ConfigError(f"config.json: `{key}` must be a number, got {value!r}")
        value = float(value)
        if not math.isfinite(value):
            raise ConfigError(f"config.json: `{key}` must be finite, got {value!r}")
    elif kind is str:
        if not isinstance(value, str):
            raise ConfigError(f"config.json: `{key}` must be a string, got {value!r}")
    return value


def optional(raw: Dict[str, Any], key: str, kind, default=None) -> Any:
    if key not in raw or raw[key] is None:
        return default
    return require(raw, key, kind)


def eos_ids(value: Any) -> List[int]:
    """``eos_token_id`` may be one id or a list (config.rs:8-21)."""
    if value is None:
        return []
    if isinstance(value, int) and not isinstance(value, bool):
        return [value]
    if isinstance(value, list) and all(isinstance(v, int) and not isinstance(v, bool) for v in value):
        return list(value)
    raise ConfigError(f"config.json: `eos_token_id` must be an id or a list of ids, got {value!r}")


def load_config(model_dir: str) -> ModelConfig:
    """Reads ``config.json`` (and ``generation_config.json`` if present) of a model folder.

    The configuration class is chosen by the registry from ``architectures[0]`` or,
    failing that, ``model_type``.
    """
    from ..models.registry import architecture_for

    raw = read_json(os.path.join(model_dir, "config.json"))
    generation = None
    gen_path = os.path.join(model_dir, "generation_config.json")
    if os.path.exists(gen_path):
        generation = read_json(gen_path)
    arch = architecture_for(raw)
    return arch.config_class.from_dict(raw, generation)
