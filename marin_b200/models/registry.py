"""One registry from an architecture's name to its configuration class and model builder.

``config.json`` chooses the model everywhere in this package: ``architectures[0]`` if
registered, else ``model_type``.  (The reference dispatches on ``model_type`` with an
if-chain, crates/model/src/qwen3/engine.rs:132-165.)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Optional

from ..config.base import ConfigError, ModelConfig
from ..parts.spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    model_type: str
    config_class: type
    build_spec: Callable[[ModelConfig], ModelSpec]


_BY_NAME: Dict[str, Architecture] = {}
_BY_MODEL_TYPE: Dict[str, Architecture] = {}


def register_architecture(name: str, model_type: str, config_class: type,
                          build_spec: Callable[[ModelConfig], ModelSpec]) -> Architecture:
    arch = Architecture(name, model_type, config_class, build_spec)
    _BY_NAME[name] = arch
    _BY_MODEL_TYPE[model_type] = arch
    return arch


def architecture_for(raw: Dict[str, Any]) -> Architecture:
    """The registered architecture a raw config.json names."""
    for name in raw.get("architectures") or []:
        if name in _BY_NAME:
            return _BY_NAME[name]
    model_type: Optional[str] = raw.get("model_type")
    if model_type in _BY_MODEL_TYPE:
        return _BY_MODEL_TYPE[model_type]
    raise ConfigError(
        f"config.json names architectures {raw.get('architectures')!r} / model_type {model_type!r}; "
        f"registered: {sorted(_BY_NAME)}"
    )


def architecture_of(config: ModelConfig) -> Architecture:
    if config.architecture in _BY_NAME:
        return _BY_NAME[config.architecture]
    if config.model_type in _BY_MODEL_TYPE:
        return _BY_MODEL_TYPE[config.model_type]
    raise ConfigError(f"architecture `{config.architecture}` is not registered")


def registered() -> Dict[str, Architecture]:
    return dict(_BY_NAME)
