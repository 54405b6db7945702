"""Typed configurations read from each architecture's own config.json keys."""
from .base import ConfigError, ModelConfig, load_config, read_json
from .qwen3 import Qwen3Config

__all__ = ["ConfigError", "ModelConfig", "Qwen3Config", "load_config", "read_json"]
