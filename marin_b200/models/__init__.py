"""Architectures known to the engine.  Importing this package registers them."""
from . import qwen3  # noqa: F401  (registration)
from .model import Model
from .registry import Architecture, architecture_for, architecture_of, register_architecture, registered

__all__ = ["Model", "Architecture", "architecture_for", "architecture_of", "register_architecture", "registered"]
