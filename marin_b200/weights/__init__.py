"""Safetensors by tensor name, and the random-weights mode."""
from .loader import Checkpoint, WeightError, check, load_tensors
from .random_init import random_tensor, random_tensors, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors

__all__ = ["Checkpoint", "WeightError", "check", "load_tensors", "random_tensor", "random_tensors",
           "write_random_model", "SafetensorsError", "SafetensorsFile", "write_safetensors"]
