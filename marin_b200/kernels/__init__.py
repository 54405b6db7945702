"""Hand-written CUDA kernels for sm_100a, built at first use and called through ctypes."""
from . import build, ops

__all__ = ["build", "ops"]
