"""The CUDA kernels of the library, as Python functions."""
from . import library, ops

__all__ = ["library", "ops"]
