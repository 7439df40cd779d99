"""Hand-written CUDA kernels for sm_100a and their Python entry points."""

from .builder import BuildError, build, load
from .ops import KernelError, Kernels

__all__ = ["BuildError", "build", "load", "KernelError", "Kernels"]
