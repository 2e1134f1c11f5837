"""CUDA sources for sm_100a, their build, and their Python bindings."""

from .bindings import KernelError, Kernels, load_kernels
from .build import BuildError, build_all, build_library

__all__ = ["KernelError", "Kernels", "load_kernels", "BuildError", "build_all", "build_library"]
