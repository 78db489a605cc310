"""The CUDA operations of the engine: `kernels` (one function per entry point of
the compiled library), `linear` (the choice of matrix product) and `library`
(building and loading).  Importing this package compiles nothing; the first
operation does."""
from . import kernels
from .library import ExtensionError, KernelError, counters, lib, require_gpu
from .linear import linear, swiglu_product

__all__ = ["kernels", "linear", "swiglu_product", "lib", "require_gpu", "ExtensionError", "KernelError", "counters"]
