from . import ops
from .build import KernelBuildError, compile_library, compile_many, load_library
from .ops import KernelError

__all__ = ["KernelBuildError", "KernelError", "compile_library", "compile_many", "load_library", "ops"]
