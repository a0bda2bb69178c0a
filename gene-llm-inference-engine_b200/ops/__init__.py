from . import kernels
from .build import BuildError, build, library_path
from .library import KernelError, lib

__all__ = ["kernels", "BuildError", "build", "library_path", "KernelError", "lib"]
