from .build import (KernelBuildError, MODULES, compile_module, compile_modules, load_module, is_built,
                    library_path, build_dir)
from .ops import KernelError, PAGE_SIZE

__all__ = ["KernelBuildError", "KernelError", "MODULES", "compile_module", "compile_modules", "load_module",
           "is_built", "library_path", "build_dir", "PAGE_SIZE"]
