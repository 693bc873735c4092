"""tenzo_b200 — B200 (sm_100a) CUDA implementation of Tenzo's quantized decode path.

The product is ``lib/libtenzo_runtime.so``: hand-written CUDA kernels, a resident decode engine
and the C ABI of ``include/tenzo.h`` (+ ``tenzo_ext.h``, ``tenzo_kernels.h``). This Python package
is a thin ctypes layer over that library for tests and benchmarks; it adds no arithmetic and has
no CPU path — loading fails loudly if the library was not built.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

from . import abi

__all__ = ["load_library", "library_path", "abi"]

_PKG = Path(__file__).resolve().parent
_lib = None


def library_path() -> Path:
    return _PKG / "lib" / "libtenzo_runtime.so"


def load_library(build_if_missing: bool = True):
    """dlopen libtenzo_runtime.so and declare every prototype. Raises if it cannot be loaded."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if not path.exists():
        if not build_if_missing:
            raise RuntimeError(f"{path} is missing: run `python -m tenzo_b200.build` (there is no CPU fallback)")
        from .build import build
        build()
    L = C.CDLL(str(path), mode=os.RTLD_GLOBAL)
    abi.declare_tenzo_abi(L)
    abi.declare_ext_abi(L)
    abi.declare_kernel_abi(L)
    _lib = L
    return L
