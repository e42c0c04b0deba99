"""Loader of ``liborinfer_core.so`` (C++ policy core; CPU only)."""

from __future__ import annotations

import ctypes
import os
from pathlib import Path

# ORINFER_CORE_LIB: load another build of the core (the sanitizer-instrumented ones)
_PATH = Path(os.environ.get("ORINFER_CORE_LIB") or
             Path(__file__).resolve().parents[1] / "_native" / "liborinfer_core.so")
_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not _PATH.exists():
            from ..ops import build
            build.build_core()
        _lib = ctypes.CDLL(str(_PATH))
        _lib.orinfer_core_last_error.restype = ctypes.c_char_p
    return _lib


def last_error() -> str:
    return lib().orinfer_core_last_error().decode()


class CoreError(ValueError):
    pass
