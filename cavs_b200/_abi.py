"""ctypes binding of libcavs_b200.so.  The library must be present and must load:
there is no Python or CPU fallback for anything it provides."""
from __future__ import annotations

import ctypes
import re
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libcavs_b200.so"
HEADER = PKG.parent / "include" / "cavs_b200.h"

_lib = None


class CavsError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"cavs_b200 status {status}: {message}")
        self.status = status


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m cavs_b200.build` (needs nvcc); "
                "cavs_b200 has no fallback implementation")
        _lib = ctypes.CDLL(str(LIB_PATH))
        _lib.cavs_last_error.restype = ctypes.c_char_p
        _lib.cavs_status_string.restype = ctypes.c_char_p
        _lib.cavs_build_info.restype = ctypes.c_char_p
    return _lib


def check(status: int) -> None:
    if status != 0:
        raise CavsError(status, lib().cavs_last_error().decode())


def declared_symbols() -> list[str]:
    """Every entry point include/cavs_b200.h declares."""
    text = HEADER.read_text()
    return sorted(set(re.findall(r"CAVS_API[^;(]*?\b(cavs_\w+)\s*\(", text)))


def ptr(a):
    """Host numpy array or raw int address -> c_void_p."""
    if a is None:
        return ctypes.c_void_p(0)
    if isinstance(a, int):
        return ctypes.c_void_p(a)
    return ctypes.c_void_p(a.ctypes.data)
