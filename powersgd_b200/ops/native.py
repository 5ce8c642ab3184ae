"""Loader for the in-tree native library (`csrc/libpsgd_b200.so`).

The library exports a plain C ABI; every entry point takes raw device pointers and a CUDA
stream handle, so it is called through ctypes with `tensor.data_ptr()` and works under
CUDA-graph capture. Nothing here falls back silently: `lib()` raises if the library is
missing, and callers on a CUDA device treat that as fatal.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

_HERE = os.path.dirname(os.path.abspath(__file__))
# PSGD_B200_LIB points at another build of the same library (e.g. one with development counters)
LIB_PATH = os.environ.get("PSGD_B200_LIB") or os.path.join(os.path.dirname(_HERE), "csrc", "libpsgd_b200.so")

_lib: Optional[ctypes.CDLL] = None
_err: Optional[str] = None


def _try_load() -> None:
    global _lib, _err
    if _lib is not None or _err is not None:
        return
    if not os.path.exists(LIB_PATH):
        _err = f"{LIB_PATH} does not exist"
        return
    try:
        _lib = ctypes.CDLL(LIB_PATH, mode=ctypes.RTLD_GLOBAL)
    except OSError as exc:  # e.g. libcudart missing
        _err = str(exc)
        return
    from . import _signatures

    _signatures.declare(_lib)


def available() -> bool:
    _try_load()
    return _lib is not None


def load_error() -> Optional[str]:
    _try_load()
    return _err


def lib() -> ctypes.CDLL:
    _try_load()
    if _lib is None:
        raise RuntimeError(f"native library not loadable: {_err}")
    return _lib


def use_for_cuda() -> bool:
    """Gate for ops that have a PyTorch restatement: True when the native kernels should run for a
    CUDA tensor. A missing library on a CUDA machine is an error, not a silent slow path, unless
    PSGD_B200_ALLOW_FALLBACK=1 opts into the PyTorch restatement."""
    if available():
        return True
    if os.environ.get("PSGD_B200_ALLOW_FALLBACK", "0") == "1":
        return False
    raise RuntimeError(
        f"powersgd_b200: a CUDA tensor was given but the native sm_100a library is not loadable ({load_error()}); "
        "build it with `python -m powersgd_b200.csrc.build` or set PSGD_B200_ALLOW_FALLBACK=1"
    )


def check(code: int, what: str) -> None:
    if code != 0:
        msg = lib().psgd_last_error()
        raise RuntimeError(f"{what} failed (code {code}): {msg.decode() if msg else ''}")
