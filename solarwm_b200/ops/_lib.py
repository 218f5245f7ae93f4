"""ctypes binding of the in-tree native library ``_native/libsolar_b200.so``.

The library is plain C ABI: every entry point takes raw device pointers, sizes and a
CUDA stream handle and returns 0 on success (the message of the last failure is
available through ``solar_last_error``).  On a machine with a GPU the CUDA path of every
op is mandatory: a missing or unloadable library raises instead of silently falling back
to PyTorch, so a green GPU test always means the native code ran.
"""
from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent.parent / "_native" / "libsolar_b200.so"
_lock = threading.Lock()
_lib = None

# Incremented by the Python wrappers each time a native kernel is launched; tests use it to
# assert that the fused path (not a PyTorch fallback) ran, and bench.py reports the total.
COUNTERS: dict[str, int] = {}


def count(name: str, n: int = 1) -> None:
    COUNTERS[name] = COUNTERS.get(name, 0) + n


def total_launches() -> int:
    """Launches of this library's own kernels (``library_*`` counters are excluded)."""
    return sum(v for k, v in COUNTERS.items() if not k.startswith("library_"))


def reset_counters() -> None:
    COUNTERS.clear()


class NativeError(RuntimeError):
    pass


def lib_path() -> Path:
    return _LIB_PATH


def available() -> bool:
    return _LIB_PATH.exists()


def load():
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not _LIB_PATH.exists():
            if os.environ.get("SOLAR_B200_AUTOBUILD", "1") == "1":
                from .. import build as _build

                _build.build_all()
            if not _LIB_PATH.exists():
                raise NativeError(
                    f"native library missing: {_LIB_PATH}; run `python -m solarwm_b200.build`"
                )
        lib = ctypes.CDLL(str(_LIB_PATH))
        lib.solar_last_error.restype = ctypes.c_char_p
        _lib = lib
        return lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = load().solar_last_error()
        raise NativeError(f"{what} failed (rc={rc}): {msg.decode() if msg else ''}")


def ptr(t):
    """Device (or host) address of a tensor's first element, or NULL for None."""
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def stream_handle():
    import torch

    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


c_int = ctypes.c_int
c_ll = ctypes.c_longlong
c_float = ctypes.c_float
