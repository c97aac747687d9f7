"""ctypes loader for the in-tree native libraries.

``cuda()`` returns the sm_100a kernel library, ``host()`` the C++ host runtime. Both are
built by ``owl_engine_b200/_native/build.py`` (``python -m owl_engine_b200._native.build``)
and live next to this file so a snapshot of the tree carries them.

Ops never fall back silently: on a CUDA tensor a missing library raises ``NativeMissing``.
"""
from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

HERE = Path(__file__).resolve().parent
_lock = threading.Lock()
_cuda = None
_host = None


class NativeMissing(RuntimeError):
    pass


class NativeError(RuntimeError):
    pass


def _load(name: str, builder: str):
    path = HERE / name
    if not path.exists():
        if os.environ.get("OWL_B200_NO_AUTOBUILD"):
            raise NativeMissing(f"{path} is missing; run python -m owl_engine_b200._native.build")
        from . import build as _b

        getattr(_b, builder)()
    if not path.exists():
        raise NativeMissing(f"{path} is missing and could not be built")
    return ctypes.CDLL(str(path))


def cuda():
    global _cuda
    if _cuda is None:
        with _lock:
            if _cuda is None:
                _cuda = _load("libowl_b200_cuda.so", "build_cuda")
    return _cuda


def host():
    global _host
    if _host is None:
        with _lock:
            if _host is None:
                _host = _load("libowl_b200_host.so", "build_host")
    return _host


def check(rc: int, what: str) -> None:
    """Launchers return 0, a negative host-side code, or -2000-cudaError."""
    if rc == 0:
        return
    if rc == -1:
        raise NativeError(f"{what}: rejected arguments (shape / alignment)")
    if rc <= -2000:
        raise NativeError(f"{what}: CUDA launch error {-(rc + 2000)}")
    raise NativeError(f"{what}: native error {rc}")


def loaded_libraries() -> list[str]:
    out = []
    if _cuda is not None:
        out.append(str(HERE / "libowl_b200_cuda.so"))
    if _host is not None:
        out.append(str(HERE / "libowl_b200_host.so"))
    return out
