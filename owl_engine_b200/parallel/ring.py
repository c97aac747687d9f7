"""Step-descriptor ring: Python face of the native shared-memory broadcast ring (``csrc/host/shm_ring.cpp``).

The leader rank creates the ring and ``push``-es one message per mirrored engine call; every follower rank opens it as
reader ``rank - 1`` and ``pop``-s every message in order. Messages are pickled ``(op, args, kwargs)`` tuples; tensors
travel as raw bytes with their dtype and shape (bf16 as 16-bit words). Nothing here touches a GPU, so the protocol is
tested with plain processes on the CPU.

Reference counterpart: the command channel of ``TpEngine::run`` (``crates/engine/src/parallel/tp.rs:545-734``).
"""
from __future__ import annotations

import ctypes
import pickle
from ctypes import c_char_p, c_int, c_int64, c_uint32, c_uint64, c_void_p

import numpy as np

from .. import _native

_lib = None


class RingClosed(RuntimeError):
    pass


class RingTimeout(RuntimeError):
    pass


def lib():
    global _lib
    if _lib is None:
        l = _native.host()
        l.owl_ring_create.restype = c_void_p
        l.owl_ring_create.argtypes = [c_char_p, c_uint64, c_int]
        l.owl_ring_open.restype = c_void_p
        l.owl_ring_open.argtypes = [c_char_p, c_int, c_int]
        l.owl_ring_push.restype = c_int
        l.owl_ring_push.argtypes = [c_void_p, c_void_p, c_uint32, c_int]
        l.owl_ring_pop.restype = c_int64
        l.owl_ring_pop.argtypes = [c_void_p, c_void_p, c_uint32, c_int, c_void_p]
        l.owl_ring_backlog.restype = c_uint64
        l.owl_ring_backlog.argtypes = [c_void_p]
        l.owl_ring_attached.restype = c_int
        l.owl_ring_attached.argtypes = [c_void_p]
        l.owl_ring_close.argtypes = [c_void_p]
        l.owl_ring_free.argtypes = [c_void_p]
        _lib = l
    return _lib


def ring_name(port: int | str, tag: str = "") -> str:
    """Name of a job's ring: derived from the rendezvous port, so that two jobs on one node never share a ring."""
    return f"/owl_b200_ring_{port}{('_' + tag) if tag else ''}"


# ---- tensors inside messages ---------------------------------------------------------------------------------------
class _Packed:
    """A tensor flattened for the ring: raw bytes + dtype name + shape."""
    __slots__ = ("data", "dtype", "shape")

    def __init__(self, data: bytes, dtype: str, shape: tuple):
        self.data, self.dtype, self.shape = data, dtype, shape


def pack_obj(o):
    """Replace every torch tensor inside lists / tuples / dicts by a ``_Packed`` (CPU bytes)."""
    import torch

    if isinstance(o, torch.Tensor):
        t = o.detach().to("cpu").contiguous()
        if t.dtype == torch.bfloat16:
            return _Packed(t.view(torch.int16).numpy().tobytes(), "bfloat16", tuple(t.shape))
        return _Packed(t.numpy().tobytes(), str(t.dtype).replace("torch.", ""), tuple(t.shape))
    if isinstance(o, (list, tuple)):
        return type(o)(pack_obj(x) for x in o)
    if isinstance(o, dict):
        return {k: pack_obj(v) for k, v in o.items()}
    return o


def unpack_obj(o):
    import torch

    if isinstance(o, _Packed):
        if o.dtype == "bfloat16":
            return torch.from_numpy(np.frombuffer(o.data, dtype=np.int16).copy()).view(torch.bfloat16).reshape(o.shape)
        return torch.from_numpy(np.frombuffer(o.data, dtype=np.dtype(o.dtype)).copy()).reshape(o.shape)
    if isinstance(o, (list, tuple)):
        return type(o)(unpack_obj(x) for x in o)
    if isinstance(o, dict):
        return {k: unpack_obj(v) for k, v in o.items()}
    return o


class StepRing:
    """One end of the ring. ``StepRing.create(name, readers)`` on the leader, ``StepRing.open(name, reader)`` on a follower."""

    def __init__(self, handle, name: str, producer: bool):
        if not handle:
            raise OSError(f"step ring {name}: {'create' if producer else 'open'} failed")
        self.h, self.name, self.producer = handle, name, producer
        self._buf = ctypes.create_string_buffer(1 << 16)

    @classmethod
    def create(cls, name: str, readers: int, capacity: int = 64 << 20) -> "StepRing":
        return cls(lib().owl_ring_create(name.encode(), capacity, readers), name, True)

    @classmethod
    def open(cls, name: str, reader: int, timeout_s: float = 60.0) -> "StepRing":
        return cls(lib().owl_ring_open(name.encode(), reader, int(timeout_s * 1e3)), name, False)

    # -- raw bytes --------------------------------------------------------------------------------------------------
    def push_bytes(self, b: bytes, timeout_s: float = 30.0) -> None:
        rc = lib().owl_ring_push(self.h, b, len(b), int(timeout_s * 1e3))
        if rc == -3:
            raise RingClosed(self.name)
        if rc == -2:
            raise RingTimeout(f"{self.name}: a follower fell {self.backlog()} bytes behind")
        if rc != 0:
            raise ValueError(f"{self.name}: message of {len(b)} bytes does not fit the ring")

    def pop_bytes(self, timeout_s: float | None = None) -> bytes:
        need = c_uint32(0)
        to = -1 if timeout_s is None else int(timeout_s * 1e3)
        while True:
            n = lib().owl_ring_pop(self.h, self._buf, len(self._buf), to, ctypes.byref(need))
            if n >= 0:
                return self._buf.raw[:n]
            if n == -4:
                self._buf = ctypes.create_string_buffer(int(need.value) + 64)
                continue
            if n == -3:
                raise RingClosed(self.name)
            if n == -2:
                raise RingTimeout(self.name)
            raise ValueError(f"{self.name}: pop rejected")

    # -- messages ---------------------------------------------------------------------------------------------------
    def push(self, op: str, *args, **kwargs) -> None:
        self.push_bytes(pickle.dumps((op, pack_obj(args), pack_obj(kwargs)), protocol=5))

    def pop(self, timeout_s: float | None = None):
        op, args, kwargs = pickle.loads(self.pop_bytes(timeout_s))
        return op, unpack_obj(args), unpack_obj(kwargs)

    def backlog(self) -> int:
        return int(lib().owl_ring_backlog(self.h))

    def attached(self) -> int:
        return int(lib().owl_ring_attached(self.h))

    def close(self) -> None:
        if self.h:
            lib().owl_ring_close(self.h)

    def free(self) -> None:
        if self.h:
            lib().owl_ring_free(self.h)
            self.h = None
