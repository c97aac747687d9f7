"""Minimal safetensors reader / writer (no dependency on the ``safetensors`` package).

File = u64 header length, JSON header {name: {dtype, shape, data_offsets}}, raw little-endian data.
Tensors are served as zero-copy views of an ``np.memmap`` (bf16 / fp8 are reinterpreted through
torch). A model directory may be a single file or shards listed in ``*.safetensors.index.json``.

Reference counterpart: ``crates/models/src/formats/{mmap_index,safetensors}.rs``.
"""
from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np
import torch

_DT = {"F32": (np.float32, torch.float32), "F16": (np.float16, torch.float16), "BF16": (np.uint16, torch.bfloat16),
       "I32": (np.int32, torch.int32), "I64": (np.int64, torch.int64), "I8": (np.int8, torch.int8),
       "U8": (np.uint8, torch.uint8), "I16": (np.int16, torch.int16), "F8_E4M3": (np.uint8, torch.float8_e4m3fn),
       "BOOL": (np.bool_, torch.bool), "F64": (np.float64, torch.float64)}
_REV = {v[1]: k for k, v in _DT.items()}


class SafeFile:
    def __init__(self, path: str | Path):
        """Read the header and memory-map the data. A truncated or damaged file is refused with a ``ValueError`` naming it:
        a header length beyond the file, a header that is not a JSON object, an entry with an unknown dtype, a shape that does
        not match its byte range, a byte range outside the file."""
        self.path = Path(path)
        size = self.path.stat().st_size
        try:
            with open(self.path, "rb") as f:
                (n,) = struct.unpack("<Q", f.read(8))
                if n > size - 8:
                    raise ValueError(f"header length {n} exceeds the file ({size} bytes)")
                self.header = json.loads(f.read(n))
            if not isinstance(self.header, dict):
                raise ValueError("the header is not a JSON object")
            self.base = 8 + n
            self.meta = self.header.pop("__metadata__", {})
            for k, info in self.header.items():
                if not isinstance(info, dict) or not isinstance(info.get("dtype"), str):
                    raise ValueError(f"tensor {k!r}: malformed entry")
                shape, off = info.get("shape"), info.get("data_offsets")
                if not isinstance(shape, list) or not all(isinstance(d, int) and d >= 0 for d in shape) or \
                        not isinstance(off, list) or len(off) != 2 or not all(isinstance(o, int) for o in off):
                    raise ValueError(f"tensor {k!r}: malformed shape / data_offsets")
                numel = 1
                for d in shape:
                    numel *= d
                lo, hi = off
                if not (0 <= lo <= hi <= size - self.base):
                    raise ValueError(f"tensor {k!r}: byte range {off} lies outside the file")
                # a dtype this reader does not decode (a newer format) is only an error when that tensor is asked for
                if info["dtype"] in _DT and hi - lo != numel * np.dtype(_DT[info["dtype"]][0]).itemsize:
                    raise ValueError(f"tensor {k!r}: byte range {off} does not fit its shape {shape}")
        except (struct.error, UnicodeDecodeError, json.JSONDecodeError, AttributeError, TypeError) as e:
            raise ValueError(f"{self.path}: truncated or corrupted safetensors header ({type(e).__name__}: {e})") from None
        except ValueError as e:
            raise ValueError(f"{self.path}: {e}") from None
        self.mm = np.memmap(self.path, dtype=np.uint8, mode="r") if size > self.base else np.zeros(0, dtype=np.uint8)

    def keys(self):
        return self.header.keys()

    def get(self, name: str) -> torch.Tensor:
        info = self.header[name]
        if info["dtype"] not in _DT:
            raise ValueError(f"{self.path}: tensor {name!r} has dtype {info['dtype']}, which this reader does not decode")
        npdt, tdt = _DT[info["dtype"]]
        lo, hi = info["data_offsets"]
        raw = self.mm[self.base + lo:self.base + hi]
        arr = np.frombuffer(raw, dtype=npdt).reshape(info["shape"])
        t = torch.from_numpy(arr.copy() if not arr.flags.writeable else arr)
        return t.view(tdt) if t.dtype != tdt else t


class SafeDir:
    """All tensors of a HF-style checkpoint directory (single file or sharded)."""

    def __init__(self, path: str | Path):
        p = Path(path)
        self.files: dict[str, SafeFile] = {}
        self.where: dict[str, str] = {}
        idx = list(p.glob("*.safetensors.index.json"))
        if p.is_file():
            shards = [p]
        elif idx:
            wm = json.loads(idx[0].read_text())["weight_map"]
            shards = sorted({p / f for f in wm.values()})
        else:
            shards = sorted(p.glob("*.safetensors"))
        if not shards:
            raise FileNotFoundError(f"no safetensors under {p}")
        for s in shards:
            sf = SafeFile(s)
            self.files[s.name] = sf
            for k in sf.keys():
                self.where[k] = s.name

    def keys(self):
        return self.where.keys()

    def __contains__(self, k):
        return k in self.where

    def get(self, name: str) -> torch.Tensor:
        return self.files[self.where[name]].get(name)


def save_file(tensors: dict, path: str | Path, metadata: dict | None = None) -> None:
    header, blobs, off = {}, [], 0
    for k, t in tensors.items():
        t = t.detach().cpu().contiguous()
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.dtype in (torch.bfloat16, torch.float8_e4m3fn) \
            else t.numpy().tobytes()                  # reshape first: a 0-dimensional tensor cannot be viewed as bytes
        header[k] = {"dtype": _REV[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    if metadata:
        header["__metadata__"] = metadata
    hj = json.dumps(header).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj)
        for b in blobs:
            f.write(b)
