"""KV tiers below the device pool: pinned host RAM, then disk, plus the restart index.

``HostTier`` is a fixed number of page-sized slots in pinned host memory (allocated in segments);
device<->host moves are ``cudaMemcpyAsync`` on a side stream, one copy per (layer, K/V) slab of a
page, issued by ``copy_out`` / ``copy_in`` and fenced with an event before the pages are reused.
``DiskTier`` stores one file per block (tmp + rename, content-addressed by chain hash) and keeps a
``ChainIndex`` file so a restarted server can rebuild the prefix tree of what is on disk.

Reference counterpart: ``crates/store/src/{host,disk,disk_index,tier}.rs``,
``crates/engine/src/mem/{disk_runtime,disk_io}.rs`` and the swap commands of the CUDA backend.
"""
from __future__ import annotations

import os
import struct
import tempfile

import numpy as np
import torch


class HostTier:
    def __init__(self, page_bytes: int, capacity_bytes: int, pin: bool = True, segment_bytes: int = 256 << 20):
        self.page_bytes = page_bytes
        self.n_slots = max(0, capacity_bytes // page_bytes)
        per_seg = max(1, segment_bytes // page_bytes)
        self.segments = []
        left = self.n_slots
        while left > 0:
            n = min(per_seg, left)
            t = torch.empty(n, page_bytes, dtype=torch.uint8)
            if pin and torch.cuda.is_available():
                t = t.pin_memory()
            self.segments.append(t)
            left -= n
        self.per_seg = per_seg
        self.free = list(range(self.n_slots - 1, -1, -1))

    def slot(self, i: int) -> torch.Tensor:
        return self.segments[i // self.per_seg][i % self.per_seg]

    def alloc(self) -> int | None:
        return self.free.pop() if self.free else None

    def release(self, i: int) -> None:
        self.free.append(i)

    @property
    def used(self) -> int:
        return self.n_slots - len(self.free)


def page_views(pool, page: int):
    """The device slabs of one KV page as byte views: k_pool[:, page], v_pool[:, page] and, for the int8 pool, the
    page's scale slabs."""
    views = [t[:, page].reshape(t.shape[0], -1) for t in (pool.k_pool, pool.v_pool)]
    views = [v if v.dtype == torch.uint8 else v.view(torch.uint8) for v in views]          # 16-bit pool: fp16 words as bytes
    for sc in (getattr(pool, "k_scale", None), getattr(pool, "v_scale", None)):
        if sc is not None:
            views.append(sc[:, page].reshape(sc.shape[0], -1).view(torch.uint8))
    return views


def page_bytes(pool) -> int:
    return int(sum(v.numel() for v in page_views(pool, 0)))


class Mover:
    """Executes planned page moves on a side stream (device -> host, host -> device)."""

    def __init__(self, pool, host: HostTier):
        self.pool, self.host = pool, host
        self.stream = torch.cuda.Stream(device=pool.device) if pool.k_pool.is_cuda else None
        self.bytes_out = self.bytes_in = 0

    def copy_out(self, page: int, slot: int) -> None:
        dst = self.host.slot(slot)
        ctx = torch.cuda.stream(self.stream) if self.stream else _null()
        with ctx:
            if self.stream:
                self.stream.wait_stream(torch.cuda.current_stream())
            off = 0
            for v in page_views(self.pool, page):
                dst[off:off + v.numel()].view_as(v).copy_(v, non_blocking=True)
                off += v.numel()
        self.bytes_out += off

    def copy_in(self, slot: int, page: int) -> None:
        src = self.host.slot(slot)
        ctx = torch.cuda.stream(self.stream) if self.stream else _null()
        with ctx:
            off = 0
            for v in page_views(self.pool, page):
                v.copy_(src[off:off + v.numel()].view_as(v), non_blocking=True)
                off += v.numel()
        self.bytes_in += off

    def fence(self) -> None:
        """Make the compute stream wait for all moves issued so far (call before pages are reused)."""
        if self.stream:
            torch.cuda.current_stream().wait_stream(self.stream)


class _null:
    def __enter__(self): return self
    def __exit__(self, *a): return False


class DiskTier:
    """One file per block, named by chain hash; atomic tmp + rename; bounded by ``capacity_bytes``."""

    MAGIC = b"OWLB2IDX"

    def __init__(self, directory: str, page_bytes: int, capacity_bytes: int):
        self.dir, self.page_bytes, self.capacity = directory, page_bytes, capacity_bytes
        os.makedirs(directory, exist_ok=True)
        self.index: dict[int, dict] = {}     # hash -> {parent, tokens}
        self.used = 0

    def path(self, h: int) -> str:
        return os.path.join(self.dir, f"{h:016x}.kv")

    def spill(self, h: int, parent: int, tokens, data: torch.Tensor) -> bool:
        if self.used + self.page_bytes > self.capacity:
            return False
        fd, tmp = tempfile.mkstemp(dir=self.dir, suffix=".tmp")
        with os.fdopen(fd, "wb") as f:
            f.write(data.cpu().numpy().tobytes())
        os.replace(tmp, self.path(h))
        self.index[h] = {"parent": parent, "tokens": list(map(int, tokens))}
        self.used += self.page_bytes
        return True

    def fill(self, h: int, out: torch.Tensor) -> None:
        raw = np.fromfile(self.path(h), dtype=np.uint8)
        out.copy_(torch.from_numpy(raw).view_as(out))

    def drop(self, h: int) -> None:
        if h in self.index:
            del self.index[h]
            self.used -= self.page_bytes
            try:
                os.unlink(self.path(h))
            except FileNotFoundError:
                pass

    # -- restart index: magic | block_tokens u32 | n u32 | n x (hash u64, parent u64, tokens i32[block]) ------
    def save_index(self, block_tokens: int) -> None:
        fd, tmp = tempfile.mkstemp(dir=self.dir, suffix=".tmp")
        with os.fdopen(fd, "wb") as f:
            f.write(self.MAGIC + struct.pack("<II", block_tokens, len(self.index)))
            for h, rec in self.index.items():
                f.write(struct.pack("<QQ", h, rec["parent"]))
                f.write(np.asarray(rec["tokens"], dtype=np.int32).tobytes())
        os.replace(tmp, os.path.join(self.dir, "chain.idx"))

    def load_index(self) -> int:
        p = os.path.join(self.dir, "chain.idx")
        if not os.path.exists(p):
            return 0
        raw = open(p, "rb").read()
        if raw[:8] != self.MAGIC:
            raise ValueError("chain.idx: bad magic")
        bt, n = struct.unpack_from("<II", raw, 8)
        off = 16
        self.index.clear()
        for _ in range(n):
            h, parent = struct.unpack_from("<QQ", raw, off)
            off += 16
            toks = np.frombuffer(raw, dtype=np.int32, count=bt, offset=off).tolist()
            off += 4 * bt
            if os.path.exists(self.path(h)):
                self.index[h] = {"parent": parent, "tokens": toks}
        self.used = len(self.index) * self.page_bytes
        return len(self.index)
