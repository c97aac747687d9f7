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
    """Executes planned page moves on a side stream (device -> host, host -> device).

    Moves are batched: the pages of a plan are packed by one gather kernel (``csrc/kvmove.cu``) into a page-major device
    staging buffer, and every run of consecutive host slots is one ``cudaMemcpyAsync`` (the pinned tier is page-major, so a
    run of slots is one contiguous range); a recall is the mirror image (copies into staging, one scatter kernel). A
    128 k-token context is 8192 pages of 32 slabs each: a quarter of a million per-slab copies become a few dozen."""

    STAGING_PAGES = 64

    def __init__(self, pool, host: HostTier):
        self.pool, self.host = pool, host
        self.stream = torch.cuda.Stream(device=pool.device) if pool.k_pool.is_cuda else None
        self.bytes_out = self.bytes_in = self.copies = 0
        self._staging = None
        self._desc = None

    # -- batched path (GPU) ---------------------------------------------------------------------------------------------
    def _tensors(self):
        ts = [self.pool.k_pool, self.pool.v_pool]
        for sc in (getattr(self.pool, "k_scale", None), getattr(self.pool, "v_scale", None)):
            if sc is not None:
                ts.append(sc)
        return ts

    def _descriptors(self):
        if self._desc is None:
            import ctypes

            ts = self._tensors()
            n = len(ts)
            bases = (ctypes.c_void_p * n)(*[t.data_ptr() for t in ts])
            slabs = [t[0, 0].numel() * t.element_size() for t in ts]
            strides = (ctypes.c_longlong * n)(*[t.shape[1] * sl for t, sl in zip(ts, slabs)])
            self._desc = (bases, strides, (ctypes.c_int * n)(*slabs), n, ts[0].shape[0])
        return self._desc

    def _stage(self, n: int) -> torch.Tensor:
        if self._staging is None:
            from ..utils.ledger import ledger_for

            self._staging = ledger_for(self.pool.device).alloc("kv mover staging", "workspace",
                                                                (self.STAGING_PAGES, self.host.page_bytes), torch.uint8)
        return self._staging[:n]

    def _runs(self, slots):
        """[(index of the first entry, first slot, length)] of maximal runs of consecutive slots inside one host segment."""
        out, i = [], 0
        while i < len(slots):
            j = i + 1
            while j < len(slots) and slots[j] == slots[j - 1] + 1 and slots[j] // self.host.per_seg == slots[i] // self.host.per_seg:
                j += 1
            out.append((i, slots[i], j - i))
            i = j
        return out

    def copy_out_many(self, pages, slots) -> None:
        """Device pages -> host slots (same order). The compute stream's writes to those pages are waited for first."""
        if not len(pages):
            return
        if self.stream is None:
            for pg, sl in zip(pages, slots):
                self.copy_out(pg, sl)
            return
        from ..ops import kernels as K

        bases, strides, slabs, nt, nl = self._descriptors()
        self.stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.stream):
            for c0 in range(0, len(pages), self.STAGING_PAGES):
                pg = list(pages[c0:c0 + self.STAGING_PAGES])
                sl = list(slots[c0:c0 + self.STAGING_PAGES])
                idx = torch.tensor(pg, dtype=torch.int32).pin_memory().to(self.pool.device, non_blocking=True)
                stg = self._stage(len(pg))
                K.call("owl_kv_pages_gather", bases, strides, slabs, nt, nl, K.ptr(idx), len(pg), K.ptr(stg), self.stream.cuda_stream)
                for i0, s0, n in self._runs(sl):
                    seg, off = self.host.segments[s0 // self.host.per_seg], s0 % self.host.per_seg
                    seg[off:off + n].copy_(stg[i0:i0 + n], non_blocking=True)
                    self.copies += 1
                self.bytes_out += len(pg) * self.host.page_bytes

    def copy_in_many(self, slots, pages) -> None:
        """Host slots -> device pages (same order); ``fence`` before the pages are read."""
        if not len(pages):
            return
        if self.stream is None:
            for sl, pg in zip(slots, pages):
                self.copy_in(sl, pg)
            return
        from ..ops import kernels as K

        bases, strides, slabs, nt, nl = self._descriptors()
        with torch.cuda.stream(self.stream):
            for c0 in range(0, len(pages), self.STAGING_PAGES):
                pg = list(pages[c0:c0 + self.STAGING_PAGES])
                sl = list(slots[c0:c0 + self.STAGING_PAGES])
                stg = self._stage(len(pg))
                for i0, s0, n in self._runs(sl):
                    seg, off = self.host.segments[s0 // self.host.per_seg], s0 % self.host.per_seg
                    stg[i0:i0 + n].copy_(seg[off:off + n], non_blocking=True)
                    self.copies += 1
                idx = torch.tensor(pg, dtype=torch.int32).pin_memory().to(self.pool.device, non_blocking=True)
                K.call("owl_kv_pages_scatter", bases, strides, slabs, nt, nl, K.ptr(idx), len(pg), K.ptr(stg), self.stream.cuda_stream)
                self.bytes_in += len(pg) * self.host.page_bytes

    # -- one page at a time (CPU pools in tests, and single promotions) ---------------------------------------------------
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

    def sync(self) -> None:
        """Host-side wait for the moves issued so far (before host slots written by a demotion are read by the CPU)."""
        if self.stream:
            self.stream.synchronize()


class _null:
    def __enter__(self): return self
    def __exit__(self, *a): return False


class DiskTier:
    """Block files named by chain hash (atomic tmp + rename), bounded by ``capacity_bytes``, written by a background thread,
    with a restart index.

    ``spill`` takes a private copy of the block's bytes and returns at once; the writer thread creates the file. A block
    that is recalled before its file exists is served from the pending copy. ``save_index`` waits for the writer and then
    stores what a restarted server needs to rebuild the prefix tree of the files: per block its hash, parent hash, tag and
    tokens (the tokens let the adopter re-derive the hash and refuse a file that does not belong to the chain), and per
    recurrent-state snapshot the prefix hash and length (``.gdn`` files written by ``put_state``).

    Index file ``chain.idx``: ``OWLB2IDX`` | version u32 = 2 | block_tokens u32 | n_blocks u32 | n_states u32 | blocks:
    (hash u64, parent u64, tag u64, n_tok u32, tokens i32[n_tok]) | states: (hash u64, n_tokens u32, bytes u64)."""

    MAGIC = b"OWLB2IDX"
    VERSION = 2

    def __init__(self, directory: str, page_bytes: int, capacity_bytes: int, background: bool = True,
                 state_capacity: int | None = None):
        """``state_capacity``: a budget of its own for the recurrent-state snapshot files (None: they share ``capacity_bytes``
        with the blocks)."""
        import queue
        import threading

        self.state_capacity, self.state_used = state_capacity, 0

        self.dir, self.page_bytes, self.capacity = directory, page_bytes, capacity_bytes
        os.makedirs(directory, exist_ok=True)
        self.index: dict[int, dict] = {}     # hash -> {parent, tag, tokens}
        self.states: dict[int, dict] = {}    # prefix hash -> {n_tokens, bytes}
        self.used = 0
        self.pending: dict = {}              # path -> bytes not yet on disk
        self._lock = threading.Lock()
        self._q: "queue.Queue" = queue.Queue()
        self._thread = None
        self.written = 0
        if background:
            self._thread = threading.Thread(target=self._writer, name="owl-disk-tier", daemon=True)
            self._thread.start()

    # -- writer ---------------------------------------------------------------------------------------------------------
    def _write_file(self, path: str, data: bytes) -> None:
        fd, tmp = tempfile.mkstemp(dir=self.dir, suffix=".tmp")
        with os.fdopen(fd, "wb") as f:
            f.write(data)
        os.replace(tmp, path)
        self.written += 1

    def _writer(self) -> None:
        while True:
            path = self._q.get()
            if path is None:
                self._q.task_done()
                return
            with self._lock:
                data = self.pending.get(path)
            if data is not None:
                try:
                    self._write_file(path, data)
                finally:
                    with self._lock:
                        if self.pending.get(path) is data:
                            del self.pending[path]
            self._q.task_done()

    def _put(self, path: str, data: bytes) -> None:
        if self._thread is None:
            self._write_file(path, data)
            return
        with self._lock:
            self.pending[path] = data
        self._q.put(path)

    def _get(self, path: str) -> np.ndarray:
        with self._lock:
            data = self.pending.get(path)
        if data is not None:
            return np.frombuffer(data, dtype=np.uint8)
        return np.fromfile(path, dtype=np.uint8)

    def flush(self) -> None:
        """Wait until everything handed to the writer is on disk."""
        if self._thread is not None:
            self._q.join()

    def close(self) -> None:
        if self._thread is not None:
            self._q.put(None)
            self._thread.join(10)
            self._thread = None

    # -- blocks ---------------------------------------------------------------------------------------------------------
    def path(self, h: int) -> str:
        return os.path.join(self.dir, f"{h:016x}.kv")

    def state_path(self, h: int) -> str:
        return os.path.join(self.dir, f"{h:016x}.gdn")

    def spill(self, h: int, parent: int, tokens, data: torch.Tensor, tag: int = 0) -> bool:
        if h in self.index:
            return True
        if self.used + self.page_bytes > self.capacity:
            return False
        self._put(self.path(h), data.cpu().numpy().tobytes())
        self.index[h] = {"parent": int(parent), "tag": int(tag), "tokens": [int(t) for t in tokens]}
        self.used += self.page_bytes
        return True

    def fill(self, h: int, out: torch.Tensor) -> None:
        raw = self._get(self.path(h))
        out.copy_(torch.from_numpy(raw.copy()).view_as(out))

    def drop(self, h: int) -> None:
        if h in self.index:
            del self.index[h]
            self.used -= self.page_bytes
            with self._lock:
                self.pending.pop(self.path(h), None)
            try:
                os.unlink(self.path(h))
            except FileNotFoundError:
                pass

    # -- recurrent-state snapshots ------------------------------------------------------------------------------------------
    def put_state(self, h: int, n_tokens: int, data: torch.Tensor) -> bool:
        nb = data.numel() * data.element_size()
        if h in self.states:
            return True
        if self.state_capacity is not None:
            if self.state_used + nb > self.state_capacity:
                return False
            self.state_used += nb
        else:
            if self.used + nb > self.capacity:
                return False
            self.used += nb
        self._put(self.state_path(h), data.cpu().contiguous().view(torch.uint8).numpy().tobytes())
        self.states[h] = {"n_tokens": int(n_tokens), "bytes": nb}
        return True

    def get_state(self, h: int) -> torch.Tensor:
        return torch.from_numpy(self._get(self.state_path(h)).copy())

    def drop_state(self, h: int) -> None:
        st = self.states.pop(h, None)
        if st:
            if self.state_capacity is not None:
                self.state_used -= st["bytes"]
            else:
                self.used -= st["bytes"]
            with self._lock:
                self.pending.pop(self.state_path(h), None)
            try:
                os.unlink(self.state_path(h))
            except FileNotFoundError:
                pass

    # -- restart index ------------------------------------------------------------------------------------------------------
    def save_index(self, block_tokens: int) -> int:
        self.flush()
        fd, tmp = tempfile.mkstemp(dir=self.dir, suffix=".tmp")
        with os.fdopen(fd, "wb") as f:
            f.write(self.MAGIC + struct.pack("<IIII", self.VERSION, block_tokens, len(self.index), len(self.states)))
            for h, rec in self.index.items():
                toks = np.asarray(rec["tokens"], dtype=np.int32)
                f.write(struct.pack("<QQQI", h, rec["parent"], rec.get("tag", 0), len(toks)))
                f.write(toks.tobytes())
            for h, st in self.states.items():
                f.write(struct.pack("<QIQ", h, st["n_tokens"], st["bytes"]))
        os.replace(tmp, os.path.join(self.dir, "chain.idx"))
        return len(self.index)

    def load_index(self) -> int:
        """Read ``chain.idx`` and keep the entries whose files exist. Returns the number of blocks (0 without an index)."""
        p = os.path.join(self.dir, "chain.idx")
        if not os.path.exists(p):
            return 0
        raw = open(p, "rb").read()
        if raw[:8] != self.MAGIC:
            raise ValueError("chain.idx: bad magic")
        ver, self.index_block_tokens, n, ns = struct.unpack_from("<IIII", raw, 8)
        if ver != self.VERSION:
            raise ValueError(f"chain.idx: version {ver}, this build reads {self.VERSION}")
        off = 24
        self.index.clear()
        self.states.clear()
        for _ in range(n):
            h, parent, tag, nt = struct.unpack_from("<QQQI", raw, off)
            off += 28
            toks = np.frombuffer(raw, dtype=np.int32, count=nt, offset=off).tolist()
            off += 4 * nt
            if os.path.exists(self.path(h)):
                self.index[h] = {"parent": parent, "tag": tag, "tokens": toks}
        for _ in range(ns):
            h, ntok, nb = struct.unpack_from("<QIQ", raw, off)
            off += 20
            if os.path.exists(self.state_path(h)) and os.path.getsize(self.state_path(h)) == nb:
                self.states[h] = {"n_tokens": ntok, "bytes": nb}
        state_bytes = sum(s["bytes"] for s in self.states.values())
        if self.state_capacity is not None:
            self.used, self.state_used = len(self.index) * self.page_bytes, state_bytes
        else:
            self.used = len(self.index) * self.page_bytes + state_bytes
        return len(self.index)

    def chain_order(self) -> list[int]:
        """Indexed block hashes with every parent before its children (roots are blocks whose parent is not indexed)."""
        kids: dict = {}
        for h, rec in self.index.items():
            kids.setdefault(rec["parent"], []).append(h)
        order, stack = [], [h for h, rec in self.index.items() if rec["parent"] not in self.index]
        while stack:
            h = stack.pop()
            order.append(h)
            stack.extend(kids.get(h, ()))
        return order
