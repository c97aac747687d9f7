"""A device-client contract and its CPU face with fault / capacity injection.

``DeviceClient`` is the small contract the memory and executor layers need from "a device":
tagged allocation with a ledger, memset, block copies, kernel launch by name, and graph
begin / end / replay. ``CpuFace`` implements it synchronously on host tensors so that engine-level
logic (budgets, eviction, capture fall-backs, error paths) is testable without a GPU, and
``MockLimits`` injects the failures a real device produces:

* ``vram_bytes``     allocations beyond the budget raise ``OutOfMemory`` (capacity planning, pressure relief)
* ``null_kernels``   launches are recorded but compute nothing (scheduling / bookkeeping tests at speed)
* ``graph_capture``  when False, ``graph_begin`` raises ``CaptureUnsupported`` (eager fall-back path)
* ``poison_uninit``  fresh allocations are filled with NaN / 0xFF so reads of unwritten memory surface

Only operations that are legal inside a capture window (launch, alloc from the capture slab, memset,
block copy) are accepted between ``graph_begin`` and ``graph_end``; anything else raises
``CaptureViolation`` -- the same gate the GPU path applies.

Reference counterpart: ``crates/backends/iface/src/contract.rs:429-1218`` (DeviceClient),
``handle.rs:55-722`` (owner / class tagged ledger), ``backends/cpu/src/{face,lib,ops}.rs`` (CPU face,
``MockLimits``), ``backends/cuda/src/server/capture_gate.rs:1-14``.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch


class OutOfMemory(RuntimeError):
    pass


class CaptureUnsupported(RuntimeError):
    pass


class CaptureViolation(RuntimeError):
    pass


@dataclass
class MockLimits:
    vram_bytes: int | None = None
    null_kernels: bool = False
    graph_capture: bool = True
    poison_uninit: bool = False


@dataclass
class Block:
    handle: int
    tensor: torch.Tensor
    owner: str
    klass: str

    @property
    def nbytes(self) -> int:
        return self.tensor.numel() * self.tensor.element_size()


@dataclass
class Graph:
    ops: list = field(default_factory=list)


class CpuFace:
    """Synchronous CPU implementation of the device-client contract."""

    def __init__(self, limits: MockLimits | None = None):
        self.limits = limits or MockLimits()
        self.blocks: dict[int, Block] = {}
        self.kernels: dict[str, callable] = {}
        self.launch_log: list = []
        self._next = 1
        self._capturing: Graph | None = None
        self.used = 0
        self.peak = 0

    # -- memory ---------------------------------------------------------------------------------
    def alloc(self, shape, dtype=torch.float32, *, owner: str = "anon", klass: str = "misc") -> int:
        t = torch.empty(shape, dtype=dtype)
        nbytes = t.numel() * t.element_size()
        if self.limits.vram_bytes is not None and self.used + nbytes > self.limits.vram_bytes:
            raise OutOfMemory(f"{owner}/{klass}: {nbytes} bytes requested, {self.limits.vram_bytes - self.used} free")
        if self.limits.poison_uninit:
            if t.is_floating_point():
                t.fill_(float("nan"))
            else:
                t.view(torch.uint8).fill_(0xFF)
        h = self._next
        self._next += 1
        self.blocks[h] = Block(h, t, owner, klass)
        self.used += nbytes
        self.peak = max(self.peak, self.used)
        return h

    def free(self, h: int) -> None:
        self._no_capture("free")
        self.used -= self.blocks.pop(h).nbytes

    def tensor(self, h: int) -> torch.Tensor:
        return self.blocks[h].tensor

    def ledger(self) -> dict:
        """Bytes by (owner, class): the view the VRAM report is built from."""
        out: dict = {}
        for b in self.blocks.values():
            out[(b.owner, b.klass)] = out.get((b.owner, b.klass), 0) + b.nbytes
        return out

    def memset(self, h: int, value=0) -> None:
        self._do(("memset", h, value), lambda: self.blocks[h].tensor.fill_(value))

    def copy_block(self, src: int, dst: int, n: int | None = None) -> None:
        def run():
            s, d = self.blocks[src].tensor.view(-1), self.blocks[dst].tensor.view(-1)
            k = n if n is not None else min(s.numel(), d.numel())
            d[:k].copy_(s[:k])
        self._do(("copy", src, dst, n), run)

    def upload(self, h: int, data: torch.Tensor) -> None:
        self._no_capture("upload")
        self.blocks[h].tensor.view(-1)[:data.numel()].copy_(data.view(-1))

    def download(self, h: int) -> torch.Tensor:
        self._no_capture("download")
        return self.blocks[h].tensor.clone()

    # -- kernels --------------------------------------------------------------------------------
    def register(self, name: str, fn) -> None:
        self.kernels[name] = fn

    def launch(self, name: str, *handles, **params) -> None:
        if name not in self.kernels:
            raise KeyError(f"unknown kernel {name!r}")
        def run():
            self.launch_log.append(name)
            if not self.limits.null_kernels:
                self.kernels[name](*[self.blocks[h].tensor for h in handles], **params)
        self._do(("launch", name, handles, params), run)

    # -- graphs ---------------------------------------------------------------------------------
    def graph_begin(self) -> None:
        if not self.limits.graph_capture:
            raise CaptureUnsupported("this device does not capture graphs")
        if self._capturing is not None:
            raise CaptureViolation("nested capture")
        self._capturing = Graph()

    def graph_end(self) -> Graph:
        g, self._capturing = self._capturing, None
        if g is None:
            raise CaptureViolation("graph_end without graph_begin")
        return g

    def graph_abort(self) -> None:
        self._capturing = None

    def graph_launch(self, g: Graph) -> None:
        self._no_capture("graph_launch")
        for run in g.ops:
            run()

    # -- internals ------------------------------------------------------------------------------
    def _do(self, what, run) -> None:
        if self._capturing is not None:
            self._capturing.ops.append(run)      # recorded, executed at replay (and once now, as capture warm-up does)
        run()

    def _no_capture(self, op: str) -> None:
        if self._capturing is not None:
            raise CaptureViolation(f"{op} is not allowed inside a capture window")
