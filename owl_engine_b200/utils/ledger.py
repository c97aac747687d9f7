"""Device-memory ledger: one object per GPU owns the declared budget and every named allocation.

``V_avail = total * vram_budget - reserve``. Everything this package places in device memory is either allocated through
``DeviceLedger.alloc`` (budget checked first, refusal is a ``BudgetError`` that names the request and what is left) or
recorded with ``track`` / ``track_tree`` right after a loader produced it (weights arrive as finished tensors). Entries
carry a class (``weights``, ``resident copies``, ``kv pool``, ``gdn state``, ``workspace``, ``graphs``, ``symmetric``,
``draft``), so ``view()`` can show mutually exclusive buckets that close to what the driver reports:

    used (driver) = sum of tracked classes + allocator slack (reserved - allocated by torch) + untracked torch tensors
                    + outside torch (CUDA context, libraries, NCCL, symmetric VMM mappings not tracked)

The last two lines are measured, not guessed, and ``closes`` says whether the unexplained part stays within
``slack_bytes``. No native launcher allocates: kernels that need scratch get it from a ledger entry.

A process without a declared budget (tests, the benchmark) uses the default ledger of its device, which records
everything and refuses nothing.

Reference counterpart: the tagged allocation ledger of the device handle (``crates/backends/iface/src/handle.rs:55-722``)
and the server's VRAM view (``apps/server/src/vram_ledger.rs``).
"""
from __future__ import annotations

import threading
from dataclasses import dataclass

import torch


class BudgetError(RuntimeError):
    pass


@dataclass
class Entry:
    name: str
    klass: str
    nbytes: int
    storage: int = 0     # address of the backing storage (entries that share one are counted once)


class DeviceLedger:
    def __init__(self, device, total_bytes: int | None = None, budget_frac: float = 1.0, reserve_bytes: int = 0,
                 enforce: bool = False, slack_bytes: int = 2 << 30):
        self.device = torch.device(device)
        self.total = total_bytes
        self.budget_frac, self.reserve, self.enforce, self.slack = budget_frac, reserve_bytes, enforce, slack_bytes
        self.entries: dict[str, Entry] = {}
        self._storages: dict[int, str] = {}
        self._lock = threading.Lock()
        self.refused = 0

    # -- budget ---------------------------------------------------------------------------------------------------------
    def _total(self) -> int:
        if self.total is None:
            if self.device.type == "cuda":
                self.total = torch.cuda.mem_get_info(self.device)[1]
            else:
                self.total = 1 << 62
        return self.total

    @property
    def avail(self) -> int:
        """Bytes this process may use on the device."""
        return int(self._total() * self.budget_frac) - self.reserve

    def used(self) -> int:
        return sum(e.nbytes for e in self.entries.values())

    def room(self) -> int:
        return self.avail - self.used()

    def check(self, name: str, nbytes: int) -> None:
        """Refuse (when enforcing) a request that does not fit what is left of the declared budget."""
        if self.enforce and nbytes > self.room():
            self.refused += 1
            raise BudgetError(f"{name}: {nbytes / 2**20:.1f} MiB requested, {max(0, self.room()) / 2**20:.1f} MiB left of the "
                              f"declared budget ({self.avail / 2**30:.2f} GiB = {self.budget_frac:.2f} x "
                              f"{self._total() / 2**30:.1f} GiB - {self.reserve / 2**20:.0f} MiB reserve); "
                              f"largest classes: {self._top()}")

    def _top(self) -> str:
        b = sorted(self.by_class().items(), key=lambda kv: -kv[1])[:3]
        return ", ".join(f"{k} {v / 2**30:.2f} GiB" for k, v in b)

    # -- recording --------------------------------------------------------------------------------------------------------
    def alloc(self, name: str, klass: str, shape, dtype, zero: bool = False) -> torch.Tensor:
        n = 1
        for s in (shape if isinstance(shape, (tuple, list)) else (shape,)):
            n *= int(s)
        nbytes = n * torch.empty(0, dtype=dtype).element_size()
        self.check(name, nbytes)
        t = (torch.zeros if zero else torch.empty)(shape, dtype=dtype, device=self.device)
        self.track(name, klass, t)
        return t

    def track(self, name: str, klass: str, what) -> None:
        """Record an existing tensor (or a byte count). A tensor whose storage is already recorded is not counted twice."""
        with self._lock:
            if isinstance(what, torch.Tensor):
                if what.device.type != self.device.type:
                    return
                st = what.untyped_storage()
                key = st.data_ptr()
                if key in self._storages and self._storages[key] in self.entries:
                    return
                nm = self._unique(name)
                self.entries[nm] = Entry(nm, klass, st.nbytes(), key)
                self._storages[key] = nm
            else:
                nm = self._unique(name)
                self.entries[nm] = Entry(nm, klass, int(what))

    def _unique(self, name: str) -> str:
        if name not in self.entries:
            return name
        i = 2
        while f"{name}#{i}" in self.entries:
            i += 1
        return f"{name}#{i}"

    def track_tree(self, prefix: str, klass: str, obj, _seen=None, _depth: int = 0) -> int:
        """Record every tensor reachable from ``obj`` (attributes, dict values, list / tuple items). Returns the bytes
        newly recorded."""
        if _seen is None:
            _seen = set()
        if id(obj) in _seen or _depth > 6:
            return 0
        _seen.add(id(obj))
        before = self.used()
        if isinstance(obj, torch.Tensor):
            self.track(prefix, klass, obj)
        elif isinstance(obj, dict):
            for k, v in obj.items():
                self.track_tree(f"{prefix}.{k}", klass, v, _seen, _depth + 1)
        elif isinstance(obj, (list, tuple)):
            for i, v in enumerate(obj):
                self.track_tree(f"{prefix}[{i}]", klass, v, _seen, _depth + 1)
        elif hasattr(obj, "__dict__") and not isinstance(obj, (type, torch.cuda.Stream, torch.cuda.CUDAGraph)):
            for k, v in vars(obj).items():
                if not k.startswith("__") and not callable(v):
                    self.track_tree(f"{prefix}.{k}", klass, v, _seen, _depth + 1)
        return self.used() - before

    def release(self, name: str) -> None:
        with self._lock:
            e = self.entries.pop(name, None)
            if e is not None and e.storage:
                self._storages.pop(e.storage, None)

    def release_prefix(self, prefix: str) -> None:
        for n in [n for n in self.entries if n.startswith(prefix)]:
            self.release(n)

    # -- views ------------------------------------------------------------------------------------------------------------
    def by_class(self) -> dict:
        out: dict = {}
        for e in self.entries.values():
            out[e.klass] = out.get(e.klass, 0) + e.nbytes
        return out

    def largest(self, n: int = 12) -> list:
        return [(e.name, e.klass, e.nbytes) for e in sorted(self.entries.values(), key=lambda e: -e.nbytes)[:n]]

    def view(self) -> dict:
        """Buckets that sum to the device total, with the measured residuals named."""
        b = dict(self.by_class())
        tracked = sum(b.values())
        if self.device.type == "cuda":
            free, total = torch.cuda.mem_get_info(self.device)
            reserved = torch.cuda.memory_reserved(self.device)
            allocated = torch.cuda.memory_allocated(self.device)
        else:
            free, total, reserved, allocated = self._total() - tracked, self._total(), tracked, tracked
        used = total - free
        tracked_torch = sum(e.nbytes for e in self.entries.values() if e.klass != "symmetric")
        b["allocator slack (reserved by torch, not in use)"] = max(0, reserved - allocated)
        b["untracked tensors (transients, library workspaces)"] = max(0, allocated - tracked_torch)
        outside = used - reserved - (tracked - tracked_torch)
        b["outside torch (context, libraries, other processes)"] = max(0, outside)
        b["free"] = free
        unexplained = total - sum(b.values())
        return {"total": total, "budget": self.avail if self.enforce else None, "tracked": tracked, "buckets": b,
                "unexplained": unexplained, "closes": abs(unexplained) <= self.slack and b[
                    "untracked tensors (transients, library workspaces)"] <= self.slack,
                "largest": self.largest(), "refused": self.refused}


_LEDGERS: dict[str, DeviceLedger] = {}


def ledger_for(device) -> DeviceLedger:
    """The ledger of a device (created on first use: records everything, enforces nothing)."""
    key = str(torch.device(device))
    if key == "cuda":
        key = f"cuda:{torch.cuda.current_device()}"
    led = _LEDGERS.get(key)
    if led is None:
        led = _LEDGERS[key] = DeviceLedger(key)
    return led


def install(ledger: DeviceLedger) -> DeviceLedger:
    """Make ``ledger`` the ledger of its device (the server installs an enforcing one built from ``[store]``)."""
    key = str(ledger.device)
    if key == "cuda":
        key = f"cuda:{torch.cuda.current_device()}"
    _LEDGERS[key] = ledger
    return ledger
