"""Memory contract: the declared budget, the boot-time plan, grants, admission and pressure.

``V_avail = total * vram_budget - reserve``; the ``MemoryPlan`` splits it into named, mutually
exclusive buckets (weights, GDN rows, workspace, KV pool) and refuses to boot when they do not fit.
Every runtime allocation is recorded in the ``Ledger`` under an owner and class so ``/debug/vram``
can show buckets that close to the driver's total. ``check_admission`` decides Admit / Hold /
Reject for a new turn from its token need; ``PressurePolicy`` turns pool occupancy into an
eviction target (start relieving at the low watermark of free pages, free up to the high one);
``plan_capacity`` cascades GPU -> host -> disk -> drop.

Reference counterpart: ``crates/store/src/{budget,plan,reservations,pressure,policy,hooks}.rs``,
``crates/backends/iface/src/handle.rs`` (alloc ledger), ``apps/server/src/vram_ledger.rs``.
"""
from __future__ import annotations

from dataclasses import dataclass, field


class BudgetError(RuntimeError):
    pass


@dataclass
class Ledger:
    entries: dict = field(default_factory=dict)    # name -> (class, bytes)

    def record(self, name: str, klass: str, nbytes: int) -> None:
        self.entries[name] = (klass, int(nbytes))

    def release(self, name: str) -> None:
        self.entries.pop(name, None)

    def total(self) -> int:
        return sum(b for _, b in self.entries.values())

    def by_class(self) -> dict:
        out: dict = {}
        for k, b in self.entries.values():
            out[k] = out.get(k, 0) + b
        return out

    def view(self, driver_total: int, driver_free: int) -> dict:
        """Mutually exclusive buckets that sum to the driver's total."""
        b = self.by_class()
        used = driver_total - driver_free
        tracked = sum(b.values())
        b["untracked (context, allocator slack, other processes)"] = max(0, used - tracked)
        b["free"] = driver_free
        return {"total": driver_total, "buckets": b, "closes": sum(b.values()) == driver_total or used < tracked}


@dataclass
class MemoryPlan:
    total: int
    budget_frac: float
    reserve: int
    weights: int
    gdn_rows: int
    workspace: int
    page_bytes: int

    @property
    def avail(self) -> int:
        return int(self.total * self.budget_frac) - self.reserve

    @property
    def kv_pool(self) -> int:
        return self.avail - self.weights - self.gdn_rows - self.workspace

    @property
    def kv_pages(self) -> int:
        return max(0, self.kv_pool // self.page_bytes)

    def check(self, min_pages: int = 64) -> None:
        if self.kv_pages < min_pages:
            raise BudgetError(f"declared budget too small: {self.avail / 2**30:.1f} GiB available, weights "
                              f"{self.weights / 2**30:.1f} + state {self.gdn_rows / 2**30:.1f} + workspace "
                              f"{self.workspace / 2**30:.1f} GiB leave {self.kv_pages} KV pages (< {min_pages})")


@dataclass
class Grant:
    turn: int
    pages: int


class Reservations:
    """Pages promised to admitted turns (so two admitted turns cannot both count the same room)."""

    def __init__(self):
        self.grants: dict[int, Grant] = {}

    def reserve(self, turn: int, pages: int) -> None:
        self.grants[turn] = Grant(turn, pages)

    def consume(self, turn: int, pages: int) -> None:
        g = self.grants.get(turn)
        if g:
            g.pages = max(0, g.pages - pages)

    def release(self, turn: int) -> None:
        self.grants.pop(turn, None)

    @property
    def outstanding(self) -> int:
        return sum(g.pages for g in self.grants.values())


ADMIT, HOLD, REJECT = "admit", "hold", "reject"


def check_admission(need_pages: int, free_pages: int, evictable_pages: int, outstanding: int, pool_pages: int,
                    free_slots: int, on_full: str = "reject") -> str:
    """A turn is admitted when its pages fit in free + evictable room not promised to others."""
    if need_pages > pool_pages:
        return REJECT                      # can never fit
    if free_slots <= 0:
        return HOLD if on_full.startswith("queue") else REJECT
    if need_pages <= free_pages + evictable_pages - outstanding:
        return ADMIT
    return HOLD if on_full.startswith("queue") else REJECT


@dataclass
class Admission:
    """An admission verdict a client can act on: why a turn was not admitted and when trying again makes sense."""
    verdict: str                 # ADMIT | HOLD | REJECT
    reason: str = ""             # "" | "never_fits" | "slots" | "memory" | "queue_timeout"
    retry_after_ms: int = 0      # 0: retrying the same request cannot help


def decide_admission(need_pages: int, free_pages: int, evictable_pages: int, outstanding: int, pool_pages: int, free_slots: int,
                     on_full: str = "reject", waited_ms: float = 0.0, eta_ms: float = 1000.0) -> Admission:
    """``check_admission`` with the reason and a retry hint. ``on_full``: ``"reject"`` refuses at once, ``"queue"`` holds the
    turn until room appears, ``"queue:<ms>"`` holds it for at most that long (``waited_ms`` = how long it has been held) and
    then rejects with ``queue_timeout``. ``eta_ms``: the caller's estimate of when a running turn will have finished."""
    if need_pages > pool_pages:
        return Admission(REJECT, "never_fits", 0)
    reason = "slots" if free_slots <= 0 else ("" if need_pages <= free_pages + evictable_pages - outstanding else "memory")
    if not reason:
        return Admission(ADMIT)
    retry = int(max(100.0, min(eta_ms, 30000.0)))
    if on_full.startswith("queue"):
        limit = float(on_full[6:]) if on_full.startswith("queue:") else None
        if limit is None or waited_ms < limit:
            return Admission(HOLD, reason, retry)
        return Admission(REJECT, "queue_timeout", retry)
    return Admission(REJECT, reason, retry)


@dataclass
class PressurePolicy:
    low: float = 0.12      # start relieving when free pages fall below 12 % of the pool
    high: float = 0.25     # and free up to 25 %

    def target(self, free_pages: int, pool_pages: int) -> int:
        """Number of pages to free now (0 when above the low watermark)."""
        if free_pages >= self.low * pool_pages:
            return 0
        return int(self.high * pool_pages) - free_pages


@dataclass
class Verdict:
    evict_pages: int
    sink: str              # "host" | "disk" | "drop"
    satisfied: bool


def plan_capacity(need: int, free_pages: int, evictable: int, host_free: int, disk_free: int) -> Verdict:
    """Need-driven eviction: how many pages to push out and where they go (GPU -> host -> disk -> drop)."""
    short = need - free_pages
    if short <= 0:
        return Verdict(0, "none", True)
    n = min(short, evictable)
    sink = "host" if host_free >= n else "disk" if disk_free >= n else "drop"
    return Verdict(n, sink, n >= short)


def lrfu_score(last_use: int, hits: int, now: int, lam: float = 0.05) -> float:
    """LRFU combined recency/frequency value (higher = keep)."""
    return hits * (0.5 ** (lam * max(0, now - last_use)))
