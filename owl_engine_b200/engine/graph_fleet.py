"""The graph fleet: every step graph a serving engine will replay, captured at boot and metered into the memory ledger.

Without it a graph is captured by the first request that needs its shape: that request pays tens of milliseconds of capture
inside its latency, and the memory a graph pins (its private pool of intermediates) appears in no budget. ``GraphFleet`` lists
the shapes a profile can reach --

    decode      (b, 1)          b = 1 .. max_batch, per context bucket
    verify      (1, d + 1)      one sequence, d drafts            (speculative decoding)
    batch spec  (b, d + 1)      b = 2 .. spec_rows sequences
    fold        d + 1 rows      replay of the accepted prefix after a rejection; batched fold for (b, d + 1)

-- captures them in that order and records what each one cost: the device memory that the capture left allocated (metering
by the allocator's counter around the capture) and the time it took. The bytes go into the ledger under class ``graphs`` by
name (``graph.decode.b4.ctx2048``), so ``/debug/vram`` accounts for them and a profile whose graphs do not fit its declared
budget is refused at boot by the ledger rather than failing on some later request. A plan entry is in one of three states:
``eager`` (graphs are switched off, or capture is not possible on this face: the step runs its kernels directly), ``planned``
(listed, not captured yet) and ``captured``.

Reference counterpart: ``crates/engine/src/graph/graph_plan.rs:1-35`` (tri-state plan with warm-up metering),
``graph/graph_fleet.rs:49-83, 266`` (session graph + per-depth verify / fold / propose + batch graph; ``assemble``).
"""
from __future__ import annotations

import time
from dataclasses import dataclass

import torch


@dataclass
class FleetEntry:
    kind: str               # "decode" | "verify" | "batch_spec" | "fold" | "fold_batch"
    b: int
    t: int
    ctx: int
    state: str = "planned"  # "planned" | "captured" | "eager"
    bytes: int = 0
    ms: float = 0.0
    error: str | None = None

    @property
    def name(self) -> str:
        base = f"graph.{self.kind}.b{self.b}" + (f".t{self.t}" if self.t > 1 else "")
        return base + (f".ctx{self.ctx}" if self.ctx else "")


class GraphFleet:
    def __init__(self, engine, max_batch: int = 8, spec_depths: tuple = (), spec_rows: int = 1, ctx_buckets: tuple = (2048,)):
        self.e = engine
        self.entries: list[FleetEntry] = []
        max_rows = engine.runner.MAX_ROWS
        for ctx in ctx_buckets:
            for b in range(1, max(1, max_batch) + 1):
                self.entries.append(FleetEntry("decode", b, 1, ctx))
            for d in spec_depths:
                t = d + 1
                self.entries.append(FleetEntry("verify", 1, t, ctx))
                for b in range(2, max(1, spec_rows) + 1):
                    if b * t <= max_rows:
                        self.entries.append(FleetEntry("batch_spec", b, t, ctx))
        for d in spec_depths:
            t = d + 1
            self.entries.append(FleetEntry("fold", 1, t, 0))
            for b in range(2, max(1, spec_rows) + 1):
                if b * t <= max_rows:
                    self.entries.append(FleetEntry("fold_batch", b, t, 0))

    def _allocated(self) -> int:
        dev = self.e.device
        return torch.cuda.memory_allocated(dev) if dev.type == "cuda" else 0

    def _capture(self, en: FleetEntry) -> None:
        r = self.e.runner
        if en.kind in ("decode", "verify", "batch_spec"):
            r.capture(en.b, en.t, ctx_hint=en.ctx)
        elif en.kind == "fold":
            r.capture_fold(en.t)
        else:
            r.capture_fold_batch(en.b, en.t)

    def assemble(self, stop_on_budget: bool = True) -> dict:
        """Capture every planned entry. Returns the report (also kept in ``self.report``)."""
        from ..utils.ledger import BudgetError

        led, r = self.e.ledger, self.e.runner
        eager = not getattr(r, "use_graphs", True)
        if any(en.kind != "decode" for en in self.entries):
            # speculative steps keep every GDN layer's inputs for the fold and use row-count-independent arithmetic; both
            # switches re-point buffers (and would drop graphs captured before them), so they come first
            if hasattr(r, "enable_gdn_save"):
                r.enable_gdn_save()
            r.uniform_rows = True
        for en in self.entries:
            if en.state != "planned":
                continue
            if en.kind.startswith("fold") and not hasattr(r, "capture_fold"):
                en.state = "eager"
                continue
            before, t0 = self._allocated(), time.perf_counter()
            try:
                self._capture(en)
            except Exception as ex:   # noqa: BLE001  (a face that cannot capture: the step stays eager and says why)
                en.state, en.error = "eager", repr(ex)
                continue
            if self.e.device.type == "cuda":
                torch.cuda.synchronize(self.e.device)
            en.ms = (time.perf_counter() - t0) * 1e3
            en.bytes = max(0, self._allocated() - before)
            en.state = "eager" if eager else "captured"
            if en.bytes:
                try:
                    led.check(en.name, en.bytes)           # an enforcing ledger refuses a fleet that outgrows the declared budget
                except BudgetError:
                    if stop_on_budget:
                        raise
                led.track(en.name, "graphs", en.bytes)
        self.report = self.facts()
        return self.report

    def facts(self) -> dict:
        by_state: dict = {}
        for en in self.entries:
            by_state[en.state] = by_state.get(en.state, 0) + 1
        return {"entries": [{"name": en.name, "state": en.state, "bytes": en.bytes, "ms": round(en.ms, 2),
                             **({"error": en.error} if en.error else {})} for en in self.entries],
                "states": by_state, "bytes": sum(en.bytes for en in self.entries),
                "capture_ms": round(sum(en.ms for en in self.entries), 1)}
