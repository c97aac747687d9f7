"""Metrics store: timers with call-tree parents, counters, events; runtime levels.

Levels: ``off`` (nothing recorded), ``counters``, ``host`` (timers on the host clock), ``gpu``
(additionally CUDA-event timers around captured regions). Timers nest strictly (LIFO); the parent
tag of a timer is whatever timer was open when it started, which yields a call tree for
``/debug/perf``. Dumps as JSON or CSV (``--perf-dump``).

Reference counterpart: ``crates/shared/src/metrics.rs`` (``timer_start!/timer_end!``, counters).
"""
from __future__ import annotations

import csv
import io
import json
import threading
import time
from contextlib import contextmanager

LEVELS = {"off": 0, "counters": 1, "host": 2, "gpu": 3}


class Metrics:
    def __init__(self):
        self.level = LEVELS["host"]
        self.lock = threading.Lock()
        self.timers: dict = {}      # tag -> [count, total_s, max_s, parent]
        self.counters: dict = {}
        self.events: list = []
        self._stack = threading.local()
        self.epoch = 0

    def set_level(self, name: str) -> None:
        self.level = LEVELS[name]

    def count(self, tag: str, n: int = 1) -> None:
        if self.level >= 1:
            with self.lock:
                self.counters[tag] = self.counters.get(tag, 0) + n

    def event(self, tag: str, **kv) -> None:
        if self.level >= 1:
            with self.lock:
                self.events.append({"t": time.time(), "tag": tag, **kv})
                if len(self.events) > 4096:
                    del self.events[:1024]

    @contextmanager
    def timer(self, tag: str):
        if self.level < 2:
            yield
            return
        st = getattr(self._stack, "s", None)
        if st is None:
            st = self._stack.s = []
        parent = st[-1] if st else ""
        st.append(tag)
        t0 = time.perf_counter()
        try:
            yield
        finally:
            dt = time.perf_counter() - t0
            top = st.pop()
            assert top == tag, f"timer nesting violated: closing {tag} while {top} is open"
            with self.lock:
                rec = self.timers.setdefault(tag, [0, 0.0, 0.0, parent])
                rec[0] += 1
                rec[1] += dt
                rec[2] = max(rec[2], dt)

    def snapshot(self, prefix: str = "") -> dict:
        with self.lock:
            return {"epoch": self.epoch,
                    "timers": {k: {"n": v[0], "total_ms": v[1] * 1e3, "max_ms": v[2] * 1e3, "parent": v[3]}
                               for k, v in self.timers.items() if k.startswith(prefix)},
                    "counters": {k: v for k, v in self.counters.items() if k.startswith(prefix)}}

    def tree(self) -> dict:
        snap = self.snapshot()["timers"]
        kids: dict = {}
        for k, v in snap.items():
            kids.setdefault(v["parent"], []).append(k)

        def build(tag):
            return {"tag": tag, **snap.get(tag, {}), "children": [build(c) for c in sorted(kids.get(tag, []))]}
        return {"roots": [build(c) for c in sorted(kids.get("", []))]}

    def reset(self) -> None:
        with self.lock:
            self.timers.clear(); self.counters.clear(); self.events.clear()
            self.epoch += 1

    def dump_json(self) -> str:
        return json.dumps(self.snapshot(), indent=1)

    def dump_csv(self) -> str:
        buf = io.StringIO()
        w = csv.writer(buf)
        w.writerow(["kind", "tag", "n", "total_ms", "max_ms", "parent"])
        snap = self.snapshot()
        for k, v in sorted(snap["timers"].items()):
            w.writerow(["timer", k, v["n"], f"{v['total_ms']:.3f}", f"{v['max_ms']:.3f}", v["parent"]])
        for k, v in sorted(snap["counters"].items()):
            w.writerow(["counter", k, v, "", "", ""])
        return buf.getvalue()


METRICS = Metrics()
