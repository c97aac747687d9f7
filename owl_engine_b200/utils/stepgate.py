"""Step gate: slow down or single-step the engine pump at named checkpoints (debugging aid).

``off``: checkpoints cost one attribute read. ``sticky``: every checkpoint sleeps ``ms``.
``single``: a checkpoint blocks until ``step()`` is called (``POST /debug/step``); ``status`` shows
where the pump is parked. Reference counterpart: ``crates/shared/src/stepgate.rs``.
"""
from __future__ import annotations

import threading
import time


class StepGate:
    def __init__(self):
        self.mode = "off"
        self.ms = 50
        self.every = 1
        self._n = 0
        self._cv = threading.Condition()
        self._tokens = 0
        self.parked_at = None

    def configure(self, mode: str = "off", ms: int = 50, every: int = 1) -> None:
        assert mode in ("off", "sticky", "single")
        with self._cv:
            self.mode, self.ms, self.every = mode, ms, max(1, every)
            self._cv.notify_all()

    def checkpoint(self, name: str) -> None:
        if self.mode == "off":
            return
        self._n += 1
        if self._n % self.every:
            return
        if self.mode == "sticky":
            time.sleep(self.ms / 1e3)
            return
        with self._cv:
            self.parked_at = name
            while self.mode == "single" and self._tokens == 0:
                self._cv.wait(timeout=0.25)
            if self._tokens:
                self._tokens -= 1
            self.parked_at = None

    def step(self, n: int = 1) -> None:
        with self._cv:
            self._tokens += n
            self._cv.notify_all()

    def status(self) -> dict:
        return {"mode": self.mode, "ms": self.ms, "every": self.every, "parked_at": self.parked_at}


GATE = StepGate()
