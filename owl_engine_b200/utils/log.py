"""Logger: levels, tag allow / deny prefixes, tee to a rotating file, runtime-adjustable.

``log.warn("store.evict", "...")``: the first argument is a dotted tag; a record passes when its
level is enabled and its tag matches the allow list (empty = everything) and no deny prefix.
The native libraries report through the same sink via ``emit_native`` (C callers pass level, tag,
message). Reference counterpart: ``crates/shared/src/log.rs`` and ``cu/owl_log.h``.
"""
from __future__ import annotations

import os
import sys
import threading
import time

LEVELS = {"error": 0, "warn": 1, "info": 2, "debug": 3, "trace": 4}


class Logger:
    def __init__(self):
        self.level = LEVELS["warn"]
        self.allow: list[str] = []
        self.deny: list[str] = []
        self.timestamp = False
        self.file = None
        self.path = None
        self.max_bytes = 0
        self.keep = 0
        self.lock = threading.Lock()
        self.ring: list[str] = []
        self.ring_cap = 512

    def configure(self, level="warn", tags_allow=(), tags_deny=(), timestamp=False, path=None, max_mb=0, keep=0):
        self.set_level(level)
        self.allow, self.deny, self.timestamp = list(tags_allow), list(tags_deny), timestamp
        self.max_bytes, self.keep = max_mb << 20, keep
        if path:
            self.path = path
            self.file = open(path, "a", buffering=1)

    def set_level(self, level: str) -> None:
        if level not in LEVELS:
            raise ValueError(f"unknown log level {level!r}")
        self.level = LEVELS[level]

    def set_tags(self, allow: list[str], deny: list[str] | None = None) -> None:
        self.allow, self.deny = list(allow), list(deny or [])

    def enabled(self, level: str, tag: str) -> bool:
        if LEVELS[level] > self.level:
            return False
        if any(tag.startswith(d) for d in self.deny):
            return False
        return not self.allow or any(tag.startswith(a) for a in self.allow)

    def emit(self, level: str, tag: str, msg: str) -> None:
        if not self.enabled(level, tag):
            return
        ts = time.strftime("%H:%M:%S ") if self.timestamp else ""
        line = f"{ts}{level.upper():5s} [{tag}] {msg}"
        with self.lock:
            self.ring.append(line)
            if len(self.ring) > self.ring_cap:
                del self.ring[:len(self.ring) - self.ring_cap]
            print(line, file=sys.stderr)
            if self.file:
                self.file.write(line + "\n")
                if self.max_bytes and self.file.tell() > self.max_bytes:
                    self._rotate()

    def _rotate(self) -> None:
        self.file.close()
        for i in range(self.keep - 1, 0, -1):
            a, b = f"{self.path}.{i}", f"{self.path}.{i + 1}"
            if os.path.exists(a):
                os.replace(a, b)
        if self.keep > 0:
            os.replace(self.path, f"{self.path}.1")
        self.file = open(self.path, "w", buffering=1)

    def tail(self, n: int = 100) -> list[str]:
        return self.ring[-n:]


LOG = Logger()


def error(tag, msg): LOG.emit("error", tag, msg)
def warn(tag, msg): LOG.emit("warn", tag, msg)
def info(tag, msg): LOG.emit("info", tag, msg)
def debug(tag, msg): LOG.emit("debug", tag, msg)
def trace(tag, msg): LOG.emit("trace", tag, msg)


def emit_native(level: int, tag: bytes, msg: bytes) -> None:
    names = ["error", "warn", "info", "debug", "trace"]
    LOG.emit(names[max(0, min(4, level))], tag.decode(errors="replace"), msg.decode(errors="replace"))
