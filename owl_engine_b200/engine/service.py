"""EngineService: the engine runs on its own OS thread; clients talk to it through a bounded inbox.

``boot`` builds the engine on the engine thread (the only thread that touches the CUDA context),
then loops: drain the inbox (submit / cancel / query / stop), pump until idle, sleep briefly when
there is nothing to do. ``EngineClient.chat`` returns an iterator of turn events fed by a bounded
per-turn queue (back-pressure). A fatal error ends the loop with ``ServiceExit(kind, code)``:
normal 0, fatal 1, panic 70.

Reference counterpart: ``crates/engine/src/service/{mod,pump,boot,diag}.rs``.
"""
from __future__ import annotations

import queue
import threading
import time
import traceback
from dataclasses import dataclass

from ..utils import log
from .running import RunningEngine, TurnOpts


@dataclass
class ServiceExit:
    kind: str        # normal | fatal | panic
    code: int
    detail: str = ""


class EngineService:
    def __init__(self, build_engine, max_batch: int = 8, on_full: str = "reject", spec_runner=None, running_kw: dict | None = None):
        """``build_engine()`` is called on the engine thread and returns an ``Engine``; ``running_kw`` goes to
        ``RunningEngine`` (session parking for droppable image segments)."""
        self._running_kw = running_kw or {}
        self.inbox: queue.Queue = queue.Queue(maxsize=64)
        self.ready = threading.Event()
        self.exit: ServiceExit | None = None
        self.re: RunningEngine | None = None
        self._args = (build_engine, max_batch, on_full, spec_runner)
        self.thread = threading.Thread(target=self._main, name="owl-engine", daemon=True)
        self.boot_error: str | None = None
        self.idle_checkpoint_s = 5.0

    def boot(self, timeout: float = 600.0) -> "EngineClient":
        self.thread.start()
        if not self.ready.wait(timeout):
            raise TimeoutError("engine did not become ready")
        if self.boot_error:
            raise RuntimeError(self.boot_error)
        return EngineClient(self)

    CHECKPOINT_BEAT = 64 << 20      # bytes written to the disk tier per idle beat
    checkpoint_beats = 0

    def _main(self) -> None:
        build, max_batch, on_full, spec_runner = self._args
        try:
            engine = build()
            # a callable spec_runner is a factory: draft heads need the engine (its runner, weights, pools)
            if callable(spec_runner) and not hasattr(spec_runner, "round"):
                spec_runner = spec_runner(engine)
            ring = getattr(engine, "_ring", None)
            if ring is not None and spec_runner is not None:
                # tensor-parallel leader: speculative rounds are mirrored to the follower ranks as whole calls
                from .tp_serve import MirroredSpec

                spec_runner = MirroredSpec(spec_runner, ring)
            self.re = RunningEngine(engine, max_batch, on_full, spec_runner, **self._running_kw)
        except Exception as ex:
            self.boot_error = f"boot failed: {ex!r}\n{traceback.format_exc()}"
            self.exit = ServiceExit("fatal", 1, self.boot_error)
            self.ready.set()
            return
        self.ready.set()
        idle_since, checkpointed = None, False
        try:
            while True:
                stop = self._drain()
                if stop:
                    self.exit = ServiceExit("normal", 0)
                    return
                if not self.re.pump():
                    # idle: after a quiet spell write the cache through to the disk tier once (restart recall)
                    idle_since = idle_since or time.monotonic()
                    if not checkpointed and self.re.e.disk is not None and time.monotonic() - idle_since > self.idle_checkpoint_s:
                        # one beat of at most CHECKPOINT_BEAT bytes, then back to the inbox: a request that arrives while
                        # the cache is being written waits for a beat, not for the whole cache
                        rep = self.re.e.checkpoint(budget_bytes=self.CHECKPOINT_BEAT)
                        self.checkpoint_beats += 1
                        checkpointed = rep.get("pending", 0) == 0
                    time.sleep(0.0005)
                else:
                    idle_since, checkpointed = None, False
        except MemoryError as ex:
            self.exit = ServiceExit("fatal", 1, repr(ex))
        except Exception as ex:
            log.error("engine.service", traceback.format_exc())
            self.exit = ServiceExit("panic", 70, repr(ex))
        finally:
            try:
                self.re.e.close()             # checkpoint + stop the disk writer (mirrored to the follower ranks)
            except Exception:                 # noqa: BLE001
                log.error("engine.service", traceback.format_exc())
            if hasattr(self.re.e, "shutdown"):
                self.re.e.shutdown()          # tensor-parallel leader: release the follower ranks, whatever ended the loop

    def _drain(self) -> bool:
        while True:
            try:
                msg = self.inbox.get_nowait()
            except queue.Empty:
                return False
            kind = msg[0]
            if kind == "stop":
                return True
            if kind == "submit":
                _, tokens, opts, sink, reply = msg
                try:
                    reply.put(self.re.submit(tokens, opts, sink))
                except ValueError as ex:          # refused at the submit boundary: the caller gets the reason
                    reply.put(ex)
            elif kind == "cancel":
                self.re.cancel_turn(msg[1])
            elif kind == "query":
                _, fn, reply = msg
                try:
                    reply.put(fn(self.re))
                except Exception as ex:
                    reply.put(ex)

    def shutdown(self, timeout: float = 30.0) -> ServiceExit:
        self.inbox.put(("stop",))
        self.thread.join(timeout)
        return self.exit or ServiceExit("fatal", 1, "engine thread did not stop")


class EngineClient:
    def __init__(self, svc: EngineService):
        self.svc = svc

    def chat(self, tokens: list[int], opts: TurnOpts | None = None):
        """Submit a turn; returns (turn_id, event_queue). Events: see ``RunningEngine``."""
        sink: queue.Queue = queue.Queue(maxsize=4096)
        reply: queue.Queue = queue.Queue()
        self.svc.inbox.put(("submit", tokens, opts, sink, reply))
        turn = reply.get(timeout=60)
        if isinstance(turn, Exception):
            raise turn
        return turn, sink

    def cancel(self, turn: int) -> None:
        self.svc.inbox.put(("cancel", turn))

    def query(self, fn, timeout: float = 30.0):
        reply: queue.Queue = queue.Queue()
        self.svc.inbox.put(("query", fn, reply))
        out = reply.get(timeout=timeout)
        if isinstance(out, Exception):
            raise out
        return out

    def queue_facts(self) -> dict:
        return self.query(lambda re: re.queue_facts())
