"""HTTP/1.1 server (asyncio streams, keep-alive, chunked SSE) and the route table.

Routes: ``POST /v1/chat/completions`` (JSON or SSE), ``GET /health``, ``GET /v1/models``,
``POST /tokenize``, and the ``/debug/*`` family (queue, log, step, vram, blocks, agent, launches,
metrics, perf, load). A client that disconnects mid-stream (write failure or EOF on the socket)
cancels its turn at the next step boundary; a queued turn gets SSE comment frames as keep-alive and
a 503 after ``queue_timeout_ms``; same-``session`` requests are serialised.

Reference counterpart: ``apps/server/src/{http,main,debug,agent_trace,load}.rs``.
"""
from __future__ import annotations

import asyncio
import collections
import json
import os
import queue as pyqueue
import threading
import time

from ..engine.running import TurnOpts
from ..engine.sampler import SamplingParams
from ..engine.tokenizer import StreamDecoder
from ..utils import log
from ..utils.log import LOG
from ..utils.metrics import METRICS
from ..utils.stepgate import GATE
from .chat_tpl import ChatTemplate
from .openai import BadRequest, ChatRequest, Streamer
from .toolcall import RepeatGuard

REASONS = {200: "OK", 400: "Bad Request", 404: "Not Found", 405: "Method Not Allowed", 413: "Content Too Large", 429: "Too Many Requests",
           503: "Service Unavailable", 500: "Internal Server Error"}


class App:
    MAX_BODY = 512 << 20        # a request body (images travel as data URLs) may not be larger than this

    def __init__(self, client, tokenizer, model_name: str, template: ChatTemplate | None = None,
                 default_sampling: SamplingParams | None = None, default_max_new: int = 4096, max_new_cap: int = 32768,
                 queue_timeout_ms: int = 30000, keepalive_ms: int = 15000, max_concurrent: int = 8, vision=None,
                 request_dump_dir: str = "", prompt_dump: bool = False, raw_completion: bool = False):
        self.client, self.tok, self.model = client, tokenizer, model_name
        self.tpl = template or ChatTemplate()
        self.default_sampling = default_sampling or SamplingParams()
        self.default_max_new, self.max_new_cap = default_max_new, max_new_cap
        self.queue_timeout, self.keepalive = queue_timeout_ms / 1e3, keepalive_ms / 1e3
        self.permits = asyncio.Semaphore(max_concurrent)
        self.session_locks: dict[str, asyncio.Lock] = {}
        self.guard = RepeatGuard()
        self.vision = vision      # Vision (tower + image cache + pad token id) or None: image parts are then refused
        # debugging aids: every request body as a file; the rendered prompt and the undivided completion text in the log
        self.request_dump_dir, self.prompt_dump, self.raw_completion = request_dump_dir, prompt_dump, raw_completion
        self._dump_seq = 0
        if request_dump_dir:
            os.makedirs(request_dump_dir, exist_ok=True)
        self.started = time.time()
        self.stop = threading.Event()
        self.agent_trace: collections.deque = collections.deque(maxlen=64)   # per turn: the output splitter's structural trace

    # -- plumbing -------------------------------------------------------------------------------
    async def handle(self, reader: asyncio.StreamReader, writer: asyncio.StreamWriter) -> None:
        try:
            while True:
                line = await reader.readline()
                if not line:
                    break
                try:
                    method, target, _ = line.decode("latin1").split(" ", 2)
                except ValueError:
                    await self._send(writer, 400, {"error": "malformed request line"})
                    break
                headers = {}
                while True:
                    h = await reader.readline()
                    if h in (b"\r\n", b"\n", b""):
                        break
                    k, _, v = h.decode("latin1").partition(":")
                    headers[k.strip().lower()] = v.strip()
                try:
                    n_body = int(headers.get("content-length") or 0)
                except ValueError:
                    n_body = -1
                if n_body < 0 or n_body > self.MAX_BODY:
                    await self._send(writer, 400 if n_body < 0 else 413,
                                     {"error": {"message": "bad Content-Length" if n_body < 0 else f"body larger than {self.MAX_BODY} bytes",
                                                "type": "invalid_request_error"}})
                    break
                body = await reader.readexactly(n_body) if n_body else b""
                keep = headers.get("connection", "keep-alive").lower() != "close"
                await self.route(method, target.split("?")[0], body, reader, writer)
                if not keep:
                    break
        except (ConnectionError, asyncio.IncompleteReadError):
            pass
        finally:
            try:
                writer.close()
            except Exception:
                pass

    async def _send(self, w, status: int, obj, ctype="application/json", headers: dict | None = None) -> None:
        data = obj if isinstance(obj, bytes) else (json.dumps(obj, ensure_ascii=False).encode() if not isinstance(obj, str) else obj.encode())
        extra = "".join(f"{k}: {v}\r\n" for k, v in (headers or {}).items())
        w.write(f"HTTP/1.1 {status} {REASONS.get(status, '')}\r\nContent-Type: {ctype}\r\nContent-Length: {len(data)}\r\n"
                f"{extra}Connection: keep-alive\r\n\r\n".encode() + data)
        await w.drain()

    async def _sse_open(self, w) -> None:
        w.write(b"HTTP/1.1 200 OK\r\nContent-Type: text/event-stream\r\nCache-Control: no-cache\r\n"
                b"Transfer-Encoding: chunked\r\nConnection: keep-alive\r\n\r\n")
        await w.drain()

    @staticmethod
    async def _sse(w, payload: str) -> None:
        data = payload.encode()
        w.write(f"{len(data):x}\r\n".encode() + data + b"\r\n")
        await w.drain()

    # -- routes ---------------------------------------------------------------------------------
    async def route(self, method, path, body, reader, writer) -> None:
        try:
            if path == "/v1/chat/completions" and method == "POST":
                return await self.chat(body, reader, writer)
            if path == "/health":
                return await self._send(writer, 200, {"status": "ok", "uptime_s": round(time.time() - self.started, 1)})
            if path == "/v1/models":
                return await self._send(writer, 200, {"object": "list", "data": [{"id": self.model, "object": "model"}]})
            if path == "/tokenize" and method == "POST":
                try:
                    d = json.loads(body or b"{}")
                    if not isinstance(d, dict):
                        raise ValueError("the body must be an object")
                    text = d.get("text") if "text" in d else self.tpl.render(d.get("messages", []), tools=d.get("tools"))
                    if not isinstance(text, str):
                        raise ValueError("text must be a string")
                except BadRequest:
                    raise
                except Exception as e:   # noqa: BLE001
                    raise BadRequest(f"cannot tokenize this body: {e!r}") from None
                ids = self.tok.encode(text)
                return await self._send(writer, 200, {"tokens": ids, "count": len(ids)})
            if path.startswith("/debug/"):
                return await self.debug(method, path[len("/debug/"):], body, writer)
            await self._send(writer, 404, {"error": f"no route {method} {path}"})
        except BadRequest as e:
            await self._send(writer, 400, {"error": {"message": str(e), "type": "invalid_request_error"}})
        except (ConnectionError, asyncio.IncompleteReadError):
            raise
        except Exception as e:
            log.error("server.route", repr(e))
            await self._send(writer, 500, {"error": {"message": repr(e), "type": "server_error"}})

    async def debug(self, method, sub, body, w) -> None:
        parts = sub.split("/")
        q = self.client.query
        if parts[0] == "queue":
            return await self._send(w, 200, self.client.queue_facts())
        if parts[0] == "metrics":
            return await self._send(w, 200, METRICS.snapshot("/".join(parts[1:])))
        if parts[0] == "perf":
            if parts[1:] == ["reset"]:
                METRICS.reset()
            return await self._send(w, 200, METRICS.tree())
        if parts[0] == "log":
            if len(parts) >= 3 and parts[1] == "level" and method == "POST":
                try:
                    LOG.set_level(parts[2])
                except ValueError as e:
                    raise BadRequest(str(e)) from None
            elif len(parts) >= 3 and parts[1] == "tags" and method == "POST":
                LOG.set_tags([t for t in parts[2].split(",") if t])
            return await self._send(w, 200, {"level": LOG.level, "tags_allow": LOG.allow, "tail": LOG.tail(100)})
        if parts[0] == "step":
            if method == "POST":
                try:
                    d = json.loads(body or b"{}")
                    if not isinstance(d, dict):
                        raise ValueError("the body must be an object")
                    if "mode" in d:
                        if d["mode"] not in ("off", "sticky", "single"):
                            raise ValueError("mode must be off | sticky | single")
                        GATE.configure(d["mode"], int(d.get("ms", GATE.ms)), int(d.get("every", 1)))
                    else:
                        GATE.step(int(d.get("n", 1)))
                except (ValueError, TypeError, UnicodeDecodeError) as e:
                    raise BadRequest(f"/debug/step: {e}") from None
            return await self._send(w, 200, GATE.status())
        if parts[0] == "vram":
            return await self._send(w, 200, q(lambda re: _vram(re)))
        if parts[0] == "blocks":
            return await self._send(w, 200, q(lambda re: {"kv": re.e.kv.stats(), "free_rows": len(re.e.states.free_rows),
                                                           "snapshots": len(re.e.states.snaps),
                                                           "host_used": re.e.host.used if re.e.host else 0,
                                                           "recall": {"last": getattr(re.e, "last_recall", {}),
                                                                      "modes": getattr(re.e, "recall_modes", {})}}))
        if parts[0] == "agent":
            if parts[1:] == ["clear"] and method == "POST":
                q(lambda re: re.trace.clear())
            if parts[1:] == ["clear"] and method == "POST":
                self.agent_trace.clear()
            n = int(parts[1]) if len(parts) > 1 and parts[1].isdigit() else 64
            if parts[1:2] == ["splitter"]:
                return await self._send(w, 200, list(self.agent_trace)[-n:])
            return await self._send(w, 200, q(lambda re: re.trace[-n:]))
        if parts[0] == "launches":
            n = int(parts[1]) if len(parts) > 1 and parts[1].isdigit() else 256
            from ..ops import kernels as K

            return await self._send(w, 200, q(lambda re: {"graphs": [list(k) for k in re.e.runner.graphs.keys()],
                                                           "fleet": re.e.graph_fleet.facts() if getattr(re.e, "graph_fleet", None) else None,
                                                           "graph_manifest": re.e.runner.graph_manifest() if hasattr(re.e.runner, "graph_manifest") else [],
                                                           "launches": K.recent_launches(n), "status": K.all_status()}))
        if parts[0] == "shutdown" and method == "POST":
            # orderly stop (tests, supervisors): the listener loop sees the flag, the engine thread checkpoints and exits
            self.stop.set()
            return await self._send(w, 200, {"stopping": True})
        if parts[0] == "load" and method == "POST":
            return await self._send(w, 200, {"loaded": self.model})
        await self._send(w, 404, {"error": "unknown debug endpoint"})

    def vision_wrap(self) -> tuple:
        """Token ids of the markers the chat template writes around an image placeholder (None when the tokenizer has
        no single token for them)."""
        if getattr(self, "_vwrap", None) is None:
            ids = []
            for text in ("<|vision_start|>", "<|vision_end|>"):
                e = self.tok.encode(text)
                ids.append(e[0] if len(e) == 1 else None)
            self._vwrap = tuple(ids) if None not in ids else (None, None)
        return self._vwrap

    def _dump_request(self, body: bytes) -> None:
        """One file per request body, named by arrival time and a counter (bodies hold user data and image data URLs:
        the directory is the operator's responsibility)."""
        self._dump_seq += 1
        path = os.path.join(self.request_dump_dir, f"{int(time.time() * 1e3):013d}-{self._dump_seq:06d}.json")
        try:
            with open(path, "wb") as f:
                f.write(body)
        except OSError as ex:
            log.warn("server.dump", f"cannot write {path}: {ex}")

    async def chat(self, body, reader, w) -> None:
        if self.request_dump_dir:
            self._dump_request(body)
        req = ChatRequest.parse(body)
        kwargs = dict(req.chat_template_kwargs)
        if req.reasoning_effort in ("none", "minimal"):
            kwargs.setdefault("enable_thinking", False)
        try:
            prompt = self.tpl.render(req.messages, tools=req.tools, **kwargs)
        except BadRequest:
            raise
        except Exception as e:   # noqa: BLE001  (a template cannot be told apart from its input here: the request gets the blame)
            raise BadRequest(f"the chat template could not render these messages: {e!r}") from None
        ids = self.tok.encode(prompt)
        if self.prompt_dump:
            log.LOG.emit("warn", "server.prompt", f"{len(ids)} tokens: {prompt!r}")
        images, evict_spans = [], []
        if req.images:
            if self.vision is None:
                raise BadRequest("this server was started without a vision tower; image parts are not accepted")
            loop0 = asyncio.get_running_loop()
            try:
                ids, images, evict_spans = await loop0.run_in_executor(
                    None, self.vision.expand, ids, [im["data"] for im in req.images], [im["evict"] for im in req.images],
                    self.vision_wrap())
            except ValueError as e:          # bytes that are not an image this server decodes: the client's fault, not ours
                raise BadRequest(f"image cannot be decoded: {e}") from None
        max_new = min(req.max_tokens or self.default_max_new, self.max_new_cap)
        opts = TurnOpts(max_new=max_new, ignore_eos=req.ignore_eos, sampling=req.sampling(self.default_sampling),
                        eos_ids=tuple(self.tok.eos_ids), session=req.session, images=images,
                        image_pad_id=self.vision.pad_id if self.vision else None, evict_spans=evict_spans)
        lock = self.session_locks.setdefault(req.session, asyncio.Lock()) if req.session else None
        try:
            await asyncio.wait_for(self.permits.acquire(), self.queue_timeout)
        except asyncio.TimeoutError:
            return await self._send(w, 503, {"error": {"message": "server busy (queue timeout)", "type": "overloaded"}})
        if lock:
            await lock.acquire()
        turn = None
        try:
            loop = asyncio.get_running_loop()
            try:
                turn, sink = await loop.run_in_executor(None, self.client.chat, ids, opts)
            except ValueError as e:              # refused at the submit boundary (e.g. droppable marks with image_evict off)
                raise BadRequest(str(e)) from None
            streamer = Streamer(self.model, StreamDecoder(self.tok), req.stop,
                                start_in_think=prompt.rstrip().endswith("<think>"), tools=req.tools)
            if req.stream:
                await self._sse_open(w)
            last_io, t_submit = time.time(), time.time()
            raw_ids: list = []
            reason, usage = "stop", {"prompt_tokens": len(ids), "completion_tokens": 0}
            while True:
                try:
                    ev = await loop.run_in_executor(None, sink.get, True, 0.25)
                except pyqueue.Empty:
                    if reader.at_eof():
                        raise ConnectionError("client closed")
                    if req.stream and time.time() - last_io > self.keepalive:
                        await self._sse(w, ": keep-alive\n\n")
                        last_io = time.time()
                    continue
                if ev[0] == "token":
                    if self.raw_completion:
                        raw_ids.append(ev[2])
                    chunks = streamer.on_token(ev[2])
                    if req.stream:
                        for c in chunks:
                            await self._sse(w, "data: " + json.dumps(c, ensure_ascii=False) + "\n\n")
                            last_io = time.time()
                    if streamer.stopped:
                        self.client.cancel(turn)
                elif ev[0] == "completed":
                    reason, usage = ("stop" if ev[2] in ("stop", "cancelled") else ev[2]), ev[3]
                    break
                elif ev[0] == "failed":
                    if req.stream:
                        await self._sse(w, "data: " + json.dumps({"error": {"message": ev[2]}}) + "\n\n")
                        await self._sse(w, "data: [DONE]\n\n")
                        w.write(b"0\r\n\r\n")
                        return await w.drain()
                    if "rejected" in ev[2]:
                        # an admission refusal the client can act on: why, and when to try again
                        import re as _re

                        m = _re.search(r"rejected \((\w+)\).*retry_after_ms=(\d+)", ev[2])
                        reason, retry = (m.group(1), int(m.group(2))) if m else ("memory", 1000)
                        hdr = {"Retry-After": str(max(1, -(-retry // 1000)))} if retry else {}
                        return await self._send(w, 429, {"error": {"message": ev[2], "type": "overloaded", "code": reason,
                                                                   "retry_after_ms": retry}}, headers=hdr)
                    return await self._send(w, 500, {"error": {"message": ev[2], "type": "engine_error"}})
            for c in streamer.tool_calls:
                if req.session and self.guard.observe(req.session, c):
                    log.warn("server.repeat", f"session {req.session}: identical tool call repeated")
            if req.stream:
                for c in streamer.finish(reason, usage, req.include_usage):
                    await self._sse(w, "data: " + json.dumps(c, ensure_ascii=False) + "\n\n")
                await self._sse(w, "data: [DONE]\n\n")
                w.write(b"0\r\n\r\n")
                await w.drain()
            else:
                streamer.drain()
                await self._send(w, 200, streamer.full_response(reason, usage))
            if self.raw_completion:
                # what the model wrote before the thinking / tool-call splitter divided it, special tokens included
                log.LOG.emit("warn", "server.raw", f"{streamer.id}: {self.tok.decode(raw_ids)!r}")
            sp = streamer.splitter
            self.agent_trace.append({"id": streamer.id, "session": req.session, "tool_calls": sp.n_calls, "malformed": sp.malformed,
                                     "strays": sp.strays, "reasoning_tokens": sp.reasoning_steps, "trace": sp.trace()})
            for m in streamer.malformed:
                log.warn("server.toolcall", f"{streamer.id}: malformed tool block ({m['kind']}, {len(m['raw'])} B): {m['raw'][:2048]!r}")
            METRICS.event("server.turn", ms=(time.time() - t_submit) * 1e3, tokens=usage["completion_tokens"])
        except (ConnectionError, asyncio.IncompleteReadError):
            if turn is not None:
                self.client.cancel(turn)       # client went away: stop generating at the next step boundary
            raise
        finally:
            if lock:
                lock.release()
                # an idle session keeps no lock object: nobody holds it and nobody waits for it
                if not lock.locked() and not getattr(lock, "_waiters", None) and self.session_locks.get(req.session) is lock:
                    del self.session_locks[req.session]
            self.permits.release()


class Vision:
    """Server-side image path: decode -> vision tower (cached by content) -> expand the single image-pad token the
    chat template wrote per image into as many pad tokens as the image has merged patches."""

    def __init__(self, tower, pad_id: int, cache_cap: int = 8):
        from ..cli import png
        from ..models.vision import ImageCache

        self.tower, self.pad_id, self.cache, self.decode = tower, pad_id, ImageCache(cache_cap), png.decode_png

    def expand(self, ids: list[int], blobs: list[bytes], evict: list | None = None, wrap: tuple = (None, None)):
        """Returns the expanded ids, the image triples and, for the images whose ``evict`` entry is true, the token spans a
        client may later drop: the pad run together with the vision-start / vision-end tokens (``wrap``) around it when
        they are there, i.e. exactly what disappears from the rendered prompt when the image part is removed."""
        images, out, spans, k = [], [], [], 0
        for j, t in enumerate(ids):
            if t == self.pad_id and k < len(blobs):
                emb, grid, fp = self.cache.get(self.tower, blobs[k], self.decode)
                images.append((emb, grid, fp))
                lo = len(out)
                out.extend([self.pad_id] * emb.shape[0])
                if evict and evict[k]:
                    hi = len(out)
                    if wrap[0] is not None and j > 0 and ids[j - 1] == wrap[0] and j + 1 < len(ids) and ids[j + 1] == wrap[1]:
                        lo, hi = lo - 1, hi + 1
                    spans.append((lo, hi))
                k += 1
            else:
                out.append(t)
        if k != len(blobs):
            raise BadRequest(f"{len(blobs)} images but {k} image placeholders in the rendered prompt")
        return out, images, spans


def _vram(re) -> dict:
    """The engine's allocation ledger as mutually exclusive buckets that close to the driver's total (``utils/ledger.py``)."""
    v = re.e.ledger.view()
    v["tiers"] = re.e.rel.facts()
    # the session table: parked conversations (their sequence keeps its pages and its state row between turns) and what
    # each holds, so that "which conversation owns the pool" has an answer
    sessions = []
    for name, (sid, hist, tick) in re.parked.items():
        seq = re.e.seqs.get(sid)
        sessions.append({"session": name, "tokens": len(hist.ids), "pages": len(seq.pages) if seq else 0,
                         "droppable_segments": len(hist.spans), "idle_ticks": re._tick - tick,
                         "snapshots": len(re.e.states.of_session(name))})
    v["sessions"] = sessions
    v["snapshots"] = {"rows": len(re.e.states.snaps), "lower_tiers": len(re.e.states.lower),
                      "by_class": {k: sum(1 for s in re.e.states.snaps.values() if s.klass == k)
                                   for k in sorted({s.klass for s in re.e.states.snaps.values()})}}
    return v


async def serve(app: App, host: str, port: int):
    server = await asyncio.start_server(app.handle, host, port)
    log.info("server", f"listening on {host}:{port}")
    return server
