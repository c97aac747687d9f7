"""Blocking HTTP / SSE client for the chat endpoint (standard library sockets only).

``Client.chat`` posts one request and, when streaming, yields deltas as they arrive; the reply
aggregates content, reasoning, tool calls, usage, time to first token and inter-token gaps.

Reference counterpart: ``apps/cli/src/client.rs``.
"""
from __future__ import annotations

import http.client
import json
import time
from dataclasses import dataclass, field


@dataclass
class ChatReply:
    content: str = ""
    reasoning: str = ""
    tool_calls: list = field(default_factory=list)
    finish_reason: str | None = None
    usage: dict = field(default_factory=dict)
    ttft_ms: float = 0.0
    total_ms: float = 0.0
    gaps_ms: list = field(default_factory=list)
    status: int = 200
    error: str | None = None

    def assistant_message(self) -> dict:
        m = {"role": "assistant", "content": self.content}
        if self.tool_calls:
            m["tool_calls"] = [{"id": c["id"], "type": "function", "function": {"name": c["name"], "arguments": c["arguments"]}}
                               for c in self.tool_calls]
        return m


class Client:
    def __init__(self, url: str, model: str | None = None, timeout: float = 600.0):
        self.hostport = url.split("://", 1)[-1].rstrip("/")
        self.model, self.timeout = model, timeout

    def _conn(self):
        return http.client.HTTPConnection(self.hostport, timeout=self.timeout)

    def get(self, path: str):
        c = self._conn()
        c.request("GET", path)
        r = c.getresponse()
        body = r.read()
        c.close()
        return r.status, (json.loads(body) if body else None)

    def post(self, path: str, obj):
        c = self._conn()
        c.request("POST", path, json.dumps(obj), {"Content-Type": "application/json"})
        r = c.getresponse()
        body = r.read()
        c.close()
        return r.status, (json.loads(body) if body else None)

    def health(self):
        return self.get("/health")

    def chat(self, messages, *, max_tokens=64, session=None, tools=None, stream=True, on_delta=None, **extra) -> ChatReply:
        body = {"model": self.model or "", "messages": messages, "max_tokens": max_tokens, "stream": stream, **extra}
        if session:
            body["session"] = session
        if tools:
            body["tools"] = tools
        if stream:
            body["stream_options"] = {"include_usage": True}
        rep, t0 = ChatReply(), time.perf_counter()
        c = self._conn()
        c.request("POST", "/v1/chat/completions", json.dumps(body), {"Content-Type": "application/json"})
        r = c.getresponse()
        rep.status = r.status
        if r.status != 200 or not stream:
            d = json.loads(r.read() or b"{}")
            c.close()
            rep.total_ms = (time.perf_counter() - t0) * 1e3
            if r.status != 200:
                rep.error = json.dumps(d.get("error", d))
                return rep
            ch = d["choices"][0]
            m = ch["message"]
            rep.content, rep.reasoning = m.get("content") or "", m.get("reasoning_content") or ""
            rep.tool_calls = [{"id": t["id"], **t["function"]} for t in m.get("tool_calls", [])]
            rep.finish_reason, rep.usage = ch["finish_reason"], d.get("usage", {})
            return rep
        last = None
        while True:
            line = r.readline()
            if not line:
                break
            line = line.strip()
            if not line.startswith(b"data: "):
                continue
            payload = line[6:]
            if payload == b"[DONE]":
                break
            d = json.loads(payload)
            if "error" in d:
                rep.error = json.dumps(d["error"])
                break
            if d.get("usage"):
                rep.usage = d["usage"]
            for ch in d.get("choices", []):
                delta = ch.get("delta", {})
                now = time.perf_counter()
                if any(k in delta for k in ("content", "reasoning_content", "tool_calls")):
                    if last is None:
                        rep.ttft_ms = (now - t0) * 1e3
                    else:
                        rep.gaps_ms.append((now - last) * 1e3)
                    last = now
                if delta.get("content"):
                    rep.content += delta["content"]
                if delta.get("reasoning_content"):
                    rep.reasoning += delta["reasoning_content"]
                for t in delta.get("tool_calls", []):
                    rep.tool_calls.append({"id": t["id"], **t["function"]})
                if on_delta:
                    on_delta(delta)
                if ch.get("finish_reason"):
                    rep.finish_reason = ch["finish_reason"]
        c.close()
        rep.total_ms = (time.perf_counter() - t0) * 1e3
        return rep
