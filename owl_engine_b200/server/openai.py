"""OpenAI-compatible request / response shapes for ``/v1/chat/completions``.

``ChatRequest.parse`` validates the body (unknown fields are ignored like OpenAI does, wrong types
are 400s) and carries the reference's extensions: ``session`` (multi-turn KV reuse),
``ignore_eos``, ``top_k``, ``chat_template_kwargs``, ``reasoning_effort`` and image parts with an
``owl_evict`` mark. ``Streamer`` turns engine token events into SSE chunks through the channel
splitter (content / reasoning_content / tool_calls deltas) and builds the final usage block.

Reference counterpart: ``apps/server/src/openai.rs:43-88, 767`` and ``toolcall.rs``.
"""
from __future__ import annotations

import base64
import json
import time
import uuid
from dataclasses import dataclass, field

from ..engine.sampler import SamplingParams
from .toolcall import ChannelSplitter


class BadRequest(ValueError):
    pass


@dataclass
class ChatRequest:
    messages: list
    model: str = ""
    max_tokens: int | None = None
    stream: bool = False
    session: str | None = None
    include_usage: bool = False
    ignore_eos: bool = False
    tools: list | None = None
    tool_choice: object = None
    chat_template_kwargs: dict = field(default_factory=dict)
    temperature: float | None = None
    top_p: float | None = None
    top_k: int | None = None
    stop: list = field(default_factory=list)
    seed: int | None = None
    reasoning_effort: str | None = None
    images: list = field(default_factory=list)     # [{"data": bytes, "evict": bool}]

    @classmethod
    def parse(cls, body: bytes) -> "ChatRequest":
        try:
            d = json.loads(body)
        except (ValueError, UnicodeDecodeError) as e:      # JSONDecodeError is a ValueError; bytes that are not UTF-8
            raise BadRequest(f"invalid JSON: {e}") from None
        if not isinstance(d, dict) or not isinstance(d.get("messages"), list) or not d["messages"]:
            raise BadRequest("messages must be a non-empty array")
        for m in d["messages"]:
            if not isinstance(m, dict) or not isinstance(m.get("role"), str) or \
                    m["role"] not in ("system", "user", "assistant", "tool", "developer"):
                raise BadRequest("every message needs a role of system|user|assistant|tool")
            c = m.get("content")
            if c is not None and not isinstance(c, (str, list)):
                raise BadRequest("message content must be a string, an array of parts or null")
            if isinstance(c, list):
                for part in c:
                    if not isinstance(part, dict) or not isinstance(part.get("type"), str):
                        raise BadRequest("every content part must be an object with a type")
                    if part["type"] == "text" and not isinstance(part.get("text"), str):
                        raise BadRequest("a text part needs a text string")
                    if part["type"] == "image_url" and not isinstance(part.get("image_url"), (dict, str)):
                        raise BadRequest("an image_url part needs an image_url object")
                    if part["type"] not in ("text", "image_url"):
                        raise BadRequest(f"content part type {part['type']!r} is not supported (text, image_url)")
            tc = m.get("tool_calls")
            if tc is not None and (not isinstance(tc, list) or not all(isinstance(x, dict) for x in tc)):
                raise BadRequest("tool_calls must be an array of objects")
            if m.get("name") is not None and not isinstance(m["name"], str):
                raise BadRequest("message name must be a string")

        def typed(k, types, what):
            v = d.get(k)
            if v is not None and not isinstance(v, types):
                raise BadRequest(f"{k} must be {what}")
            return v

        typed("session", str, "a string")
        typed("stream_options", dict, "an object")
        typed("chat_template_kwargs", dict, "an object")
        typed("reasoning_effort", str, "a string")
        tools = typed("tools", list, "an array")
        if tools is not None and not all(isinstance(t, dict) and isinstance(t.get("function", {}), dict) for t in tools):
            raise BadRequest("every tool must be an object with a function object")
        for k in ("stream", "ignore_eos"):
            typed(k, bool, "a boolean")

        def num(k, typ, lo=None, hi=None):
            v = d.get(k)
            if v is None:
                return None
            if isinstance(v, bool) or not isinstance(v, (int, float)):
                raise BadRequest(f"{k} must be a number")
            if (lo is not None and v < lo) or (hi is not None and v > hi):
                raise BadRequest(f"{k} out of range")
            return typ(v)

        stop = d.get("stop") or []
        if isinstance(stop, str):
            stop = [stop]
        if not isinstance(stop, list) or not all(isinstance(s, str) for s in stop):
            raise BadRequest("stop must be a string or an array of strings")
        images = []
        for m in d["messages"]:
            if isinstance(m.get("content"), list):
                for part in m["content"]:
                    if part.get("type") == "image_url":
                        iu = part.get("image_url")
                        url = iu if isinstance(iu, str) else (iu or {}).get("url", "")
                        if not isinstance(url, str) or not url.startswith("data:") or "," not in url:
                            raise BadRequest("only data: URLs are accepted for images")
                        try:
                            raw = base64.b64decode(url.split(",", 1)[1])
                        except Exception:
                            raise BadRequest("image data URL is not valid base64") from None
                        images.append({"data": raw, "evict": bool(part.get("owl_evict", False))})
        mt = num("max_tokens", int, 1) or num("max_completion_tokens", int, 1)
        return cls(messages=d["messages"], model=str(d.get("model", "")), max_tokens=mt, stream=bool(d.get("stream", False)),
                   session=d.get("session"), include_usage=bool((d.get("stream_options") or {}).get("include_usage", False)),
                   ignore_eos=bool(d.get("ignore_eos", False)), tools=d.get("tools"), tool_choice=d.get("tool_choice"),
                   chat_template_kwargs=dict(d.get("chat_template_kwargs") or {}), temperature=num("temperature", float, 0, 5),
                   top_p=num("top_p", float, 0, 1), top_k=num("top_k", int, 1), stop=stop, seed=num("seed", int),
                   reasoning_effort=d.get("reasoning_effort"), images=images)

    def sampling(self, default: SamplingParams) -> SamplingParams:
        if self.temperature is None and self.top_p is None and self.top_k is None:
            return SamplingParams(default.mode, default.temp, default.topk, default.topp, default.rep_penalty,
                                  self.seed or default.seed)
        temp = default.temp if self.temperature is None else self.temperature
        return SamplingParams("greedy" if temp == 0 else "sampling", temp, self.top_k or default.topk,
                              self.top_p if self.top_p is not None else default.topp, default.rep_penalty, self.seed or 0)


class Streamer:
    """Engine tokens -> OpenAI chunks. One instance per response."""

    def __init__(self, model: str, decoder, stop: list[str], start_in_think: bool = False, tools=None):
        self.id = "chatcmpl-" + uuid.uuid4().hex[:24]
        self.model, self.created = model, int(time.time())
        self.decoder, self.splitter = decoder, ChannelSplitter(start_in_think, tools=tools)
        self.malformed: list = []        # tool blocks that could not be parsed (logged by the server, never emitted as text)
        self.stop, self.text_tail, self.stopped = stop, "", False
        self.content, self.reasoning, self.tool_calls = [], [], []
        self.first = True

    def _chunk(self, delta: dict, finish=None, usage=None) -> dict:
        c = {"id": self.id, "object": "chat.completion.chunk", "created": self.created, "model": self.model,
             "choices": [{"index": 0, "delta": delta, "finish_reason": finish}]}
        if usage is not None:
            c["usage"] = usage
        return c

    def _events_to_chunks(self, events) -> list[dict]:
        out = []
        for ev in events:
            delta = {}
            if self.first:
                delta["role"] = "assistant"
                self.first = False
            if ev[0] == "text":
                text = ev[1]
                if self.stop:
                    text = self._hold_for_stop(text)
                if text:
                    self.content.append(text)
                    delta["content"] = text
            elif ev[0] == "reasoning":
                self.reasoning.append(ev[1])
                delta["reasoning_content"] = ev[1]
            elif ev[0] == "malformed":
                self.malformed.append(ev[1])
            else:
                i = len(self.tool_calls)
                self.tool_calls.append(ev[1])
                delta["tool_calls"] = [{"index": i, "id": ev[1]["id"], "type": "function",
                                        "function": {"name": ev[1]["name"], "arguments": ev[1]["arguments"]}}]
            if len(delta) > (1 if "role" in delta else 0) or "role" in delta:
                out.append(self._chunk(delta))
            if self.stopped:
                break
        return out

    def _hold_for_stop(self, text: str) -> str:
        """Release text only when it can no longer be the start of a stop string."""
        buf = self.text_tail + text
        hit = min((buf.find(s) for s in self.stop if s in buf), default=-1)
        if hit >= 0:
            self.stopped, self.text_tail = True, ""
            return buf[:hit]
        hold = 0
        for s in self.stop:
            for n in range(min(len(s) - 1, len(buf)), 0, -1):
                if buf.endswith(s[:n]):
                    hold = max(hold, n)
                    break
        self.text_tail = buf[len(buf) - hold:] if hold else ""
        return buf[:len(buf) - hold]

    def on_token(self, token: int) -> list[dict]:
        piece = self.decoder.push(token)
        return self._events_to_chunks(self.splitter.feed(piece)) if piece and not self.stopped else []

    def finish(self, reason: str, usage: dict, include_usage: bool) -> list[dict]:
        out = [] if self.stopped else self._events_to_chunks(self.splitter.finish())
        if not self.stopped:
            out += self._events_to_chunks(self._flush_tail())
        fr = "tool_calls" if self.tool_calls else ("stop" if self.stopped else reason)
        out.append(self._chunk({}, finish=fr, usage=self.usage(usage) if include_usage else None))
        return out

    def _flush_tail(self) -> list:
        """Text held back as a possible stop-string prefix is released when the turn ends."""
        tail, self.text_tail, self.stop = self.text_tail, "", []
        return [("text", tail)] if tail else []

    def drain(self) -> None:
        if not self.stopped:
            self._events_to_chunks(self.splitter.finish())
        if not self.stopped:
            self._events_to_chunks(self._flush_tail())

    def usage(self, u: dict) -> dict:
        return {"prompt_tokens": u["prompt_tokens"], "completion_tokens": u["completion_tokens"],
                "total_tokens": u["prompt_tokens"] + u["completion_tokens"],
                "prompt_tokens_details": {"cached_tokens": u.get("cached_tokens", 0)},
                "completion_tokens_details": {"reasoning_tokens": self.splitter.reasoning_steps}}

    def full_response(self, reason: str, usage: dict) -> dict:
        msg = {"role": "assistant", "content": "".join(self.content)}
        if self.reasoning:
            msg["reasoning_content"] = "".join(self.reasoning)
        if self.tool_calls:
            msg["tool_calls"] = [{"id": c["id"], "type": "function", "function": {"name": c["name"], "arguments": c["arguments"]}}
                                 for c in self.tool_calls]
        fr = "tool_calls" if self.tool_calls else ("stop" if self.stopped else reason)
        return {"id": self.id, "object": "chat.completion", "created": self.created, "model": self.model,
                "choices": [{"index": 0, "message": msg, "finish_reason": fr}], "usage": self.usage(usage)}
