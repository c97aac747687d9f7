"""Three-channel incremental splitter of the model's output stream.

The token stream interleaves plain text, a reasoning block (``<think> ... </think>``) and tool
calls (``<tool_call> ... </tool_call>`` holding either a JSON object ``{"name": ..,
"arguments": {..}}`` or the XML function form ``<function=name><parameter=key>value</parameter>
</function>``). ``feed(delta)`` returns the events that are certain so far:

    ("text", str) | ("reasoning", str) | ("tool_call", {"id", "name", "arguments": json-string})

Invariants: nothing is emitted that could still turn out to be the beginning of a tag (the
longest suffix of the buffer that is a prefix of any tag is held back); text inside a tool call
never leaks to the text channel; an unterminated tool call at end of stream is flushed as text by
``finish`` so no output is lost; concatenating all text events gives the text outside the blocks.

Reference counterpart: ``apps/server/src/toolcall.rs`` (channel splitter, invariants I3-I5).
"""
from __future__ import annotations

import json
import re

TAGS = ("<think>", "</think>", "<tool_call>", "</tool_call>")


def _held(buf: str, tags) -> int:
    """Length of the longest suffix of buf that is a proper prefix of a tag."""
    best = 0
    for t in tags:
        for n in range(min(len(t) - 1, len(buf)), 0, -1):
            if buf.endswith(t[:n]):
                best = max(best, n)
                break
    return best


def parse_tool_body(body: str) -> dict | None:
    b = body.strip()
    if b.startswith("{"):
        try:
            obj = json.loads(b)
            args = obj.get("arguments", obj.get("parameters", {}))
            return {"name": obj["name"], "arguments": args if isinstance(args, str) else json.dumps(args, ensure_ascii=False)}
        except (json.JSONDecodeError, KeyError, TypeError):
            return None
    m = re.search(r"<function=([^>\s]+)>(.*?)</function>", b, re.S)
    if m:
        args = {}
        for pm in re.finditer(r"<parameter=([^>\s]+)>(.*?)</parameter>", m.group(2), re.S):
            v = pm.group(2).strip("\n")
            try:
                args[pm.group(1)] = json.loads(v)
            except json.JSONDecodeError:
                args[pm.group(1)] = v
        return {"name": m.group(1), "arguments": json.dumps(args, ensure_ascii=False)}
    return None


class ChannelSplitter:
    def __init__(self, start_in_think: bool = False):
        self.buf = ""
        self.mode = "think" if start_in_think else "text"
        self.n_calls = 0

    def feed(self, delta: str) -> list:
        self.buf += delta
        out = []
        while True:
            if self.mode == "text":
                i_think, i_tool = self.buf.find("<think>"), self.buf.find("<tool_call>")
                cands = [(i, t) for i, t in ((i_think, "<think>"), (i_tool, "<tool_call>")) if i >= 0]
                if cands:
                    i, tag = min(cands)
                    if i:
                        out.append(("text", self.buf[:i]))
                    self.buf = self.buf[i + len(tag):]
                    self.mode = "think" if tag == "<think>" else "tool"
                    continue
                keep = _held(self.buf, ("<think>", "<tool_call>"))
                if len(self.buf) > keep:
                    out.append(("text", self.buf[:len(self.buf) - keep]))
                    self.buf = self.buf[len(self.buf) - keep:]
                return out
            if self.mode == "think":
                i = self.buf.find("</think>")
                if i >= 0:
                    if i:
                        out.append(("reasoning", self.buf[:i]))
                    self.buf = self.buf[i + len("</think>"):]
                    self.mode = "text"
                    continue
                keep = _held(self.buf, ("</think>",))
                if len(self.buf) > keep:
                    out.append(("reasoning", self.buf[:len(self.buf) - keep]))
                    self.buf = self.buf[len(self.buf) - keep:]
                return out
            # tool call: wait for the closing tag, nothing is emitted until the call is complete
            i = self.buf.find("</tool_call>")
            if i < 0:
                return out
            body, self.buf = self.buf[:i], self.buf[i + len("</tool_call>"):]
            call = parse_tool_body(body)
            if call is None:
                out.append(("text", "<tool_call>" + body + "</tool_call>"))   # not a call after all: keep the bytes
            else:
                call["id"] = f"call_{self.n_calls}"
                self.n_calls += 1
                out.append(("tool_call", call))
            self.mode = "text"

    def finish(self) -> list:
        out = []
        if self.mode == "tool":
            call = parse_tool_body(self.buf)
            if call is not None:
                call["id"] = f"call_{self.n_calls}"
                self.n_calls += 1
                out.append(("tool_call", call))
            elif self.buf:
                out.append(("text", "<tool_call>" + self.buf))
        elif self.buf:
            out.append(("reasoning" if self.mode == "think" else "text", self.buf))
        self.buf = ""
        return out


class RepeatGuard:
    """Flags a session whose consecutive turns issue the identical tool call (observability only)."""

    def __init__(self, threshold: int = 3):
        self.threshold, self.last, self.count = threshold, {}, {}

    def observe(self, session: str, call: dict) -> bool:
        key = (call.get("name"), call.get("arguments"))
        if self.last.get(session) == key:
            self.count[session] = self.count.get(session, 1) + 1
        else:
            self.last[session], self.count[session] = key, 1
        return self.count[session] >= self.threshold
