"""Three-channel incremental splitter of the model's output stream.

The generated text interleaves plain text, a reasoning block and tool calls. ``feed(delta)`` (one call per engine
token) returns the events that are certain so far; ``finish()`` flushes the rest:

    ("text", str) | ("reasoning", str) | ("tool_call", {"id", "index", "name", "arguments": json-string})
    | ("malformed", {"kind": str, "raw": str})

Recognised forms

* reasoning: ``<think> .. </think>`` and the aliases ``<thinking>`` / ``<thought>``;
* tool call, wrapped: ``<tool_call> BODY </tool_call>`` with BODY either a JSON object
  ``{"name": .., "arguments": {..}}`` (tolerantly parsed, see ``lenient_json``) or the XML function form
  ``<function=name><parameter=key>value</parameter>..</function>``. The XML form is complete at ``</function>``:
  the call is emitted there, before the closing wrapper arrives, and several functions may share one wrapper;
* tool call, bare: ``<function=name>..</function>`` without a wrapper (some templates drop it);
* tool call, invoke form: ``<function_calls><invoke name=".."><parameter name="..">v</parameter></invoke>..
  </function_calls>`` (one or more invokes; a ``<function=..>`` or JSON body inside this wrapper is accepted too).

Invariants: (1) a marker never reaches the text or reasoning channel, not even one that is out of place for the
current state (it is swallowed and counted in ``strays``); (2) nothing is emitted that could still be the beginning
of a marker: the longest suffix that is a proper prefix of an active marker is held back; (3) ``arguments`` is always
a valid JSON string; (4) call indices are consecutive; (5) a tool block that cannot be parsed is never dropped
silently: it becomes a ``malformed`` event (``unclosed``, ``overflow``, ``no_function``, ``json_invalid``, ..) and is
counted; at end of stream an unclosed block whose body is complete is still salvaged; (6) the line feeds the chat
template writes after the closing reasoning marker (at most two) belong to the template, not to the content.

XML parameter values are text. With the request's ``tools`` schemas they are converted to the declared JSON type
(``integer``, ``number``, ``boolean``, ``array``, ``object``); a parameter without a declared type stays a string when
its tool is known and is read as JSON when it parses otherwise. Nothing is validated: a wrong tool name or argument goes
to the client as it is.

Reference counterpart: ``apps/server/src/toolcall.rs`` (channel splitter and its invariants I3-I5, marker aliases,
bare and invoke forms, Malformed items, structural trace, lenient JSON).
"""
from __future__ import annotations

import json
import math

THINK_OPEN = ("<think>", "<thinking>", "<thought>")
THINK_CLOSE = ("</think>", "</thinking>", "</thought>")
TOOL_OPEN, TOOL_CLOSE = "<tool_call>", "</tool_call>"
FUNC_OPEN, FUNC_CLOSE = "<function=", "</function>"
CALLS_OPEN, CALLS_CLOSE = "<function_calls>", "</function_calls>"
MARKS = THINK_OPEN + THINK_CLOSE + (TOOL_OPEN, TOOL_CLOSE, FUNC_OPEN, CALLS_OPEN, CALLS_CLOSE)
TOOL_MARKS = (TOOL_OPEN, TOOL_CLOSE, FUNC_OPEN, CALLS_OPEN, CALLS_CLOSE)
BETWEEN_MARKS = (TOOL_CLOSE, TOOL_OPEN, FUNC_OPEN, CALLS_OPEN, CALLS_CLOSE)
NS_PREFIX = "ant" + "ml:"      # a namespace prefix some models copy in front of invoke / parameter tag names
MAX_TOOL_BYTES = 1 << 20      # an unclosed tool block may not eat memory without bound
TRACE_CAP = 512

TEXT, THINK, TOOL, BARE, INVOKE, BETWEEN = "text", "think", "tool", "bare_tool", "invoke_tool", "between_tool"


def _held(buf: str, tags) -> int:
    """Length of the longest suffix of buf that is a proper prefix of a tag."""
    best = 0
    for t in tags:
        for n in range(min(len(t) - 1, len(buf)), best, -1):
            if buf.endswith(t[:n]):
                best = n
                break
    return best


def _canon(m: str) -> str:
    if m in THINK_OPEN:
        return "<think>"
    if m in THINK_CLOSE:
        return "</think>"
    return m


# ---- tolerant JSON ------------------------------------------------------------------------------------------------
class _Lenient:
    """Recursive-descent reader for almost-JSON: single or double quotes, bare keys, trailing commas, ``//`` and
    ``/* */`` comments, Python / JS literals (True, None, nil, NaN, Infinity), numbers like ``.5`` or ``1.``, missing
    closing brackets (closed at end of input) and trailing text after the first complete value (ignored)."""

    WORDS = {"true": True, "false": False, "null": None, "none": None, "nil": None, "nan": None, "infinity": None,
             "-infinity": None}

    def __init__(self, s: str):
        self.s, self.i = s, 0

    def ws(self) -> None:
        s = self.s
        while self.i < len(s):
            c = s[self.i]
            if c.isspace():
                self.i += 1
            elif s.startswith("//", self.i):
                j = s.find("\n", self.i)
                self.i = len(s) if j < 0 else j
            elif s.startswith("/*", self.i):
                j = s.find("*/", self.i + 2)
                self.i = len(s) if j < 0 else j + 2
            else:
                return

    def string(self) -> str:
        q = self.s[self.i]
        self.i += 1
        out = []
        s = self.s
        while self.i < len(s):
            c = s[self.i]
            self.i += 1
            if c == q:
                break
            if c == "\\" and self.i < len(s):
                e = s[self.i]
                self.i += 1
                if e == "u" and self.i + 4 <= len(s):
                    try:
                        out.append(chr(int(s[self.i:self.i + 4], 16)))
                        self.i += 4
                        continue
                    except ValueError:
                        pass
                out.append({"n": "\n", "t": "\t", "r": "\r", "b": "\b", "f": "\f", "/": "/"}.get(e, e))
            else:
                out.append(c)
        return "".join(out)

    def bare(self) -> str:
        j = self.i
        while j < len(self.s) and self.s[j] not in ",:{}[]\"'\n" and not self.s[j].isspace():
            j += 1
        w, self.i = self.s[self.i:j], j
        return w

    def value(self, depth: int = 0):
        if depth > 64:
            raise ValueError("nesting")
        self.ws()
        if self.i >= len(self.s):
            raise ValueError("eof")
        c = self.s[self.i]
        if c == "{":
            self.i += 1
            obj = {}
            while True:
                self.ws()
                if self.i >= len(self.s):
                    return obj                      # missing closer: close at end of input
                c = self.s[self.i]
                if c == "}":
                    self.i += 1
                    return obj
                if c == ",":
                    self.i += 1
                    continue
                key = self.string() if c in "\"'" else self.bare()
                if key == "" and c not in "\"'":
                    raise ValueError("key")
                self.ws()
                if self.i < len(self.s) and self.s[self.i] in ":=":
                    self.i += 1
                else:
                    raise ValueError("colon")
                try:
                    obj[key] = self.value(depth + 1)
                except ValueError:
                    if self.i >= len(self.s):
                        return obj                  # value cut off by the end of input: keep what was read
                    raise
        if c == "[":
            self.i += 1
            arr = []
            while True:
                self.ws()
                if self.i >= len(self.s):
                    return arr
                if self.s[self.i] == "]":
                    self.i += 1
                    return arr
                if self.s[self.i] == ",":
                    self.i += 1
                    continue
                arr.append(self.value(depth + 1))
        if c in "\"'":
            return self.string()
        w = self.bare()
        if not w:
            raise ValueError("token")
        lw = w.lower()
        if lw in self.WORDS:
            return self.WORDS[lw]
        try:
            f = float(w)
        except ValueError:
            raise ValueError("token") from None
        if not math.isfinite(f):
            return None
        try:
            return int(w)
        except ValueError:
            return int(f) if f.is_integer() and "e" not in lw and "." not in w else f


def lenient_json(s: str):
    """Parse almost-JSON (see ``_Lenient``). Returns ``(value, repaired)``; raises ValueError when nothing can be read."""
    t = s.strip()
    try:
        return json.loads(t), False
    except json.JSONDecodeError:
        pass
    except RecursionError:                    # nesting deeper than the interpreter's stack: the model ran away, not JSON
        raise ValueError("nesting") from None
    return _Lenient(t).value(), True


# ---- request-side schemas -----------------------------------------------------------------------------------------
class ToolSchemas:
    """``name -> property -> JSON type`` from the request's ``tools`` array (nested ``{type, function: {..}}`` or flat).
    Used only to give XML parameter values their declared type; nothing is validated."""

    def __init__(self, tools=None):
        self.types: dict = {}
        for t in tools or []:
            f = t.get("function", t) if isinstance(t, dict) else None
            if not isinstance(f, dict) or not isinstance(f.get("name"), str):
                continue
            props = {}
            pp = (f.get("parameters") or {}).get("properties") if isinstance(f.get("parameters"), dict) else None
            for k, v in (pp or {}).items():
                ty = self._type_of(v)
                if ty:
                    props[k] = ty
            self.types[f["name"]] = props

    @staticmethod
    def _type_of(v):
        if not isinstance(v, dict):
            return None
        if isinstance(v.get("type"), str):
            return v["type"]
        if isinstance(v.get("type"), list):
            return next((t for t in v["type"] if t != "null"), None)
        for key in ("anyOf", "oneOf"):
            for item in v.get(key) or []:
                if isinstance(item, dict) and isinstance(item.get("type"), str) and item["type"] != "null":
                    return item["type"]
        return None

    def knows(self, name: str) -> bool:
        return name in self.types

    @staticmethod
    def _json_or_quoted(raw: str):
        """Bare JSON, or JSON wrapped in JSON quotes (``"512"`` -> 512); ``...`` (Ellipsis) when it is neither."""
        try:
            v = json.loads(raw.strip())
        except (json.JSONDecodeError, RecursionError):
            return ...
        if isinstance(v, str):
            try:
                return json.loads(v.strip())
            except (json.JSONDecodeError, RecursionError):
                return v
        return v

    def coerce(self, tool: str, prop: str, raw: str):
        if tool not in self.types:
            v = self._json_or_quoted(raw) if raw.strip()[:1] in "-0123456789tfn[{" else ...
            return raw if v is ... or isinstance(v, str) else v
        ty = self.types[tool].get(prop)
        if ty is None:
            return raw
        v = self._json_or_quoted(raw)
        if ty in ("number", "float"):
            return v if isinstance(v, (int, float)) and not isinstance(v, bool) else raw
        if ty == "integer":
            if isinstance(v, bool) or not isinstance(v, (int, float)):
                return raw
            return int(v) if float(v).is_integer() else v
        if ty == "boolean":
            if isinstance(v, bool):
                return v
            return {"true": True, "false": False}.get(raw.strip().lower(), raw)
        if ty in ("array", "object"):
            return v if isinstance(v, (list, dict)) else raw
        return raw


# ---- tool bodies --------------------------------------------------------------------------------------------------
class Malformed(Exception):
    def __init__(self, kind: str):
        super().__init__(kind)
        self.kind = kind


def _strip_nl(v: str) -> str:
    if v.startswith("\n"):
        v = v[1:]
    if v.endswith("\n"):
        v = v[:-1]
    return v


def _args_string(args) -> str:
    """The ``arguments`` field as a valid JSON string, whatever the model put there."""
    if isinstance(args, str):
        try:
            json.loads(args)
            return args
        except (json.JSONDecodeError, RecursionError):
            try:
                return json.dumps(lenient_json(args)[0], ensure_ascii=False)
            except ValueError:
                return json.dumps(args, ensure_ascii=False)
    return json.dumps({} if args is None else args, ensure_ascii=False)


def _call_from_obj(obj) -> tuple[str, str]:
    if not isinstance(obj, dict):
        raise Malformed("json_not_object")
    fn = obj.get("function") if isinstance(obj.get("function"), dict) else None
    name = obj.get("name") or (fn or {}).get("name") or obj.get("tool") or (obj.get("function") if isinstance(obj.get("function"), str) else None)
    if not isinstance(name, str) or not name:
        raise Malformed("json_no_name")
    src = fn if fn is not None and "name" not in obj else obj
    args = next((src[k] for k in ("arguments", "parameters", "args", "input") if k in src), {})
    return name, _args_string(args)


def parse_function_blocks(body: str, schemas: ToolSchemas) -> list[tuple[str, str]]:
    """One or more ``<function=name>[<parameter=key>value</parameter>..]</function>`` blocks (the closing tag of the last
    one may be missing: the caller cut the body there)."""
    calls, at = [], 0
    while True:
        i = body.find(FUNC_OPEN, at)
        if i < 0:
            break
        if body[at:i].strip():
            raise Malformed("unexpected_text")
        gt = body.find(">", i)
        if gt < 0:
            raise Malformed("bad_function_tag")
        name = body[i + len(FUNC_OPEN):gt].strip().strip("\"'")
        if not name:
            raise Malformed("empty_name")
        end = body.find(FUNC_CLOSE, gt)
        inner = body[gt + 1:end if end >= 0 else len(body)]
        args, p = {}, 0
        while True:
            a = inner.find("<parameter", p)
            if a < 0:
                break
            b = inner.find(">", a)
            if b < 0:
                raise Malformed("bad_parameter_tag")
            tag = inner[a + len("<parameter"):b]
            key = tag[1:].strip().strip("\"'") if tag.startswith("=") else (_attr(tag, "name") or "")
            c = inner.find("</parameter>", b)
            nxt = inner.find("<parameter", b)
            if c < 0 or (0 <= nxt < c):
                # a parameter without its closing tag ends where the next one starts (or at the end of the block)
                val, p = inner[b + 1:nxt if nxt >= 0 else len(inner)], (nxt if nxt >= 0 else len(inner))
            else:
                val, p = inner[b + 1:c], c + len("</parameter>")
            if key:
                args[key] = schemas.coerce(name, key, _strip_nl(val))
        calls.append((name, json.dumps(args, ensure_ascii=False)))
        at = len(body) if end < 0 else end + len(FUNC_CLOSE)
    if not calls:
        raise Malformed("no_function")
    if body[at:].strip():
        raise Malformed("unexpected_text")
    return calls


def _attr(tag: str, attr: str):
    """Value of a quoted attribute inside a tag's text, or None."""
    at = 0
    while True:
        i = tag.find(attr, at)
        if i < 0:
            return None
        j = i + len(attr)
        if (i == 0 or tag[i - 1].isspace()) and tag[j:].lstrip()[:1] == "=":
            rest = tag[j:].lstrip()[1:].lstrip()
            if rest[:1] in ("\"", "'"):
                k = rest.find(rest[0], 1)
                return rest[1:k] if k > 0 else None
            return None
        at = j


def parse_invoke_blocks(body: str, schemas: ToolSchemas) -> list[tuple[str, str]]:
    calls, at = [], 0
    while True:
        i = body.find("<invoke", at)
        if i < 0:
            break
        if body[at:i].strip():
            raise Malformed("invoke_unexpected_text")
        gt = body.find(">", i)
        if gt < 0:
            raise Malformed("invoke_bad_tag")
        name = _attr(body[i + len("<invoke"):gt], "name")
        if not name:
            raise Malformed("invoke_no_name")
        end = body.find("</invoke>", gt)
        if end < 0:
            raise Malformed("invoke_unclosed")
        inner, args, p = body[gt + 1:end], {}, 0
        while True:
            a = inner.find("<parameter", p)
            if a < 0:
                break
            if inner[p:a].strip():
                raise Malformed("invoke_unexpected_text")
            b = inner.find(">", a)
            c = inner.find("</parameter>", b)
            if b < 0 or c < 0:
                raise Malformed("invoke_param_unclosed")
            tag = inner[a + len("<parameter"):b]
            key = _attr(tag, "name") or tag.lstrip("=").strip().strip("\"'")
            if key:
                args[key] = schemas.coerce(name, key, _strip_nl(inner[b + 1:c]))
            p = c + len("</parameter>")
        if inner[p:].strip():
            raise Malformed("invoke_unexpected_text")
        calls.append((name, json.dumps(args, ensure_ascii=False)))
        at = end + len("</invoke>")
    if body[at:].strip():
        raise Malformed("invoke_unexpected_text")
    if not calls:
        raise Malformed("invoke_none")
    return calls


def parse_json_calls(body: str) -> tuple[list[tuple[str, str]], bool]:
    try:
        v, repaired = lenient_json(body)
    except ValueError:
        raise Malformed("json_invalid") from None
    items = v if isinstance(v, list) else [v]
    if not items:
        raise Malformed("json_empty")
    return [_call_from_obj(o) for o in items], repaired


def parse_tool_body(body: str, schemas: ToolSchemas | None = None):
    """Body of one wrapped or bare tool block -> ``[(name, arguments json string)]`` (normally one), plus whether a near
    miss was repaired. Raises ``Malformed``. Kept as a function for callers that hold a complete block."""
    schemas = schemas or ToolSchemas()
    b = body.strip()
    if b.endswith(TOOL_CLOSE):
        b = b[:-len(TOOL_CLOSE)].rstrip()
    if not b:
        raise Malformed("empty")
    if b.startswith(FUNC_OPEN) or (FUNC_OPEN in b and not b.startswith(("{", "["))):
        return parse_function_blocks(b[b.find(FUNC_OPEN):], schemas), not b.startswith(FUNC_OPEN)
    if b.startswith("<invoke") or "<invoke" in b and not b.startswith(("{", "[")):
        return parse_invoke_blocks(b[b.find("<invoke"):], schemas), True
    return parse_json_calls(b)


def _body_complete(raw: str) -> bool:
    """An unclosed block at end of stream is worth salvaging when its body looks whole."""
    b = raw.strip()
    if not b:
        return False
    if b.startswith(("{", "[")):
        depth, q, esc = 0, "", False
        for c in b:
            if q:
                if esc:
                    esc = False
                elif c == "\\":
                    esc = True
                elif c == q:
                    q = ""
            elif c in "\"'":
                q = c
            elif c in "{[":
                depth += 1
            elif c in "}]":
                depth -= 1
        return depth <= 0 and not q
    return FUNC_CLOSE in b or "</invoke>" in b


# ---- the splitter -------------------------------------------------------------------------------------------------
class ChannelSplitter:
    def __init__(self, start_in_think: bool = False, tools=None, parse_tools: bool = True):
        """``start_in_think``: the chat template already wrote the opening reasoning marker into the prompt, so the
        generated stream starts inside the reasoning block. ``tools``: the request's OpenAI ``tools`` array.
        ``parse_tools`` = False lets tool markers through as plain text (diagnostics)."""
        self.buf = ""
        self.mode = THINK if start_in_think else TEXT
        self.schemas = tools if isinstance(tools, ToolSchemas) else ToolSchemas(tools)
        self.parse_tools = parse_tools
        self.n_calls = 0
        self.strays = 0
        self.malformed = 0
        self.reasoning_steps = 0       # feeds that arrived while inside the reasoning block (one feed = one token)
        self.swallow_lf = 0
        self._trace: list[str] = []
        self._trace_dropped = 0

    # -- observability ----------------------------------------------------------------------------------------------
    def _note(self, line: str) -> None:
        if len(self._trace) < TRACE_CAP:
            self._trace.append(line)
        else:
            self._trace_dropped += 1

    def trace(self) -> list[str]:
        """Structure of the turn (state changes, swallowed markers, tools, repairs), never the text itself."""
        return self._trace + ([f"...(+{self._trace_dropped} dropped)"] if self._trace_dropped else [])

    def _go(self, to: str) -> None:
        if to != self.mode:
            self._note(f"state {self.mode}->{to}")
            self.mode = to

    # -- emission helpers -------------------------------------------------------------------------------------------
    def _emit_calls(self, out: list, calls, repair: str | None) -> None:
        for name, args in calls:
            if repair:
                self._note(f"repair {name} {repair}")
            out.append(("tool_call", {"id": f"call_{self.n_calls}", "index": self.n_calls, "name": name, "arguments": args}))
            self._note(f"tool #{self.n_calls} {name} args={len(args)}B")
            self.n_calls += 1

    def _emit_malformed(self, out: list, kind: str, raw: str) -> None:
        self.malformed += 1
        self._note(f"malformed {kind} {len(raw)}B")
        out.append(("malformed", {"kind": kind, "raw": raw}))

    def _close_block(self, out: list, body: str, invoke: bool = False, repair: str | None = None) -> None:
        try:
            if invoke:
                b = body.strip().replace("<" + NS_PREFIX, "<").replace("</" + NS_PREFIX, "</")
                if b.endswith(TOOL_CLOSE):
                    b = b[:-len(TOOL_CLOSE)].rstrip()
                try:
                    calls, rep = parse_invoke_blocks(b, self.schemas), False
                except Malformed as first:
                    if FUNC_OPEN in b:
                        calls, rep = parse_function_blocks(b[b.find(FUNC_OPEN):], self.schemas), True
                    elif b.startswith(("{", "[")):
                        calls, rep = parse_json_calls(b)[0], True
                    else:
                        raise first
                self._emit_calls(out, calls, repair or ("mixed_wrapper" if rep else None))
            else:
                calls, rep = parse_tool_body(body, self.schemas)
                self._emit_calls(out, calls, repair or ("near_miss" if rep else None))
        except Malformed as m:
            self._emit_malformed(out, ("invoke_" if invoke and not m.kind.startswith("invoke") else "") + m.kind, body)

    # -- state machine ----------------------------------------------------------------------------------------------
    def _marks(self):
        return MARKS if self.parse_tools else tuple(m for m in MARKS if m not in TOOL_MARKS)

    def _on_mark(self, m: str) -> None:
        c = _canon(m)
        if self.mode in (TEXT, THINK) and c == TOOL_OPEN:
            self._go(TOOL)            # a tool opened inside the reasoning block is a tool, not reasoning
        elif self.mode in (TEXT, THINK) and c == FUNC_OPEN:
            self._go(BARE)
        elif self.mode in (TEXT, THINK) and c == CALLS_OPEN:
            self._go(INVOKE)
        elif self.mode == TEXT and c == "<think>":
            self._go(THINK)
        elif self.mode == THINK and c == "</think>":
            self.swallow_lf = 2
            self._go(TEXT)
        else:
            self.strays += 1
            self._note(f"stray {c}")

    def feed(self, delta: str) -> list:
        if self.mode == THINK:
            self.reasoning_steps += 1
        self.buf += delta
        return self._drain()

    def _drain(self) -> list:
        out: list = []
        while True:
            if self.swallow_lf and self.mode == TEXT:
                n = 0
                while self.swallow_lf and self.buf[:1] == "\n":
                    self.buf, self.swallow_lf, n = self.buf[1:], self.swallow_lf - 1, n + 1
                if n:
                    self._note(f"swallow_lf {n}")
                if self.swallow_lf:
                    if not self.buf:
                        return out           # cannot decide yet: wait for the next piece
                    self.swallow_lf = 0
            if self.mode in (TEXT, THINK):
                marks = self._marks()
                hit = None
                for m in marks:
                    p = self.buf.find(m)
                    if p >= 0 and (hit is None or p < hit[0] or (p == hit[0] and len(m) > len(hit[1]))):
                        hit = (p, m)
                chan = "reasoning" if self.mode == THINK else "text"
                if hit is None:
                    keep = _held(self.buf, marks)
                    if len(self.buf) > keep:
                        out.append((chan, self.buf[:len(self.buf) - keep]))
                        self.buf = self.buf[len(self.buf) - keep:]
                    return out
                p, m = hit
                if p:
                    out.append((chan, self.buf[:p]))
                # the bare function marker stays in the buffer: the body parser reads the name from it
                self.buf = self.buf[p if m == FUNC_OPEN else p + len(m):]
                self._on_mark(m)
                if m == FUNC_OPEN and self.mode != BARE:
                    self.buf = self.buf[len(m):]          # stray: swallowed like any other marker
                continue
            if self.mode == TOOL:
                xml = self.buf.lstrip().startswith(FUNC_OPEN)
                f = self.buf.find(FUNC_CLOSE) if xml else -1
                t = self.buf.find(TOOL_CLOSE)
                if f >= 0 and (t < 0 or f < t):
                    body, self.buf = self.buf[:f + len(FUNC_CLOSE)], self.buf[f + len(FUNC_CLOSE):]
                    self._close_block(out, body)
                    self._go(BETWEEN)
                    continue
                if t >= 0:
                    body, self.buf = self.buf[:t], self.buf[t + len(TOOL_CLOSE):]
                    self._close_block(out, body)
                    self._go(TEXT)
                    continue
            elif self.mode == BARE:
                f = self.buf.find(FUNC_CLOSE)
                if f >= 0:
                    body, self.buf = self.buf[:f + len(FUNC_CLOSE)], self.buf[f + len(FUNC_CLOSE):]
                    self._close_block(out, body)
                    self._go(BETWEEN)
                    continue
            elif self.mode == INVOKE:
                c = self.buf.find(CALLS_CLOSE)
                if c >= 0:
                    body, self.buf = self.buf[:c], self.buf[c + len(CALLS_CLOSE):]
                    self._close_block(out, body, invoke=True)
                    self._go(TEXT)
                    continue
            elif self.mode == BETWEEN:
                # white space between a closed function and the next structural marker belongs to the template
                hit = min(((p, m) for m in BETWEEN_MARKS if (p := self.buf.find(m)) >= 0), default=None)
                if hit is not None:
                    p, m = hit
                    if self.buf[:p].strip():
                        # real text before the marker: hand it to the text channel, without the template's white space in
                        # front of it (the same text arriving in smaller pieces is stripped below: one rule for both)
                        self.buf = self.buf.lstrip()
                        self._go(TEXT)
                        continue
                    self.buf = self.buf[p if m == FUNC_OPEN else p + len(m):]
                    self._go({TOOL_CLOSE: TEXT, CALLS_CLOSE: TEXT, TOOL_OPEN: TOOL, FUNC_OPEN: BARE, CALLS_OPEN: INVOKE}[m])
                    continue
                if _held(self.buf, BETWEEN_MARKS) == len(self.buf):
                    return out                            # everything held could still become a marker
                self.buf = self.buf.lstrip()
                if not self.buf:
                    return out
                if _held(self.buf, BETWEEN_MARKS) == len(self.buf):
                    return out
                self._go(TEXT)
                continue
            # inside a tool block without its closing marker yet
            if len(self.buf) > MAX_TOOL_BYTES:
                raw, self.buf = self.buf, ""
                self._emit_malformed(out, f"{self.mode}_overflow", raw)
                self._go(TEXT)
                continue
            return out

    def finish(self) -> list:
        out: list = []
        if self.mode in (TOOL, BARE, INVOKE):
            raw, self.buf = self.buf, ""
            kind = {TOOL: "unclosed", BARE: "bare_unclosed", INVOKE: "invoke_unclosed"}[self.mode]
            if _body_complete(raw):
                # cut off before the closing marker (budget, stop) but the body is whole: emit it, and say so
                before = self.malformed
                self._close_block(out, raw, invoke=self.mode == INVOKE, repair=f"{kind}:missing_close")
                if self.malformed > before and not any(e[0] == "tool_call" for e in out):
                    out[:] = [e for e in out if e[0] != "malformed"]
                    self.malformed = before
                    self._emit_malformed(out, kind, raw)
            else:
                self._emit_malformed(out, kind, raw)
            self._go(TEXT)
        else:
            if self.swallow_lf:
                n = 0
                while self.swallow_lf and self.buf[:1] == "\n":
                    self.buf, self.swallow_lf, n = self.buf[1:], self.swallow_lf - 1, n + 1
                self.swallow_lf = 0
                if n:
                    self._note(f"swallow_lf {n}")
            if self.mode == BETWEEN:
                self.buf = self.buf.lstrip()
            if self.buf:
                out.append(("reasoning" if self.mode == THINK else "text", self.buf))
        self._note(f"finish {self.mode} held={len(self.buf)}B")
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
