"""Agent-workload end-to-end harness: drives a live server with real tool execution and images.

Suites: ``core`` (text multi-turn, tool round trip, vision chat, image identity, mixed tool+image,
decode-vs-prefill concurrency), ``gui`` (GUI agent whose every tool result carries a screenshot,
window of the newest three images), ``gui-capability`` (a capability question must still call
``screenshot``), ``image-evict`` (image deletion shapes: marked, middle, last, with a tool round,
sliding window), ``all``.

Every scenario makes two kinds of checks. Protocol checks (status codes, usage accounting,
``cached_tokens`` growth across turns of one session, finish reasons, stream framing) hold for any
weights and always run. Semantic checks (the model names the colour on the screenshot, calls the
right tool) need a trained checkpoint and run only with ``semantic=True``.

Reference counterpart: ``apps/cli/src/workload/{mod,scenarios,gui,tools,concurrency,report}.rs``.
"""
from __future__ import annotations

import json
import os
import random
import threading
import time
from dataclasses import dataclass, field

from . import png
from .client import ChatReply, Client

WORDS = ("amber basin cobalt delta ember fjord garnet harbor iris jasper kelp lumen meadow nimbus onyx prism quartz raven "
         "sable tundra umber vapor willow xenon yarrow zephyr anchor beacon cinder dune").split()


class Failed(AssertionError):
    pass


def ensure(cond, msg):
    if not cond:
        raise Failed(msg)


@dataclass
class Report:
    name: str
    ok: bool = True
    error: str | None = None
    turns: list = field(default_factory=list)
    notes: dict = field(default_factory=dict)

    def turn(self, label: str, r: ChatReply):
        self.turns.append({"label": label, "status": r.status, "finish": r.finish_reason, "ttft_ms": round(r.ttft_ms, 1),
                           "total_ms": round(r.total_ms, 1), "usage": r.usage, "tool_calls": [c["name"] for c in r.tool_calls],
                           "max_gap_ms": round(max(r.gaps_ms), 1) if r.gaps_ms else 0.0})
        return r

    def line(self) -> str:
        mark = "PASS" if self.ok else "FAIL"
        n = sum(t["usage"].get("completion_tokens", 0) for t in self.turns)
        return f"[{mark}] {self.name}: {len(self.turns)} turns, {n} tokens" + (f" -- {self.error}" if self.error else "")


@dataclass
class Ctx:
    client: Client
    max_tokens: int = 64
    semantic: bool = False
    server_log: str | None = None
    pid: int = field(default_factory=os.getpid)

    def session(self, tag: str) -> str:
        return f"wl-{self.pid}-{tag}-{random.getrandbits(24):06x}"

    def log_text(self) -> str:
        if self.server_log and os.path.exists(self.server_log):
            return open(self.server_log, errors="replace").read()
        return ""


def cached(r: ChatReply) -> int:
    return (r.usage.get("prompt_tokens_details") or {}).get("cached_tokens", 0)


def nonce() -> str:
    return " ".join(random.choice(WORDS) for _ in range(6))


def image_part(url: str, evict: bool) -> dict:
    p = {"type": "image_url", "image_url": {"url": url}}
    if evict:
        p["owl_evict"] = True
    return p


def remove_image(history: list, url: str) -> bool:
    """Drop one image part from the history in place (the client-side half of image eviction)."""
    for m in history:
        if isinstance(m.get("content"), list):
            for i, part in enumerate(m["content"]):
                if part.get("type") == "image_url" and part["image_url"]["url"] == url:
                    del m["content"][i]
                    return True
    return False


# ---- coding tools (really executed) ------------------------------------------------------------
class Sandbox:
    """In-memory file system + calculator the tool scenarios execute against."""

    def __init__(self):
        self.files = {"notes.txt": "the launch code word is " + nonce()}

    SCHEMAS = [
        {"type": "function", "function": {"name": "read_file", "description": "Read a text file",
                                          "parameters": {"type": "object", "properties": {"path": {"type": "string"}}, "required": ["path"]}}},
        {"type": "function", "function": {"name": "write_file", "description": "Write a text file",
                                          "parameters": {"type": "object", "properties": {"path": {"type": "string"}, "text": {"type": "string"}},
                                                         "required": ["path", "text"]}}},
        {"type": "function", "function": {"name": "add", "description": "Add two integers",
                                          "parameters": {"type": "object", "properties": {"a": {"type": "integer"}, "b": {"type": "integer"}},
                                                         "required": ["a", "b"]}}},
    ]

    def run(self, call: dict) -> str:
        try:
            a = json.loads(call["arguments"] or "{}")
        except json.JSONDecodeError:
            return json.dumps({"error": "arguments are not JSON"})
        if call["name"] == "read_file":
            return json.dumps({"text": self.files.get(a.get("path", ""), None)})
        if call["name"] == "write_file":
            self.files[a.get("path", "")] = a.get("text", "")
            return json.dumps({"ok": True})
        if call["name"] == "add":
            return json.dumps({"sum": int(a.get("a", 0)) + int(a.get("b", 0))})
        return json.dumps({"error": f"unknown tool {call['name']}"})


class GuiAgent:
    """Simulated desktop: a solid-colour screen that actions change; every result attaches a screenshot."""

    W = H = 256
    ORDER = [png.PURPLE, png.RED, png.GREEN, png.BLUE, png.YELLOW]
    SCHEMAS = [{"type": "function", "function": {"name": n, "description": d, "parameters": {"type": "object", "properties": p}}}
               for n, d, p in (("screenshot", "Capture the screen", {}),
                               ("click", "Click at a position", {"x": {"type": "integer"}, "y": {"type": "integer"}}),
                               ("type_text", "Type text", {"text": {"type": "string"}}))]

    def __init__(self):
        self.screen, self.clicks, self.typed, self.actions = png.PURPLE, 0, "", 0

    def url(self) -> str:
        return png.data_url_png(self.W, self.H, self.screen)

    def run(self, call: dict) -> list:
        self.actions += 1
        if call["name"] == "click":
            self.clicks += 1
            self.screen = self.ORDER[self.clicks % len(self.ORDER)]
            text = "clicked"
        elif call["name"] == "type_text":
            try:
                self.typed += json.loads(call["arguments"] or "{}").get("text", "")
            except json.JSONDecodeError:
                pass
            text = "typed"
        else:
            text = "screenshot taken"
        # the trailing newline keeps the text/image boundary stable when the image is removed later
        return [{"type": "text", "text": text + "\n"}, image_part(self.url(), True), {"type": "text", "text": "End of tool result."}]


def tool_loop(ctx: Ctx, rep: Report, history: list, tools: list, run, session: str, max_rounds: int = 4, keep_images: int = 0):
    """Chat, execute tool calls, feed results back; optionally keep only the newest N images."""
    r = None
    for i in range(max_rounds):
        r = rep.turn(f"round{i}", ctx.client.chat(history, max_tokens=ctx.max_tokens, session=session, tools=tools))
        ensure(r.status == 200 and r.error is None, f"round {i}: {r.status} {r.error}")
        history.append(r.assistant_message())
        if not r.tool_calls:
            break
        for c in r.tool_calls:
            history.append({"role": "tool", "tool_call_id": c["id"], "content": run(c)})
        if keep_images:
            urls = [p["image_url"]["url"] for m in history if isinstance(m.get("content"), list)
                    for p in m["content"] if p.get("type") == "image_url"]
            for u in urls[:-keep_images]:
                remove_image(history, u)
    return r


# ---- scenarios ---------------------------------------------------------------------------------
def text_multiturn(ctx: Ctx, rep: Report):
    s, hist = ctx.session("text"), [{"role": "system", "content": "You are terse. " + nonce()}]
    prev_prompt = 0
    for i, q in enumerate(["Remember the word " + random.choice(WORDS) + ".", "What word did I ask you to remember?", "Spell it backwards."]):
        hist.append({"role": "user", "content": q})
        r = rep.turn(f"t{i}", ctx.client.chat(hist, max_tokens=ctx.max_tokens, session=s))
        ensure(r.status == 200 and r.error is None, f"turn {i}: {r.status} {r.error}")
        ensure(r.usage.get("prompt_tokens", 0) > prev_prompt, "prompt did not grow across turns")
        if i > 0:
            ensure(cached(r) > 0, f"turn {i}: no cached prefix in a same-session follow-up")
        prev_prompt = r.usage["prompt_tokens"]
        hist.append(r.assistant_message())


def tool_roundtrip(ctx: Ctx, rep: Report):
    sb = Sandbox()
    hist = [{"role": "user", "content": "Read notes.txt and tell me the launch code word."}]
    r = tool_loop(ctx, rep, hist, Sandbox.SCHEMAS, sb.run, ctx.session("tool"))
    if ctx.semantic:
        ensure(any("read_file" in t["tool_calls"] for t in rep.turns), "model never called read_file")
        ensure(sb.files["notes.txt"].split()[-1] in r.content, "answer does not contain the word from the file")


def vision_chat(ctx: Ctx, rep: Report):
    url = png.data_url_png(256, 256, png.GREEN)
    hist = [{"role": "user", "content": [{"type": "text", "text": "What colour is this image? One word."}, image_part(url, False)]}]
    r = rep.turn("vision", ctx.client.chat(hist, max_tokens=ctx.max_tokens, session=ctx.session("vis")))
    ensure(r.status == 200 and r.error is None, f"{r.status} {r.error}")
    if ctx.semantic:
        ensure("green" in r.content.lower(), f"expected green, got {r.content!r}")


def image_content_identity(ctx: Ctx, rep: Report):
    """Same pixels => prefix reuse; different pixels at the same position => no reuse past the image."""
    s = ctx.session("ident")
    q = lambda rgb: [{"role": "user", "content": [{"type": "text", "text": "Colour? " + tag}, image_part(png.data_url_png(128, 128, rgb), False)]}]
    tag = nonce()
    a = rep.turn("first", ctx.client.chat(q(png.RED), max_tokens=8, session=s))
    b = rep.turn("same", ctx.client.chat(q(png.RED), max_tokens=8, session=s))
    c = rep.turn("other", ctx.client.chat(q(png.BLUE), max_tokens=8, session=s))
    for r in (a, b, c):
        ensure(r.status == 200 and r.error is None, f"{r.status} {r.error}")
    ensure(cached(b) >= cached(c), "a different image reused more prefix than the identical one")


def mixed_tool_image(ctx: Ctx, rep: Report):
    g = GuiAgent()
    hist = [{"role": "user", "content": "Take a screenshot, then add 2 and 3."}]
    both = GuiAgent.SCHEMAS + Sandbox.SCHEMAS
    sb = Sandbox()
    tool_loop(ctx, rep, hist, both, lambda c: g.run(c) if c["name"] in ("screenshot", "click", "type_text") else sb.run(c),
              ctx.session("mixed"))


def gui_agent_screenshots(ctx: Ctx, rep: Report):
    g = GuiAgent()
    hist = [{"role": "system", "content": "You operate a desktop through tools. Look at screenshots before answering."},
            {"role": "user", "content": "Click once, then tell me the colour of the screen."}]
    r = tool_loop(ctx, rep, hist, GuiAgent.SCHEMAS, g.run, ctx.session("gui"), max_rounds=6, keep_images=3)
    n_img = sum(1 for m in hist if isinstance(m.get("content"), list) for p in m["content"] if p.get("type") == "image_url")
    ensure(n_img <= 3, f"window kept {n_img} images")
    if ctx.semantic:
        ensure(g.actions > 0, "model never used a tool")
        ensure(png.NAMES[g.screen] in r.content.lower(), f"expected {png.NAMES[g.screen]}, got {r.content!r}")


def gui_capability_prompt(ctx: Ctx, rep: Report):
    g = GuiAgent()
    hist = [{"role": "user", "content": "Can you see my screen? What is on it?"}]
    tool_loop(ctx, rep, hist, GuiAgent.SCHEMAS, g.run, ctx.session("cap"), max_rounds=3, keep_images=3)
    if ctx.semantic:
        ensure("screenshot" in rep.turns[0]["tool_calls"], "a capability question must call screenshot first")


def _delete_arm(ctx: Ctx, rep: Report, colours: list, drop: int, evict_marks: bool, with_tool: bool = False):
    """Build a conversation with several images, delete one, continue: the prefix before the deleted
    image stays cached, and with marks the engine removes the image's KV in place instead of
    re-prefilling what follows."""
    s, hist, urls = ctx.session("del"), [{"role": "system", "content": "Image log. " + nonce()}], []
    for i, rgb in enumerate(colours):
        u = png.data_url_png(128, 128, rgb, box=(8 * i, 8 * i, 8 * i + 40, 8 * i + 40))
        urls.append(u)
        hist.append({"role": "user", "content": [{"type": "text", "text": f"Image {i}.\n"}, image_part(u, evict_marks), {"type": "text", "text": "Noted?"}]})
        r = rep.turn(f"img{i}", ctx.client.chat(hist, max_tokens=8, session=s, tools=Sandbox.SCHEMAS if with_tool else None))
        ensure(r.status == 200 and r.error is None, f"image {i}: {r.status} {r.error}")
        hist.append(r.assistant_message())
        if with_tool and r.tool_calls:
            sb = Sandbox()
            for c in r.tool_calls:
                hist.append({"role": "tool", "tool_call_id": c["id"], "content": sb.run(c)})
    before = rep.turns[-1]["usage"].get("prompt_tokens", 0)
    ensure(remove_image(hist, urls[drop]), "image to delete not found")
    hist.append({"role": "user", "content": "How many images are left?"})
    r = rep.turn("after_delete", ctx.client.chat(hist, max_tokens=ctx.max_tokens, session=s))
    ensure(r.status == 200 and r.error is None, f"after delete: {r.status} {r.error}")
    ensure(cached(r) > 0, "nothing cached after deleting one image")
    rep.notes.update(prompt_before=before, prompt_after=r.usage.get("prompt_tokens"), cached_after=cached(r))
    log = ctx.log_text()
    if log and evict_marks:
        ensure("image_evict absorbed" in log, "server log shows no absorbed image deletion")


def image_delete_marked(ctx, rep): _delete_arm(ctx, rep, [png.RED, png.GREEN, png.BLUE], 0, True)
def image_delete_middle(ctx, rep): _delete_arm(ctx, rep, [png.RED, png.GREEN, png.BLUE], 1, True)
def image_delete_last_image(ctx, rep): _delete_arm(ctx, rep, [png.RED, png.GREEN, png.BLUE], 2, True)
def image_delete_with_tool_round(ctx, rep): _delete_arm(ctx, rep, [png.RED, png.GREEN], 0, True, with_tool=True)


def image_sliding_window(ctx: Ctx, rep: Report):
    g, s = GuiAgent(), ctx.session("slide")
    hist = [{"role": "user", "content": "Keep clicking and describing."}]
    for i in range(5):
        call = {"id": f"call_{i}", "name": "click", "arguments": "{}"}
        hist.append({"role": "assistant", "content": "", "tool_calls": [{"id": call["id"], "type": "function", "function": {"name": "click", "arguments": "{}"}}]})
        hist.append({"role": "tool", "tool_call_id": call["id"], "content": g.run(call)})
        urls = [p["image_url"]["url"] for m in hist if isinstance(m.get("content"), list) for p in m["content"] if p.get("type") == "image_url"]
        for u in urls[:-3]:
            remove_image(hist, u)
        r = rep.turn(f"slide{i}", ctx.client.chat(hist, max_tokens=8, session=s, tools=GuiAgent.SCHEMAS))
        ensure(r.status == 200 and r.error is None, f"slide {i}: {r.status} {r.error}")
        hist.append(r.assistant_message())
        if i > 0:
            ensure(cached(r) > 0, f"slide {i}: window shift lost the whole prefix")


def decode_vs_prefill(ctx: Ctx, rep: Report, long_words: int = 6000):
    """Session A streams (decode) while session B arrives with a long prompt (prefill): both finish,
    and A's largest inter-token gap stays bounded while B prefills."""
    out = {}

    def stream_a():
        out["a"] = ctx.client.chat([{"role": "user", "content": "Count upward slowly. " + nonce()}], max_tokens=max(128, ctx.max_tokens),
                                   session=ctx.session("dec"), ignore_eos=True)

    ta = threading.Thread(target=stream_a)
    ta.start()
    time.sleep(0.3)
    st, qf = ctx.client.get("/debug/queue")
    long_prompt = " ".join(random.choice(WORDS) for _ in range(long_words))
    b = ctx.client.chat([{"role": "user", "content": long_prompt + "\nSummarise."}], max_tokens=16, session=ctx.session("pre"))
    ta.join()
    a = out["a"]
    rep.turn("decode_side", a)
    rep.turn("prefill_side", b)
    ensure(a.status == 200 and a.error is None, f"decode side: {a.status} {a.error}")
    ensure(b.status == 200 and b.error is None, f"prefill side: {b.status} {b.error}")
    ensure(a.usage.get("completion_tokens", 0) >= 128, "decode side stopped early")
    rep.notes.update(mode="concurrent" if (qf or {}).get("active", 0) >= 1 else "queued", max_gap_ms=max(a.gaps_ms) if a.gaps_ms else 0.0,
                     prefill_ttft_ms=b.ttft_ms)
    ensure(rep.notes["max_gap_ms"] < 5000, f"decode stalled {rep.notes['max_gap_ms']:.0f} ms behind a prefill")


SUITES = {
    "core": [text_multiturn, tool_roundtrip, vision_chat, image_content_identity, mixed_tool_image, decode_vs_prefill],
    "text": [text_multiturn, tool_roundtrip, decode_vs_prefill],
    "gui": [gui_agent_screenshots],
    "gui-capability": [gui_capability_prompt],
    "image-evict": [image_delete_marked, image_delete_middle, image_delete_last_image, image_delete_with_tool_round, image_sliding_window],
}
SUITES["all"] = SUITES["core"] + SUITES["gui"] + SUITES["gui-capability"] + SUITES["image-evict"]


def run_suite(client: Client, suite: str, only: str | None = None, max_tokens: int = 64, semantic: bool = False,
              server_log: str | None = None, as_json: bool = False, out=print) -> bool:
    ctx, reports = Ctx(client, max_tokens, semantic, server_log), []
    for fn in SUITES[suite]:
        if only and fn.__name__ != only:
            continue
        rep = Report(fn.__name__)
        try:
            fn(ctx, rep)
        except Failed as e:
            rep.ok, rep.error = False, str(e)
        except (OSError, ValueError, KeyError) as e:
            rep.ok, rep.error = False, f"{type(e).__name__}: {e}"
        reports.append(rep)
        if not as_json:
            out(rep.line())
    if as_json:
        out(json.dumps([r.__dict__ for r in reports], indent=1))
    else:
        out(f"{sum(r.ok for r in reports)}/{len(reports)} scenarios passed")
    return all(r.ok for r in reports)
