"""Gates against a RUNNING server (HTTP only): each probe prints its criteria with pass / fail and the exit code says whether
all passed (0), a criterion failed (2) or a request failed (1).

    session-identity   conversations WITHOUT a ``session`` key are recognised by content: a second conversation does not join
                       the first one's session although both start with the same chat-template preamble; follow-up turns
                       find their own session; an explicit key is sticky. Judged on the session table of ``/debug/vram``,
                       not on ``cached_tokens`` alone (the content-addressed tree hits across sessions too).
    prefix-reuse       the same long prompt twice: the second is served from the cache (cached tokens, shorter time to the
                       first token); a prompt that shares only the system message reuses up to the message boundary.
    keep-alive         many requests over ONE connection (HTTP/1.1 keep-alive), then an SSE stream on the same connection.
    lag                while a long prompt prefills, a running stream's largest gap between tokens stays bounded (the
                       scheduler grants one prefill chunk per few decode beats).

``python -m owl_engine_b200.fixtures.server_probes --url http://127.0.0.1:8137 session-identity``

Reference counterpart: ``apps/server/tests/{session_identity_probe,prefix_reuse_probe,keep_alive_probe,lag_probe}.py``.
"""
from __future__ import annotations

import argparse
import http.client
import json
import sys
import threading
import time

from ..cli.client import Client


class Gate:
    def __init__(self, name: str):
        self.name, self.rows = name, []

    def check(self, ok: bool, what: str) -> bool:
        self.rows.append((bool(ok), what))
        return bool(ok)

    def report(self) -> dict:
        return {"probe": self.name, "passed": all(ok for ok, _ in self.rows),
                "criteria": [{"ok": ok, "what": what} for ok, what in self.rows]}


def _sessions(c: Client) -> list:
    st, v = c.get("/debug/vram")
    if st != 200:
        raise RuntimeError(f"/debug/vram answered {st}")
    return [s["session"] for s in v.get("sessions", [])]


def _cached(rep) -> int:
    u = rep.usage or {}
    return int(u.get("prompt_tokens_details", {}).get("cached_tokens", u.get("cached_tokens", 0)))


def _turn(c: Client, msgs: list, text: str, max_tokens: int, **kw):
    msgs.append({"role": "user", "content": text})
    rep = c.chat(msgs, max_tokens=max_tokens, stream=False, temperature=0, **kw)
    if rep.error:
        raise RuntimeError(rep.error)
    msgs.append({"role": "assistant", "content": rep.content})
    return rep


def session_identity(c: Client, nonce: str, max_tokens: int = 8) -> dict:
    g = Gate("session-identity")
    base = set(_sessions(c))
    new = lambda: set(_sessions(c)) - base
    a, b, k = [], [], []
    _turn(c, a, f"[{nonce}] conversation A: tell me about rivers, lakes and the sea in one long paragraph.", max_tokens)
    g.check(len(new()) == 1, "A1 opens one session")
    _turn(c, b, f"[{nonce}] conversation B: list some prime numbers and explain why they are prime.", max_tokens)
    g.check(len(new()) == 2, "B1 opens a second session (the shared template preamble does not join it to A)")
    ra2 = _turn(c, a, "and mountains?", max_tokens)
    g.check(len(new()) == 2, "A2 finds A's session (no new one)")
    ra3 = _turn(c, a, "and deserts?", max_tokens)
    g.check(len(new()) == 2, "A3 finds A's session")
    rb2 = _turn(c, b, "and composite numbers?", max_tokens)
    g.check(len(new()) == 2, "B2 finds B's session")
    _turn(c, k, f"[{nonce}] conversation C with an explicit key.", max_tokens, session=f"probe-{nonce}")
    g.check(f"probe-{nonce}" in new() and len(new()) == 3, "C1 opens the named session")
    rc2 = _turn(c, k, "go on.", max_tokens, session=f"probe-{nonce}")
    g.check(len(new()) == 3, "C2 stays in the named session")
    g.check(_cached(ra2) > 0 and _cached(ra3) >= _cached(ra2), f"A's cached tokens grow over the turns ({_cached(ra2)} -> {_cached(ra3)})")
    g.check(_cached(rb2) > 0, f"B2 is served from B's history ({_cached(rb2)} cached)")
    g.check(_cached(rc2) > 0, f"C2 is served from C's history ({_cached(rc2)} cached)")
    return g.report()


def prefix_reuse(c: Client, nonce: str, words: int = 400, max_tokens: int = 8) -> dict:
    g = Gate("prefix-reuse")
    system = f"[{nonce}] " + " ".join(f"rule{i}" for i in range(words))
    ask = lambda user: c.chat([{"role": "system", "content": system}, {"role": "user", "content": user}], max_tokens=max_tokens,
                              temperature=0)
    r1 = ask("first question")
    r2 = ask("first question")
    r3 = ask("a different question about the same rules")
    for r in (r1, r2, r3):
        if r.error:
            raise RuntimeError(r.error)
    n = r1.usage.get("prompt_tokens", 0)
    g.check(_cached(r1) == 0, "the first request is cold")
    g.check(_cached(r2) >= n - 48, f"the repeated prompt is served from the cache ({_cached(r2)} of {n} tokens)")
    g.check(r2.content == r1.content, "and produces the same completion")
    g.check(_cached(r3) >= n // 2, f"another user message reuses the system message ({_cached(r3)} tokens)")
    g.check(r2.ttft_ms < r1.ttft_ms, f"time to first token drops ({r1.ttft_ms:.0f} -> {r2.ttft_ms:.0f} ms)")
    return g.report()


def keep_alive(c: Client, n: int = 6) -> dict:
    g = Gate("keep-alive")
    conn = http.client.HTTPConnection(c.hostport, timeout=c.timeout)
    ok = 0
    for i in range(n):
        conn.request("POST", "/v1/chat/completions", json.dumps({"messages": [{"role": "user", "content": f"ping {i}"}],
                                                                 "max_tokens": 4}), {"Content-Type": "application/json"})
        r = conn.getresponse()
        body = r.read()
        ok += int(r.status == 200 and b"choices" in body)
    g.check(ok == n, f"{ok} of {n} requests answered over one connection")
    conn.request("GET", "/health")
    r = conn.getresponse()
    r.read()
    g.check(r.status == 200, "a GET on the same connection")
    conn.request("POST", "/v1/chat/completions", json.dumps({"messages": [{"role": "user", "content": "stream"}], "max_tokens": 6,
                                                             "stream": True}), {"Content-Type": "application/json"})
    r = conn.getresponse()
    body = r.read()
    g.check(r.status == 200 and b"[DONE]" in body, "an SSE stream on the same connection ends with [DONE]")
    conn.close()
    return g.report()


def lag(c: Client, nonce: str, long_words: int = 3000, stream_tokens: int = 96, bound_ms: float = 2000.0) -> dict:
    g = Gate("lag")
    out = {}

    def streamer():
        out["rep"] = c.chat([{"role": "user", "content": f"[{nonce}] count slowly"}], max_tokens=stream_tokens, ignore_eos=True,
                            temperature=0)
    t = threading.Thread(target=streamer)
    t.start()
    time.sleep(0.2)
    big = c.chat([{"role": "user", "content": f"[{nonce}] " + " ".join(f"w{i}" for i in range(long_words))}], max_tokens=4,
                 temperature=0)
    t.join()
    rep = out["rep"]
    if rep.error or big.error:
        raise RuntimeError(rep.error or big.error)
    worst = max(rep.gaps_ms) if rep.gaps_ms else 0.0
    g.check(rep.usage.get("completion_tokens", 0) == stream_tokens, "the stream ran to its length while the long prompt was served")
    g.check(worst <= bound_ms, f"largest gap between tokens {worst:.0f} ms (bound {bound_ms:.0f} ms)")
    g.check(big.usage.get("prompt_tokens", 0) > long_words, "the long prompt was admitted and answered")
    return g.report()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--url", default="http://127.0.0.1:8137")
    ap.add_argument("--model", default=None)
    ap.add_argument("probe", choices=["session-identity", "prefix-reuse", "keep-alive", "lag", "all"])
    a = ap.parse_args(argv)
    c = Client(a.url, a.model)
    nonce = f"{time.time_ns() % 10**9:09d}"
    runs = {"session-identity": lambda: session_identity(c, nonce), "prefix-reuse": lambda: prefix_reuse(c, nonce),
            "keep-alive": lambda: keep_alive(c), "lag": lambda: lag(c, nonce)}
    reports = []
    try:
        for name in (runs if a.probe == "all" else [a.probe]):
            reports.append(runs[name]())
    except (RuntimeError, OSError) as ex:
        print(json.dumps({"error": str(ex), "reports": reports}))
        return 1
    print(json.dumps(reports, indent=1))
    return 0 if all(r["passed"] for r in reports) else 2


if __name__ == "__main__":
    sys.exit(main())
