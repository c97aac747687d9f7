"""``python -m owl_engine_b200.cli.main [--url U] [--max-tokens N] [--session K] [--model M]
[--workload core|text|gui|gui-capability|image-evict|all [--only NAME] [--semantic] [--json]
[--server-log PATH]]``.

Without ``--workload``: probe ``/health``, then a blocking REPL -- read a line, POST the whole
history with ``stream`` on, render deltas as they arrive (reasoning dimmed), repeat. The session
key stays fixed so the server reuses the conversation's KV. ``/new`` starts a fresh conversation,
``/help``, ``/quit``.

Reference counterpart: ``apps/cli/src/main.rs:1-32``.
"""
from __future__ import annotations

import argparse
import os
import sys
import time

from .client import Client
from .workload import SUITES, run_suite


def repl(client: Client, max_tokens: int, session: str, inp=sys.stdin, out=sys.stdout) -> int:
    st, h = client.health()
    if st != 200:
        print(f"server not healthy: {st}", file=sys.stderr)
        return 1
    _, models = client.get("/v1/models")
    out.write(f"connected: {models['data'][0]['id']} (session {session}); /new /help /quit\n")
    history = []
    while True:
        out.write("> ")
        out.flush()
        line = inp.readline()
        if not line or line.strip() == "/quit":
            return 0
        line = line.strip()
        if not line:
            continue
        if line == "/help":
            out.write("/new  start a fresh conversation\n/quit leave\n")
            continue
        if line == "/new":
            history, session = [], f"cli-{int(time.time() * 1e3)}"
            out.write(f"new session {session}\n")
            continue
        history.append({"role": "user", "content": line})

        def show(delta):
            if delta.get("reasoning_content"):
                out.write("\x1b[2m" + delta["reasoning_content"] + "\x1b[0m")
            if delta.get("content"):
                out.write(delta["content"])
            for t in delta.get("tool_calls", []):
                out.write(f"\n[tool call {t['function']['name']}({t['function']['arguments']})]")
            out.flush()

        r = client.chat(history, max_tokens=max_tokens, session=session, on_delta=show)
        if r.error:
            out.write(f"\n[error {r.status}: {r.error}]\n")
            history.pop()
            continue
        n = r.usage.get("completion_tokens", 0)
        rate = n / max(1e-9, (r.total_ms - r.ttft_ms) / 1e3) if n > 1 else 0.0
        out.write(f"\n[{n} tok, ttft {r.ttft_ms:.0f} ms, {rate:.1f} tok/s]\n")
        history.append(r.assistant_message())


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="owl-b200-cli")
    ap.add_argument("--url", default=os.environ.get("OWL_SERVER_URL", "http://127.0.0.1:8135"))
    ap.add_argument("--max-tokens", type=int, default=64)
    ap.add_argument("--session", default=f"cli-{int(time.time() * 1e3)}")
    ap.add_argument("--model")
    ap.add_argument("--workload", choices=sorted(SUITES))
    ap.add_argument("--only")
    ap.add_argument("--semantic", action="store_true", help="also assert on what the model says (needs a trained checkpoint)")
    ap.add_argument("--server-log")
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args(argv)
    client = Client(a.url, a.model)
    if a.workload:
        return 0 if run_suite(client, a.workload, a.only, a.max_tokens, a.semantic, a.server_log, a.json) else 1
    return repl(client, a.max_tokens, a.session)


if __name__ == "__main__":
    sys.exit(main())
