"""The HTTP surface under hostile input: whatever a client sends as a chat request, the answer is 200, 400, 404 or 429, never a
500 or a dead connection, and the server keeps serving."""
import asyncio
import json
import threading

from hypothesis import HealthCheck, given, settings, strategies as st

from owl_engine_b200.engine.core import Engine, EngineConfig
from owl_engine_b200.engine.service import EngineService
from owl_engine_b200.engine.tokenizer import ByteTokenizer
from owl_engine_b200.server.http import App, serve

_server = {}


def server():
    if not _server:
        tok = ByteTokenizer()
        ecfg = EngineConfig(model="test-hybrid", n_pages=256, n_slots=4, n_snap_rows=2, max_seqs=4, max_seq=2048, prefill_chunk=128)
        svc = EngineService(lambda: Engine(ecfg, device="cpu"), max_batch=4)
        client = svc.boot()
        loop, started = asyncio.new_event_loop(), threading.Event()

        def run():
            asyncio.set_event_loop(loop)

            async def main():
                app = App(client, tok, "test-hybrid", max_new_cap=64)
                srv = await serve(app, "127.0.0.1", 0)
                _server.update(port=srv.sockets[0].getsockname()[1], app=app, svc=svc)
                started.set()
                async with srv:
                    while not app.stop.is_set():
                        await asyncio.sleep(0.05)
            loop.run_until_complete(main())
        threading.Thread(target=run, daemon=True).start()
        started.wait(10)
    return _server


def post(port, raw: bytes, path="/v1/chat/completions"):
    import http.client

    c = http.client.HTTPConnection("127.0.0.1", port, timeout=30)
    c.request("POST", path, raw, {"Content-Type": "application/json"})
    r = c.getresponse()
    body = r.read()
    c.close()
    return r.status, body


scalar = st.one_of(st.none(), st.booleans(), st.integers(-10 ** 6, 10 ** 6), st.floats(allow_nan=False, allow_infinity=False, width=32),
                   st.text(max_size=20))
anything = st.recursive(scalar, lambda c: st.one_of(st.lists(c, max_size=3), st.dictionaries(st.text(max_size=6), c, max_size=3)), max_leaves=6)
message = st.fixed_dictionaries({}, optional={
    "role": st.one_of(st.sampled_from(["system", "user", "assistant", "tool", "alien"]), anything),
    "content": st.one_of(st.text(max_size=40), st.lists(st.fixed_dictionaries({}, optional={
        "type": st.sampled_from(["text", "image_url", "audio"]), "text": anything, "image_url": anything}), max_size=3), anything),
    "tool_calls": anything, "name": anything})
body = st.fixed_dictionaries({}, optional={
    "messages": st.one_of(st.lists(message, max_size=4), anything), "max_tokens": st.one_of(st.integers(-5, 500), anything),
    # the CPU face has no sampler kernels: numeric temperatures stay at 0 (greedy), other types must be refused
    "stream": st.one_of(st.booleans(), anything), "temperature": st.one_of(st.just(0), st.text(max_size=3), st.lists(scalar, max_size=2)),
    "top_p": st.one_of(st.none(), st.text(max_size=3)), "top_k": st.one_of(st.none(), st.text(max_size=3)), "seed": anything,
    "stop": anything, "tools": anything, "session": anything, "ignore_eos": anything, "chat_template_kwargs": anything,
    "reasoning_effort": anything, "stream_options": anything, "model": anything})


@settings(max_examples=150, deadline=None, suppress_health_check=[HealthCheck.too_slow])
@given(body)
def test_any_chat_body_gets_a_client_error_or_an_answer(b):
    s = server()
    status, raw = post(s["port"], json.dumps(b).encode())
    assert status in (200, 400, 429), (status, raw[:300], b)
    if status != 200 or not b.get("stream"):
        assert isinstance(json.loads(raw), dict)
    status, raw = post(s["port"], json.dumps({"messages": [{"role": "user", "content": "still there?"}], "max_tokens": 2}).encode())
    assert status == 200 and s["svc"].exit is None


@settings(max_examples=60, deadline=None, suppress_health_check=[HealthCheck.too_slow])
@given(st.binary(max_size=200), st.sampled_from(["/v1/chat/completions", "/tokenize", "/debug/log", "/debug/step", "/debug/load", "/nope"]))
def test_bytes_that_are_not_json_never_take_the_server_down(raw, path):
    s = server()
    status, _ = post(s["port"], raw, path)
    assert status in (200, 400, 404, 405), (status, raw, path)
    assert post(s["port"], json.dumps({"messages": [{"role": "user", "content": "ok"}], "max_tokens": 1}).encode())[0] == 200


@settings(max_examples=80, deadline=None, suppress_health_check=[HealthCheck.too_slow])
@given(st.one_of(st.binary(max_size=120),
                 st.builds(lambda m, p, h, b: f"{m} {p} HTTP/1.1\r\n{h}\r\n\r\n".encode("latin1", "replace") + b,
                           st.sampled_from(["GET", "POST", "PUT", "", "G E T"]), st.text("/abc?%", max_size=12),
                           st.sampled_from(["Content-Length: 5", "Content-Length: -1", "Content-Length: x", "Content-Length: 99999999999",
                                            "Host: x", ": novalue", "A" * 300]), st.binary(max_size=40))))
def test_raw_bytes_on_the_socket_never_take_the_listener_down(raw):
    import socket

    s = server()
    with socket.create_connection(("127.0.0.1", s["port"]), timeout=5) as c:
        c.sendall(raw)
        c.shutdown(socket.SHUT_WR)
        c.settimeout(5)
        try:
            while c.recv(4096):
                pass
        except (TimeoutError, ConnectionError, OSError):
            pass
    assert post(s["port"], json.dumps({"messages": [{"role": "user", "content": "ok"}], "max_tokens": 1}).encode())[0] == 200
