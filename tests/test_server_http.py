"""HTTP surface against a fake engine client (no GPU): SSE framing, tool calls, errors, debug routes."""
import asyncio
import json
import queue
import threading

from owl_engine_b200.engine.tokenizer import ByteTokenizer
from owl_engine_b200.server.http import App, serve


class FakeClient:
    """Echoes a scripted completion token by token."""

    def __init__(self, tok, script: str):
        self.tok, self.script, self.cancelled = tok, script, []

    def chat(self, tokens, opts):
        sink = queue.Queue()
        ids = self.tok.encode(self.script)[:opts.max_new]
        def feed():
            sink.put(("prefill", 0, len(tokens), len(tokens)))
            for t in ids:
                sink.put(("token", 0, t))
            sink.put(("completed", 0, "stop", {"prompt_tokens": len(tokens), "completion_tokens": len(ids), "cached_tokens": 16}))
        threading.Thread(target=feed, daemon=True).start()
        return 0, sink

    def cancel(self, turn): self.cancelled.append(turn)
    def queue_facts(self): return {"queued": 0}
    def query(self, fn): return {}


async def request(port, method, path, body=None):
    r, w = await asyncio.open_connection("127.0.0.1", port)
    data = json.dumps(body).encode() if body is not None else b""
    w.write(f"{method} {path} HTTP/1.1\r\nHost: x\r\nContent-Length: {len(data)}\r\nConnection: close\r\n\r\n".encode() + data)
    await w.drain()
    raw = await r.read()
    w.close()
    head, _, payload = raw.partition(b"\r\n\r\n")
    return int(head.split()[1]), head.decode(), payload


def dechunk(payload: bytes) -> str:
    out, i = b"", 0
    while i < len(payload):
        j = payload.index(b"\r\n", i)
        n = int(payload[i:j], 16)
        if n == 0:
            break
        out += payload[j + 2:j + 2 + n]
        i = j + 2 + n + 2
    return out.decode()


def test_http_surface():
    async def main():
        tok = ByteTokenizer()
        script = '<think>hm</think>Hello <tool_call>\n{"name": "f", "arguments": {"a": 1}}\n</tool_call>'
        app = App(FakeClient(tok, script), tok, "test-model")
        server = await serve(app, "127.0.0.1", 0)
        port = server.sockets[0].getsockname()[1]
        async with server:
            st, _, body = await request(port, "GET", "/health")
            assert st == 200 and json.loads(body)["status"] == "ok"
            st, _, body = await request(port, "GET", "/v1/models")
            assert json.loads(body)["data"][0]["id"] == "test-model"
            st, _, body = await request(port, "POST", "/tokenize", {"text": "ab"})
            assert json.loads(body)["tokens"] == [97, 98]
            msgs = [{"role": "user", "content": "hi"}]
            st, _, body = await request(port, "POST", "/v1/chat/completions", {"messages": msgs, "max_tokens": 200})
            resp = json.loads(body)
            m = resp["choices"][0]["message"]
            assert st == 200 and m["content"] == "Hello " and m["reasoning_content"] == "hm"
            assert m["tool_calls"][0]["function"]["name"] == "f" and resp["choices"][0]["finish_reason"] == "tool_calls"
            assert resp["usage"]["prompt_tokens_details"]["cached_tokens"] == 16
            st, head, body = await request(port, "POST", "/v1/chat/completions",
                                           {"messages": msgs, "stream": True, "stream_options": {"include_usage": True}})
            assert st == 200 and "text/event-stream" in head
            events = [l[6:] for l in dechunk(body).split("\n\n") if l.startswith("data: ")]
            assert events[-1] == "[DONE]"
            chunks = [json.loads(e) for e in events[:-1]]
            assert "".join(c["choices"][0]["delta"].get("content", "") for c in chunks) == "Hello "
            assert any("tool_calls" in c["choices"][0]["delta"] for c in chunks) and "usage" in chunks[-1]
            st, _, body = await request(port, "POST", "/v1/chat/completions", {"messages": []})
            assert st == 400
            st, _, body = await request(port, "POST", "/v1/chat/completions", {"messages": msgs, "stop": ["llo"]})
            assert json.loads(body)["choices"][0]["message"]["content"] == "He"
            st, _, _ = await request(port, "GET", "/debug/queue")
            assert st == 200
            st, _, body = await request(port, "POST", "/debug/step", {"mode": "off"})
            assert json.loads(body)["mode"] == "off"
            st, _, _ = await request(port, "GET", "/nope")
            assert st == 404
    asyncio.run(main())


def test_owl_evict_marks_become_droppable_spans_and_refusals_are_400():
    """An image part with ``owl_evict: true`` reaches the engine as a token span that covers the image's pad run and its
    vision-start / vision-end markers; an engine that refuses the marks (image_evict off) yields a 400 with the reason."""
    import base64

    from owl_engine_b200.cli import png
    from owl_engine_b200.models import vision as V
    from owl_engine_b200.server.http import Vision

    class Recorder(FakeClient):
        def __init__(self, tok, script, refuse=False):
            super().__init__(tok, script)
            self.seen, self.refuse = [], refuse

        def chat(self, tokens, opts):
            if self.refuse and opts.evict_spans:
                raise ValueError("rejected: segments are marked droppable (owl_evict) but image_evict is off in this profile")
            self.seen.append((list(tokens), opts))
            return super().chat(tokens, opts)

    async def main():
        tok = ByteTokenizer()
        vis = Vision(V.VisionTower(V.tiny_vision(out_hidden=64)), tok.image_pad_id)
        url = "data:image/png;base64," + base64.b64encode(png.encode_png(96, 64, png.RED)).decode()
        body = {"model": "m", "max_tokens": 4, "messages": [{"role": "user", "content": [
            {"type": "text", "text": "look"}, {"type": "image_url", "image_url": {"url": url}, "owl_evict": True},
            {"type": "image_url", "image_url": {"url": url}}, {"type": "text", "text": "done"}]}]}
        out = {}
        for name, refuse in (("ok", False), ("refused", True)):
            client = Recorder(tok, "hi", refuse)
            app = App(client, tok, "test-model", vision=vis)
            server = await serve(app, "127.0.0.1", 0)
            port = server.sockets[0].getsockname()[1]
            out[name] = (await request(port, "POST", "/v1/chat/completions", body), client)
            server.close()
            await server.wait_closed()
        return out

    out = asyncio.run(main())
    (code, _, payload), client = out["ok"]
    assert code == 200, payload
    tokens, opts = client.seen[0]
    tok = ByteTokenizer()
    assert len(opts.images) == 2 and len(opts.evict_spans) == 1                  # only the marked image is droppable
    lo, hi = opts.evict_spans[0]
    n = opts.images[0][0].shape[0]
    assert hi - lo == n + 2 and tokens[lo] == tok.special_ids["<|vision_start|>"] and tokens[hi - 1] == tok.special_ids["<|vision_end|>"]
    assert tokens[lo + 1:hi - 1] == [tok.image_pad_id] * n and opts.image_pad_id == tok.image_pad_id
    (code, _, payload), _ = out["refused"]
    assert code == 400 and b"image_evict" in payload
