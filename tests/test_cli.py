"""CLI pieces without a GPU: PNG writer round trip, blocking client + workload harness against a scripted server."""
import asyncio
import io
import threading

import numpy as np

from owl_engine_b200.cli import png
from owl_engine_b200.cli.client import Client
from owl_engine_b200.cli.main import repl
from owl_engine_b200.cli.workload import remove_image, run_suite
from owl_engine_b200.engine.tokenizer import ByteTokenizer
from owl_engine_b200.server.http import App, serve
from test_server_http import FakeClient


def test_png_round_trip():
    data = png.encode_png(40, 24, png.BLUE, box=(4, 4, 20, 12), box_rgb=(1, 2, 3))
    img = png.decode_png(data)
    assert img.shape == (24, 40, 3)
    assert tuple(img[0, 0]) == png.BLUE and tuple(img[5, 5]) == (1, 2, 3) and tuple(img[12, 5]) == png.BLUE
    assert png.data_url_png(8, 8, png.RED).startswith("data:image/png;base64,iVBOR")


def test_remove_image():
    h = [{"role": "user", "content": [{"type": "text", "text": "a"}, {"type": "image_url", "image_url": {"url": "u1"}}]}]
    assert remove_image(h, "u1") and not remove_image(h, "u1") and len(h[0]["content"]) == 1


class Server:
    def __enter__(self):
        self.loop = asyncio.new_event_loop()
        tok = ByteTokenizer()
        self.app_client = FakeClient(tok, "ok <tool_call>\n{\"name\": \"add\", \"arguments\": {\"a\": 2, \"b\": 3}}\n</tool_call>")
        ready = threading.Event()

        def run():
            asyncio.set_event_loop(self.loop)
            app = App(self.app_client, tok, "fake")
            self.server = self.loop.run_until_complete(serve(app, "127.0.0.1", 0))
            self.port = self.server.sockets[0].getsockname()[1]
            ready.set()
            self.loop.run_forever()
        self.t = threading.Thread(target=run, daemon=True)
        self.t.start()
        ready.wait(10)
        return self

    def __exit__(self, *a):
        self.loop.call_soon_threadsafe(self.loop.stop)
        self.t.join(5)


def test_client_and_workload_against_scripted_server():
    with Server() as s:
        c = Client(f"http://127.0.0.1:{s.port}")
        assert c.health()[0] == 200
        r = c.chat([{"role": "user", "content": "hi"}], max_tokens=200)
        assert r.content == "ok " and r.tool_calls[0]["name"] == "add" and r.finish_reason == "tool_calls"
        assert r.usage["completion_tokens"] > 0 and r.ttft_ms > 0
        r2 = c.chat([{"role": "user", "content": "hi"}], max_tokens=200, stream=False)
        assert r2.content == r.content and r2.tool_calls == r.tool_calls
        lines = []
        ok = run_suite(c, "text", only="tool_roundtrip", max_tokens=200, out=lines.append)
        assert ok and lines[0].startswith("[PASS] tool_roundtrip")
        out = io.StringIO()
        assert repl(c, 200, "s", inp=io.StringIO("hello\n/new\n/quit\n"), out=out) == 0
        assert "ok " in out.getvalue() and "tool call add" in out.getvalue()


def test_needle_and_ladder_fixtures_against_scripted_server():
    from owl_engine_b200.fixtures import needle

    with Server() as s:
        c = Client(f"http://127.0.0.1:{s.port}")
        rows = needle.run_needle(c, [50], [0.5])
        assert rows[0]["hit_rate"] == 0.0 and rows[0]["words"] == 50        # the scripted reply never contains the value
        lad = needle.run_ladder(c, [30], new_tokens=8)
        assert lad[0]["error"] is None and lad[0]["prompt_tokens"] > 30


def test_png_decoder_reads_every_filter_and_refuses_damaged_files():
    """Images come from clients: all five row filters decode (checked against rows filtered here, independently of the
    writer), and truncated, flipped or lying files raise ValueError before anything large is allocated."""
    import random
    import struct
    import zlib

    import numpy as np
    import pytest

    from owl_engine_b200.cli import png

    rng = np.random.default_rng(0)
    h, w, bpp = 20, 30, 3
    img = rng.integers(0, 256, (h, w, bpp), dtype=np.uint8)

    def paeth(a, b, c):
        p = a + b - c
        pa, pb, pc = abs(p - a), abs(p - b), abs(p - c)
        return a if pa <= pb and pa <= pc else (b if pb <= pc else c)
    raw, prev = bytearray(), np.zeros(w * bpp, dtype=np.int32)
    for y in range(h):
        f, line = y % 5, img[y].reshape(-1).astype(np.int32)
        enc = np.zeros_like(line)
        for i in range(w * bpp):
            a, b, c = (line[i - bpp] if i >= bpp else 0), prev[i], (prev[i - bpp] if i >= bpp else 0)
            enc[i] = (line[i] - {0: 0, 1: a, 2: b, 3: (a + b) // 2, 4: paeth(a, b, c)}[f]) & 255
        raw.append(f)
        raw += enc.astype(np.uint8).tobytes()
        prev = line
    chunk = lambda t, b: struct.pack(">I", len(b)) + t + b + struct.pack(">I", zlib.crc32(t + b) & 0xFFFFFFFF)
    sig = bytes([0x89]) + b"PNG" + bytes([13, 10, 26, 10])
    good = sig + chunk(b"IHDR", struct.pack(">IIBBBBB", w, h, 8, 2, 0, 0, 0)) + chunk(b"IDAT", zlib.compress(bytes(raw))) + chunk(b"IEND", b"")
    assert np.array_equal(png.decode_png(good), img)
    huge = sig + chunk(b"IHDR", struct.pack(">IIBBBBB", 2 ** 31 - 1, 2 ** 31 - 1, 8, 2, 0, 0, 0)) + chunk(b"IDAT", zlib.compress(b"x"))
    with pytest.raises(ValueError, match="sides must be"):
        png.decode_png(huge)
    bomb = sig + chunk(b"IHDR", struct.pack(">IIBBBBB", 4, 4, 8, 2, 0, 0, 0)) + chunk(b"IDAT", zlib.compress(bytes(50_000_000)))
    with pytest.raises(ValueError, match="inflates to"):
        png.decode_png(bomb)                                # a small header with a large stream behind it is cut off, not inflated
    rnd = random.Random(3)
    for _ in range(600):
        b = bytearray(good)
        mode = rnd.randrange(3)
        if mode == 0:
            b = b[:rnd.randrange(len(b))]
        elif mode == 1:
            for _ in range(rnd.randrange(1, 5)):
                b[rnd.randrange(len(b))] = rnd.randrange(256)
        else:
            b = bytearray(rnd.randbytes(rnd.randrange(0, 120)))
        try:
            out = png.decode_png(bytes(b))
            assert out.shape[2] == 3
        except ValueError:
            pass
