"""The server probes (session identity, prefix reuse, keep-alive, lag) run against the whole serving stack on the CPU face."""
import asyncio
import threading

from owl_engine_b200.cli.client import Client
from owl_engine_b200.engine.core import Engine, EngineConfig
from owl_engine_b200.engine.service import EngineService
from owl_engine_b200.engine.tokenizer import ByteTokenizer
from owl_engine_b200.fixtures import server_probes as P
from owl_engine_b200.server.http import App, serve


def _serve(ecfg, running_kw):
    tok = ByteTokenizer()
    svc = EngineService(lambda: Engine(ecfg, device="cpu"), max_batch=4, running_kw=running_kw)
    client = svc.boot()
    loop = asyncio.new_event_loop()
    started, box = threading.Event(), {}

    def run():
        asyncio.set_event_loop(loop)

        async def main():
            app = App(client, tok, "test-hybrid")
            server = await serve(app, "127.0.0.1", 0)
            box["port"], box["app"] = server.sockets[0].getsockname()[1], app
            started.set()
            async with server:
                while not app.stop.is_set():
                    await asyncio.sleep(0.05)
        loop.run_until_complete(main())
    t = threading.Thread(target=run, daemon=True)
    t.start()
    started.wait(10)
    return svc, box, t


def test_probes_pass_against_the_cpu_face_server():
    tok = ByteTokenizer()
    ecfg = EngineConfig(model="test-hybrid", n_pages=1024, n_slots=6, n_snap_rows=8, max_seqs=6, max_seq=8192, prefill_chunk=256,
                        msg_open_ids=tuple(tok.encode("<|im_start|>")), snap_msg_min_gap=32, snap_msg_recent=4, snap_decode_stride=1)
    svc, box, t = _serve(ecfg, {"park_sessions": True, "max_parked": 6, "auto_sessions": True})
    try:
        c = Client(f"http://127.0.0.1:{box['port']}")
        rep = P.session_identity(c, "n1")
        assert rep["passed"], rep
        rep = P.prefix_reuse(c, "n2", words=120)
        assert all(r["ok"] for r in rep["criteria"][:4]), rep          # the timing criterion is a property of a real device
        rep = P.keep_alive(c)
        assert rep["passed"], rep
        rep = P.lag(c, "n3", long_words=300, stream_tokens=24, bound_ms=5000)
        assert rep["passed"], rep
    finally:
        box["app"].stop.set()
        t.join(5)
        assert svc.shutdown().code == 0
