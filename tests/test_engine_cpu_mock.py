"""The engine on the CPU face: boot, budget refusal, prefix reuse, tier round trips and agent sessions without a GPU.

The stand-in model (``engine/cpu_mock.py``) makes every next token depend on the sequence's recurrent state row and on a
mark in every page of its context, so these tests fail if the host logic adopts, moves or drops the wrong bytes."""
import pytest
import torch

from owl_engine_b200.engine.core import Engine, EngineConfig
from owl_engine_b200.engine.running import RunningEngine, TurnOpts
from owl_engine_b200.utils.cpuface import CaptureUnsupported, MockLimits
from owl_engine_b200.utils.ledger import BudgetError


def cfg(**kw):
    base = dict(model="test-hybrid", n_pages=64, n_slots=4, n_snap_rows=3, max_seqs=4, max_seq=512, prefill_chunk=64)
    base.update(kw)
    return EngineConfig(**base)


def toks(n, seed=0, vocab=500):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def test_boot_generates_deterministically_and_counts_pages():
    a, b = Engine(cfg(), device="cpu"), Engine(cfg(), device="cpu")
    p = toks(70)
    out = a.generate(p, 20)
    assert out == b.generate(p, 20) and len(set(out)) > 5
    assert a.kv.free_pages + a.kv.stats()["device_nodes"] == a.cfg.n_pages          # nothing leaked
    assert a.runner.launches == 70 + 19


def test_vram_limit_refuses_the_boot_loudly():
    with pytest.raises(BudgetError) as ei:
        Engine(cfg(n_pages=4096), device="cpu", limits=MockLimits(vram_bytes=8 << 20))
    assert "kv pool" in str(ei.value) and "MiB" in str(ei.value)
    Engine(cfg(), device="cpu", limits=MockLimits(vram_bytes=1 << 30))            # and a pool that fits is accepted


def test_prefix_hit_restores_state_and_pages():
    e = Engine(cfg(), device="cpu")
    p = toks(100, 1)
    want = e.generate(p + toks(9, 2), 12)
    assert e.prefix_hits == 0
    again = e.generate(p + toks(9, 2), 12)                # same prompt: adopted up to the snapshot boundary
    assert again == want and e.prefix_hits == 1
    sid = e.add_sequence(p + toks(30, 3))                 # shares only the first 100 tokens
    assert e.seqs[sid].reused == 0 or e.seqs[sid].reused % 16 == 0
    e.free_sequence(sid, publish=False)


def test_pressure_demotes_to_the_host_tier_and_replays_promote_back(tmp_path):
    e = Engine(cfg(n_pages=24, host_cache_mb=1, disk_cache_mb=4, disk_dir=str(tmp_path)), device="cpu")
    prompts = [toks(150, 10 + i) for i in range(3)]      # 9 full blocks each: the third one pushes the oldest tails to the host
    first = [e.generate(p, 6) for p in prompts]
    assert e.rel.demoted > 0 and e.kv.stats()["device_nodes"] < e.kv.stats()["nodes"]
    hits0 = e.prefix_hits
    for p, w in zip(prompts, first):                      # every prompt again: demoted blocks are promoted, the state row restored
        sid = e.add_sequence(p)
        assert e.seqs[sid].reused == 144
        out = [e.prefill(sid)]
        while len(out) < 6:
            out.append(e.decode_step([sid])[0])
        e.free_sequence(sid)
        assert out == w
    assert e.prefix_hits == hits0 + 3
    # a restart adopts what the disk tier and its index hold
    e.checkpoint()
    e.close()
    e2 = Engine(cfg(n_pages=24, host_cache_mb=1, disk_cache_mb=4, disk_dir=str(tmp_path)), device="cpu")
    assert e2.adopted["blocks"] > 0
    assert e2.generate(prompts[2], 6) == first[2]


def test_parked_session_resume_and_leave_gap_drop():
    e = Engine(cfg(n_pages=96), device="cpu")
    re_ = RunningEngine(e, max_batch=2, park_sessions=True, max_parked=2, evict_pad_id=499)
    hist = toks(80, 20)
    out = re_.generate(hist, TurnOpts(max_new=5, ignore_eos=True, session="s"))
    hist += out
    img = [498] * 32                                      # a droppable segment (client coordinates)
    new = toks(10, 21) + img + toks(7, 22)
    spans = [(len(hist) + 10, len(hist) + 42)]
    hist2 = hist + new
    out2 = re_.generate(hist2, TurnOpts(max_new=5, ignore_eos=True, session="s", evict_spans=spans))
    assert re_.resumed == 1
    hist2 += out2
    # the client drops the segment: the engine unlinks its pages instead of recomputing the history
    lo, hi = spans[0]
    hist3 = hist2[:lo] + hist2[hi:] + toks(6, 23)
    launches0 = e.runner.launches
    out3 = re_.generate(hist3, TurnOpts(max_new=4, ignore_eos=True, session="s"))
    assert re_.resumed == 2 and re_.gap_drops == 1 and len(out3) == 4
    assert e.runner.launches - launches0 < 20             # only the new tail ran, not the history


def test_capture_limit_surfaces():
    e = Engine(cfg(), device="cpu", limits=MockLimits(graph_capture=False))
    sid = e.add_sequence(toks(20))
    e.prefill(sid)
    with pytest.raises(CaptureUnsupported):
        e.decode_step([sid])


def test_http_server_end_to_end_on_the_cpu_face():
    """The whole serving stack without a GPU: HTTP surface -> engine service thread -> RunningEngine -> engine on the CPU face.
    Non-stream and SSE agree, the debug endpoints answer, an identical prompt is served from the prefix tree."""
    import asyncio
    import json

    from owl_engine_b200.engine.service import EngineService
    from owl_engine_b200.engine.tokenizer import ByteTokenizer
    from owl_engine_b200.server.http import App, serve
    from test_server_http import dechunk, request

    svc = EngineService(lambda: Engine(cfg(n_pages=128), device="cpu"), max_batch=4)
    client = svc.boot()
    tok = ByteTokenizer()

    async def main():
        app = App(client, tok, "test-hybrid")
        server = await serve(app, "127.0.0.1", 0)
        port = server.sockets[0].getsockname()[1]
        async with server:
            body = {"messages": [{"role": "user", "content": "hello there, cpu face"}], "max_tokens": 12, "ignore_eos": True}
            st, _, a = await request(port, "POST", "/v1/chat/completions", body)
            assert st == 200
            ra = json.loads(a)
            assert ra["usage"]["completion_tokens"] == 12
            st, _, b = await request(port, "POST", "/v1/chat/completions", {**body, "stream": True})
            events = [l[6:] for l in dechunk(b).split("\n\n") if l.startswith("data: ")]
            assert events[-1] == "[DONE]" and len(events) > 3
            st, _, v = await request(port, "GET", "/debug/blocks")
            assert st == 200 and "kv" in json.loads(v)
            st, _, v = await request(port, "GET", "/debug/vram")
            vram = json.loads(v)
            assert st == 200 and vram["sessions"] == [] and vram["snapshots"]["rows"] >= 1 and "durable" in vram["snapshots"]["by_class"]
            st, _, c = await request(port, "POST", "/v1/chat/completions", body)
            rc = json.loads(c)
            assert rc["choices"][0]["message"] == ra["choices"][0]["message"]
    try:
        asyncio.run(main())
    finally:
        assert svc.shutdown().code == 0


def test_graph_fleet_plans_and_meters_on_the_cpu_face():
    """The fleet lists every step shape the profile can reach and captures them at boot; on the CPU face a capture is a
    replay object and costs no device memory, and a face that cannot capture leaves its entries eager with the reason."""
    from owl_engine_b200.engine.graph_fleet import GraphFleet

    e = Engine(cfg(), device="cpu")
    fleet = GraphFleet(e, max_batch=4, spec_depths=(3,), spec_rows=2)
    names = [en.name for en in fleet.entries]
    assert names[:4] == ["graph.decode.b1.ctx2048", "graph.decode.b2.ctx2048", "graph.decode.b3.ctx2048", "graph.decode.b4.ctx2048"]
    assert "graph.verify.b1.t4.ctx2048" in names and "graph.batch_spec.b2.t4.ctx2048" in names and "graph.fold.b1.t4" in names
    rep = fleet.assemble()
    assert rep["states"] == {"captured": 8}                      # decode x 4, verify, batched verify, fold, batched fold
    assert {(4, 1), (1, 4), (2, 4), ("fold", 4), ("foldb", 2, 4)} <= set(e.runner.graphs) and rep["bytes"] == 0
    off = Engine(cfg(), device="cpu", limits=MockLimits(graph_capture=False))
    rep = GraphFleet(off, max_batch=2).assemble()
    assert rep["states"] == {"eager": 2} and "CaptureUnsupported" in rep["entries"][0]["error"]


def test_nameless_turns_find_their_session_by_content():
    """Session identity = content identity: a turn without a session name continues the parked conversation whose last
    prompt it repeats in full; a conversation that only shares the preamble gets a session of its own; named sessions
    stay named."""
    e = Engine(cfg(n_pages=256, max_seq=1024), device="cpu")
    re_ = RunningEngine(e, max_batch=2, park_sessions=True, max_parked=4, auto_sessions=True)
    opts = lambda **kw: TurnOpts(max_new=6, ignore_eos=True, **kw)
    preamble = toks(24, 50)                                  # longer than a page and common to every conversation
    a1 = preamble + toks(40, 51)
    out_a1 = re_.generate(a1, opts())
    assert sorted(re_.parked) == ["auto:0"] and re_.auto_matched == 0
    b1 = preamble + toks(44, 52)
    out_b1 = re_.generate(b1, opts())
    assert len(re_.parked) == 2 and re_.auto_matched == 0     # the shared preamble does not make it A's session
    a2 = a1 + out_a1 + toks(10, 53)
    out_a2 = re_.generate(a2, opts())
    assert re_.auto_matched == 1 and re_.resumed == 1 and len(re_.parked) == 2
    a3 = a2 + out_a2 + toks(7, 54)
    re_.generate(a3, opts())
    b2 = b1 + out_b1 + toks(5, 55)
    re_.generate(b2, opts())
    assert re_.auto_matched == 3 and re_.resumed == 3 and len(re_.parked) == 2
    # a client that re-renders the answer differently still lands in its session (prompt segment covered), resumes by prefix
    a4 = a3 + toks(6, 56) + toks(9, 57)
    re_.generate(a4, opts())
    assert re_.auto_matched == 4 and re_.resumed == 3
    c1 = preamble + toks(30, 60)
    out_c1 = re_.generate(c1, opts(session="named"))
    re_.generate(c1 + out_c1 + toks(4, 61), opts(session="named"))
    assert "named" in re_.parked and re_.queue_facts()["sessions"].count("named") == 1
    fresh = Engine(cfg(n_pages=256, max_seq=1024), device="cpu")
    assert fresh.generate(a2, 6) == out_a2                    # resumed turns produce what a cold engine produces


def test_http_rejections_are_actionable():
    """A request the pool can never hold answers 429 with the reason and no retry hint; one that only has to wait for a
    running turn answers 429 with ``Retry-After``."""
    import asyncio
    import json

    from owl_engine_b200.engine.service import EngineService
    from owl_engine_b200.engine.tokenizer import ByteTokenizer
    from owl_engine_b200.server.http import App, serve
    from owl_engine_b200.utils.stepgate import GATE
    from test_server_http import request

    svc = EngineService(lambda: Engine(cfg(n_pages=24, max_seq=2048), device="cpu"), max_batch=2, on_full="reject")
    client = svc.boot()
    tok = ByteTokenizer()

    async def main():
        app = App(client, tok, "test-hybrid", max_new_cap=4096)
        server = await serve(app, "127.0.0.1", 0)
        port = server.sockets[0].getsockname()[1]
        async with server:
            big = {"messages": [{"role": "user", "content": "x" * 900}], "max_tokens": 8}
            st, head, raw = await request(port, "POST", "/v1/chat/completions", big)
            err = json.loads(raw)["error"]
            assert st == 429 and err["code"] == "never_fits" and err["retry_after_ms"] == 0 and "Retry-After" not in head
            # a slow turn occupies most of the pool; a second one of the same size has to wait for it
            GATE.configure("sticky", 20)
            slow = {"messages": [{"role": "user", "content": "y" * 150}], "max_tokens": 60, "ignore_eos": True}
            first = asyncio.create_task(request(port, "POST", "/v1/chat/completions", slow))
            await asyncio.sleep(0.4)
            st, head, raw = await request(port, "POST", "/v1/chat/completions", slow)
            GATE.configure("off")
            err = json.loads(raw)["error"]
            assert st == 429 and err["code"] == "memory" and err["retry_after_ms"] >= 100 and "Retry-After: " in head
            assert (await first)[0] == 200
    try:
        asyncio.run(main())
    finally:
        GATE.configure("off")
        assert svc.shutdown().code == 0


def test_parked_sessions_give_way_to_new_turns():
    """Parked conversations hold rows and pages; a new turn that needs them is admitted, and the session idle longest is
    released (its blocks become evictable prefix blocks) instead of the newcomer being refused."""
    e = Engine(cfg(n_pages=40, n_slots=3, max_seqs=3, max_seq=512), device="cpu")
    re_ = RunningEngine(e, max_batch=2, park_sessions=True, max_parked=3, auto_sessions=True)
    opts = lambda: TurnOpts(max_new=6, ignore_eos=True)
    outs = [re_.generate(toks(150, 70 + i), opts()) for i in range(3)]       # three parked conversations: every row, 30 of 40 pages
    assert len(re_.parked) == 3 and len(e.states.free_rows) == 0
    out = re_.generate(toks(200, 80), opts())                                 # needs a row and 13 pages
    assert len(out) == 6 and len(re_.parked) <= 3 and "auto:0" not in re_.parked
    assert all(len(o) == 6 for o in outs)
    fresh = Engine(cfg(n_pages=40, n_slots=3, max_seqs=3, max_seq=512), device="cpu")
    assert fresh.generate(toks(200, 80), 6) == out


def test_a_turn_cancelled_between_prefill_chunks_leaves_an_anchor_for_the_retry():
    """Abort, then retry: the cancelled turn publishes the blocks it wrote AND saves the state of the point it reached, so
    the same prompt resumes there instead of starting over."""
    e = Engine(cfg(n_pages=128, max_seq=1024, prefill_chunk=64), device="cpu")
    re_ = RunningEngine(e, max_batch=2)
    prompt = toks(400, 90)
    tid = re_.submit(prompt, TurnOpts(max_new=4, ignore_eos=True))
    for _ in range(4):                     # begin + three chunks of 64
        re_.pump()
    assert e.seqs[re_.turns[tid].sid].n_cached == 192
    re_.cancel_turn(tid)
    re_.pump()
    assert tid not in re_.turns and not e.seqs
    sid = e.add_sequence(prompt)
    assert e.seqs[sid].reused == 192
    e.free_sequence(sid, publish=False)
    want = Engine(cfg(n_pages=128, max_seq=1024, prefill_chunk=64), device="cpu").generate(prompt, 6)
    assert re_.generate(prompt, TurnOpts(max_new=6, ignore_eos=True)) == want
    assert re_.trace[-1]["cached_tokens"] == 192


def test_recall_report_tells_exact_from_context_only_from_miss():
    e = Engine(cfg(n_snap_rows=1), device="cpu")
    p, other = toks(100, 1), toks(100, 2)
    e.generate(p, 4)
    assert e.last_recall["mode"] == "miss"
    e.generate(p, 4)
    assert e.last_recall["mode"] == "exact" and e.last_recall["used_blocks"] == 6 and e.last_recall["snapshot_tokens"] == 96
    e.generate(other, 4)                                   # takes the only snapshot row: p's blocks stay, its state is gone
    sid = e.add_sequence(p)
    assert e.last_recall["mode"] == "context_only" and e.last_recall["matched_blocks"] == 6 and e.seqs[sid].reused == 0
    e.free_sequence(sid, publish=False)
    assert e.recall_modes == {"miss": 2, "exact": 1, "context_only": 1}


def test_two_turns_of_one_session_side_by_side_do_not_orphan_a_parked_sequence():
    e = Engine(cfg(n_pages=64), device="cpu")
    re_ = RunningEngine(e, max_batch=2, park_sessions=True, max_parked=2)
    a = re_.submit(toks(40, 1), TurnOpts(max_new=3, ignore_eos=True, session="s"))
    b = re_.submit(toks(40, 1), TurnOpts(max_new=5, ignore_eos=True, session="s"))
    assert a != b
    re_.run_until_idle()
    assert list(re_.parked) == ["s"] and len(e.seqs) == 1               # one parked sequence, the other was released
    re_._release_parked("s")
    assert not e.seqs and e.kv.free_pages + e.kv.stats()["device_nodes"] == e.cfg.n_pages
