"""Engine layer on a GPU: prefix reuse equals cold computation, batching, sampling, service thread."""
import pytest
import torch

from owl_engine_b200.engine import sampler as S
from owl_engine_b200.engine.core import Engine, EngineConfig
from owl_engine_b200.engine.running import RunningEngine, TurnOpts
from owl_engine_b200.engine.service import EngineService

pytestmark = pytest.mark.gpu


# snap_cut=True: these tests compare a cold prefill with a prefix-reusing one token for token, which needs the rows after
# the last block boundary to go through the same kernels in both (a chunk of their own); the default takes the snapshot
# inside the chunk instead (test_snapshot_inside_a_chunk_equals_the_cut_chunk covers that path).
def make_engine(**kw):
    cfg = EngineConfig(model="test-hybrid", snap_cut=True, n_pages=128, n_slots=4, n_snap_rows=2, max_seqs=4, max_seq=512,
                       prefill_chunk=64, **kw)
    return Engine(cfg)


@pytest.fixture
def uniform_tail(monkeypatch):
    """Bit-equality of a warm and a cold prefill needs the same GEMM arithmetic for every chunk length: keep the
    few-row tail chunks on the GEMM kernel instead of the (integer-activation) weight-streaming kernel."""
    from owl_engine_b200.ops import linear

    monkeypatch.setattr(linear, "SKINNY_UPTO", 0)


def test_prefix_reuse_gives_same_tokens_as_cold_run(uniform_tail):
    eng = make_engine()
    g = torch.Generator().manual_seed(0)
    base = torch.randint(0, eng.spec.vocab, (100,), generator=g).tolist()
    a = eng.generate(base, 6)
    assert eng.kv.stats()["published"] >= 6
    # a longer prompt sharing the 96-token block-aligned prefix: reuse + snapshot restore
    ext = base + torch.randint(0, eng.spec.vocab, (21,), generator=g).tolist()
    sid = eng.add_sequence(ext)
    assert eng.seqs[sid].reused == 96
    eng.free_sequence(sid, publish=False)
    warm = eng.generate(ext, 6)
    cold_eng = make_engine()
    cold = cold_eng.generate(ext, 6)
    assert warm == cold
    assert eng.generate(base, 6) == a and eng.prefix_hits >= 2


def test_pressure_demotes_to_host_then_disk_and_recall_gives_same_tokens(tmp_path, uniform_tail):
    """A pool too small for the working set: published prefixes leave for the pinned-host tier, the host tier's oldest
    blocks leave for disk files, and a returning prompt is served from disk -> host -> device with unchanged output."""
    eng = Engine(EngineConfig(model="test-hybrid", snap_cut=True, n_pages=20, n_slots=4, n_snap_rows=8, max_seqs=4,
                                                  max_seq=512, prefill_chunk=64, host_cache_mb=1,
                                                  disk_cache_mb=4, disk_dir=str(tmp_path / "kv")))
    keep = 4
    eng.host.free = eng.host.free[-keep:]                      # a host tier of four blocks
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, eng.spec.vocab, (100,), generator=g).tolist() for _ in range(4)]
    first = eng.generate(prompts[0], 5)
    for p in prompts[1:]:
        eng.generate(p, 5)
    assert eng.spilled > 0 and len(eng.disk.index) > 0
    assert eng.generate(prompts[0], 5) == first
    assert eng.recalled > 0 and eng.prefix_hits >= 1
    cold = Engine(EngineConfig(model="test-hybrid", snap_cut=True, n_pages=128, n_slots=4, n_snap_rows=2, max_seqs=4, max_seq=512,
                               prefill_chunk=64))
    assert cold.generate(prompts[0], 5) == first


def test_running_engine_batches_and_events():
    re = RunningEngine(make_engine(), max_batch=4)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (20, 70, 33)]
    solo = [RunningEngine(make_engine()).generate(p, TurnOpts(max_new=5)) for p in prompts]
    import queue

    sinks = [queue.Queue() for _ in prompts]
    tids = [re.submit(p, TurnOpts(max_new=5), sink=q) for p, q in zip(prompts, sinks)]
    re.run_until_idle()
    assert not re.turns          # finished turns leave the ledger
    for tid, want, q in zip(tids, solo, sinks):
        evs = list(q.queue)
        toks = [e[2] for e in evs if e[0] == "token"]
        assert toks == want and evs[-1][0] == "completed" and evs[-1][2] == "length"
        assert evs[0][0] == "prefill"
    assert re.idle() and re.e.kv.free_pages + re.e.kv.stats()["device_nodes"] == 128


def test_sampling_is_seeded_and_cancel_publishes():
    re = RunningEngine(make_engine(), max_batch=2)
    p = list(range(40))
    o = TurnOpts(max_new=8, sampling=S.SamplingParams(mode="sampling", temp=0.9, topk=20, topp=0.9, seed=42))
    a = re.generate(p, o)
    b = re.generate(p, o)
    assert a == b and len(a) == 8
    import queue

    q = queue.Queue()
    tid = re.submit(list(range(100, 180)), TurnOpts(max_new=50), sink=q)
    for _ in range(4):
        re.pump()
    re.cancel_turn(tid)
    re.run_until_idle()
    assert list(q.queue)[-1][2] == "cancelled" and tid not in re.turns
    assert re.e.kv.stats()["nodes"] >= 4


def test_service_thread_roundtrip():
    svc = EngineService(lambda: make_engine(), max_batch=2)
    client = svc.boot(timeout=300)
    tid, sink = client.chat(list(range(30)), TurnOpts(max_new=4))
    toks = []
    while True:
        ev = sink.get(timeout=60)
        if ev[0] == "token":
            toks.append(ev[2])
        elif ev[0] in ("completed", "failed"):
            break
    assert len(toks) == 4 and client.queue_facts()["decode"] == 0
    ex = svc.shutdown()
    assert ex.kind == "normal" and ex.code == 0


def test_http_server_end_to_end():
    """Real engine thread behind the HTTP surface: non-stream and SSE give the same greedy text."""
    import asyncio
    import json

    from owl_engine_b200.engine.tokenizer import ByteTokenizer
    from owl_engine_b200.server.http import App, serve
    from test_server_http import dechunk, request

    svc = EngineService(lambda: make_engine(), max_batch=4)
    client = svc.boot()
    tok = ByteTokenizer()

    async def main():
        app = App(client, tok, "test-hybrid")
        server = await serve(app, "127.0.0.1", 0)
        port = server.sockets[0].getsockname()[1]
        async with server:
            body = {"messages": [{"role": "user", "content": "hello"}], "max_tokens": 12, "ignore_eos": True}
            st, _, a = await request(port, "POST", "/v1/chat/completions", body)
            assert st == 200
            ra = json.loads(a)
            assert ra["usage"]["completion_tokens"] == 12
            st, _, b = await request(port, "POST", "/v1/chat/completions", {**body, "stream": True})
            events = [l[6:] for l in dechunk(b).split("\n\n") if l.startswith("data: ")]
            assert events[-1] == "[DONE]"
            st, _, v = await request(port, "GET", "/debug/vram")
            assert st == 200 and json.loads(v)["total"] > 0
            st, _, v = await request(port, "GET", "/debug/blocks")
            assert st == 200 and "kv" in json.loads(v)
            # second identical prompt reuses the published prefix
            st, _, c = await request(port, "POST", "/v1/chat/completions", body)
            assert json.loads(c)["choices"][0]["message"] == ra["choices"][0]["message"]
    try:
        asyncio.run(main())
    finally:
        assert svc.shutdown().code == 0


def test_image_prompt_embeds_positions_and_content_keyed_prefix_cache():
    """Image rows come from the vision tower, positions are (t, h, w), and the prefix cache keys image
    blocks by pixel content: the same tokens with other pixels must not hit."""
    from owl_engine_b200.cli import png
    from owl_engine_b200.models import vision as V

    eng = make_engine()
    spec = V.tiny_vision(out_hidden=eng.spec.hidden)
    tower, cache = V.VisionTower(spec), V.ImageCache()
    pad = 500

    def build(rgb):
        emb, grid, fp = cache.get(tower, png.encode_png(96, 64, rgb), png.decode_png)
        n = tower.n_tokens(grid)
        g = torch.Generator().manual_seed(5)
        head = torch.randint(0, 400, (9,), generator=g).tolist()
        tail = torch.randint(0, 400, (40,), generator=g).tolist()
        return head + [pad] * n + tail, [(emb * 20, grid, fp)]

    def run(rgb):
        prompt, images = build(rgb)
        sid = eng.add_sequence(prompt, images=images, image_pad_id=pad)
        seq = eng.seqs[sid]
        reused = seq.reused
        assert seq.rope_delta == 3 - 6            # a 2 x 3 merged grid spans 3 positions for 6 tokens
        out = [eng.prefill(sid)]
        for _ in range(5):
            out += eng.decode_step([sid])
        eng.free_sequence(sid, publish=True)
        return out, reused

    a, r0 = run(png.RED)
    b, r1 = run(png.RED)
    c, r2 = run(png.BLUE)
    assert r0 == 0 and r1 >= 32 and a == b          # same pixels: cached prefix reused, same continuation
    assert r2 <= 0 + 16 * 0 and c != a              # other pixels: no reuse past the text head, other output


def test_kv_selection_view_covers_everything_or_a_bounded_set():
    """KV selection: with a budget above the context nothing changes; with a small budget decode steps attend to a
    view of sink + recent + scored blocks whose page table sits in the sequence's second block-table row."""
    from owl_engine_b200.store import select as S

    g = torch.Generator().manual_seed(5)
    base = EngineConfig(model="test-hybrid", snap_cut=True, n_pages=128, n_slots=4, n_snap_rows=2, max_seqs=4, max_seq=512, prefill_chunk=64)
    prompt = torch.randint(0, 512, (150,), generator=g).tolist()
    plain = Engine(base).generate(prompt, 20)
    from dataclasses import replace
    wide = Engine(replace(base, kvmem_budget=4096))
    assert wide.generate(prompt, 20) == plain
    eng = Engine(replace(base, kvmem_budget=96, kvmem_sink=1, kvmem_recent=2))
    sid = eng.add_sequence(prompt)
    eng.prefill(sid)
    for _ in range(20):
        eng.decode_step([sid])
    seq = eng.seqs[sid]
    cur = (seq.n_cached - 1) // 16
    assert seq.view is not None and len(seq.view) == 6 and seq.view[0] == 0 and seq.view[-2:] == [cur - 1, cur]
    assert seq.view == sorted(seq.view) and seq.meank_n == cur
    row = eng.runner.block_table[seq.row + 4, :6].tolist()
    assert row == [seq.pages[b] for b in seq.view]
    # the GPU index equals the host formula on the pool's own keys
    sp, fi = eng.spec, eng.spec.n_full - 1
    k = eng.pool.k_pool[fi][seq.pages[2]].view(torch.float8_e4m3fn).float().cpu()          # [16, hkv, hd]
    pos = torch.arange(32, 48).float()
    inv = eng.runner.inv_freq.cpu()
    ang = pos[:, None] * inv[None]
    want = S.mean_k_index(S.derope(k, ang.cos(), ang.sin())[None])[0]
    assert torch.allclose(seq.meank[2].cpu(), want, atol=2e-3, rtol=1e-3)
    q = torch.randn(1, sp.hq, sp.hd, generator=g).bfloat16()
    got = S.score_blocks_gpu(q.to(eng.device), torch.tensor([200], dtype=torch.int32, device=eng.device), seq.meank[:cur],
                             eng.runner.inv_freq, sp.rotary_dim).cpu()
    a200 = torch.tensor([200.0])[:, None] * inv[None]
    ref = S.score_blocks(S.derope(q.float(), a200.cos(), a200.sin()), seq.meank[:cur].cpu())
    assert torch.allclose(got, ref, atol=2e-3)
    p = S.softmax_scores_gpu(got.to(eng.device), 4.0).cpu()
    assert torch.allclose(p, torch.softmax(got * 4.0, 0), atol=1e-5)
    eng.free_sequence(sid, publish=False)


def test_snapshot_inside_a_chunk_equals_the_cut_chunk(uniform_tail):
    """The GDN snapshot taken inside the chunk that contains the last block boundary holds the same state as the one taken
    after a chunk cut at the boundary, and a request that reuses it continues identically."""
    g = torch.Generator().manual_seed(11)
    prompt = torch.randint(0, 512, (150,), generator=g).tolist()
    outs, snaps = [], []
    for cut in (True, False):
        eng = Engine(EngineConfig(model="test-hybrid", n_pages=128, n_slots=4, n_snap_rows=2, max_seqs=4, max_seq=512,
                                  prefill_chunk=256, snap_cut=cut))
        sid = eng.add_sequence(prompt)
        assert eng.prefill_plan(sid) == ([(0, 144), (144, 150)] if cut else [(0, 150)])
        eng.prefill(sid)
        first = eng.runner.logits[:1].float().cpu().clone()
        snap = eng.states.find(eng.seqs[sid].chain)
        assert snap is not None and snap.n_tokens == 144
        snaps.append((eng.pool.rec_state[:, snap.row].clone(), eng.pool.conv_state[:, snap.row].clone()))
        eng.free_sequence(sid)
        outs.append((first, eng.generate(prompt + [7, 8, 9], 6), eng.prefix_hits))
    assert torch.equal(snaps[0][1], snaps[1][1])
    assert (snaps[0][0] - snaps[1][0]).norm() / snaps[0][0].norm() < 1e-3          # 144 rows vs 144 rows: same chunked scan
    assert (outs[0][0] - outs[1][0]).norm() / outs[0][0].norm() < 1e-2
    assert outs[0][2] >= 1 and outs[1][2] >= 1 and len(outs[0][1]) == len(outs[1][1]) == 6


def test_leave_gap_deletion_and_extension_of_a_live_sequence():
    """An agent session on a live sequence: a page-aligned segment in the middle of the history is unlinked (pages freed, block
    table compacted, survivors keep KV and positions, the position ledger keeps the hole), decoding continues, and the next turn's
    tokens are appended from the old maximum position + 1. Before the hole everything is exact: the same steps on a sequence
    that never had the segment after it agree token for token up to the deletion point's first new token only in mechanics,
    so the checks are the ledgers and that the carried context is the one attended to."""
    from owl_engine_b200.engine import img_evict as E

    eng = make_engine()
    g = torch.Generator().manual_seed(9)
    a = torch.randint(0, 500, (27,), generator=g).tolist()
    img = torch.randint(0, 500, (40,), generator=g).tolist()
    b = torch.randint(0, 500, (13,), generator=g).tolist()
    seq0 = E.pad_rule(a + img + b, [(27, 67)], 16, 511)
    sp = seq0.spans[0]
    assert sp.start == 32 and sp.hi == 80
    free0 = eng.kv.stats()["free_pages"]
    sid = eng.add_sequence(seq0.ids)
    eng.prefill(sid)
    for _ in range(3):
        eng.decode_step([sid])
    seq = eng.seqs[sid]
    n_before, pages_before = seq.n_cached, list(seq.pages)
    ranges, suffix = E.detect_deletions(seq0, a + b + [5, 6, 7])
    assert ranges == [(32, 80)] and suffix == [5, 6, 7]
    removed = eng.drop_ranges(sid, ranges)
    assert removed == 48 and seq.n_cached == n_before - 48 and seq.rope_delta == 48 and seq.gap_from == 32
    assert seq.pages == pages_before[:2] + pages_before[5:]
    assert eng.runner.block_table[seq.row, :len(seq.pages)].tolist() == seq.pages
    assert eng.kv.stats()["free_pages"] == free0 - len(seq.pages)
    assert seq.tokens[:32] == seq0.ids[:32] and seq.tokens[32:32 + len(seq0.ids) - 80] == seq0.ids[80:]
    t1 = eng.decode_step([sid])[0]                                  # position = cache index + 48
    assert int(eng.h_inp_np[H_pos_index(eng)]) == seq.n_cached - 1 + 48
    nxt = eng.extend_sequence(sid, suffix)
    assert 0 <= nxt < eng.spec.vocab and seq.n_cached == len(seq.tokens) - 1
    out = [eng.decode_step([sid])[0] for _ in range(4)]
    assert all(0 <= t < eng.spec.vocab for t in [t1] + out)
    # only the exact part is published
    eng.free_sequence(sid)
    sid2 = eng.add_sequence(seq0.ids[:32] + [1, 2, 3])
    assert eng.seqs[sid2].reused in (0, 16, 32)
    eng.free_sequence(sid2, publish=False)


def H_pos_index(eng):
    from owl_engine_b200.models import hybrid as H

    return H.StepLayout(1, 1).pos3


def test_parked_session_resumes_with_a_dropped_screenshot():
    """Agent session over the running engine: turn 1 has a droppable segment, turn 2 arrives without it and with new text:
    the parked sequence is continued (segment unlinked in place, only the new tokens prefilled); turn 3 appends again."""
    eng = make_engine()
    re_ = RunningEngine(eng, max_batch=2, park_sessions=True, max_parked=1, evict_pad_id=511)
    g = torch.Generator().manual_seed(13)
    a = torch.randint(0, 500, (27,), generator=g).tolist()
    img = torch.randint(0, 500, (40,), generator=g).tolist()
    b = torch.randint(0, 500, (13,), generator=g).tolist()
    o1 = re_.generate(a + img + b, TurnOpts(max_new=4, ignore_eos=True, session="s", evict_spans=[(27, 67)]))
    assert len(o1) == 4 and "s" in re_.parked and len(eng.seqs) == 1
    pages1 = len(next(iter(eng.seqs.values())).pages)
    t2 = a + b + o1 + [3, 4, 5]
    o2 = re_.generate(t2, TurnOpts(max_new=4, ignore_eos=True, session="s"))
    assert re_.resumed == 1 and re_.gap_drops == 1 and len(o2) == 4
    seq = next(iter(eng.seqs.values()))
    assert seq.rope_delta == 48 and len(seq.pages) <= pages1 - 2
    assert re_.trace[-1]["cached_tokens"] > 0
    o3 = re_.generate(t2 + o2 + [9, 9], TurnOpts(max_new=3, ignore_eos=True, session="s"))
    assert re_.resumed == 2 and len(o3) == 3
    # another session parks too: the older parked sequence is released
    re_.generate(a, TurnOpts(max_new=2, ignore_eos=True, session="other"))
    assert list(re_.parked) == ["other"] and len(eng.seqs) == 1
    # a prompt that is not a continuation starts over
    re_.generate(b + a, TurnOpts(max_new=2, ignore_eos=True, session="other"))
    assert re_.resumed == 2


def test_parked_session_with_screenshots_drops_one_and_takes_a_new_one():
    """The screenshot loop of a GUI agent: turn 1 carries two same-sized droppable images; turn 2 arrives without the FIRST one and
    with a new image behind the history; turn 3 drops the second. Each turn continues the parked sequence: the dropped image's pages
    are unlinked, the kept image stays (identified by content, not by size), the new image's (t, h, w) block starts at the
    sequence's next position and is droppable itself."""
    from owl_engine_b200.cli import png
    from owl_engine_b200.models import vision as V

    eng = make_engine()
    tower, cache = V.VisionTower(V.tiny_vision(out_hidden=eng.spec.hidden)), V.ImageCache()
    pad = 500
    re_ = RunningEngine(eng, max_batch=2, park_sessions=True, max_parked=1, evict_pad_id=511)

    def img(rgb):
        emb, grid, fp = cache.get(tower, png.encode_png(96, 64, rgb), png.decode_png)
        return (emb * 20, grid, fp)

    red, blue, green = img(png.RED), img(png.BLUE), img((0, 255, 0))
    n = red[0].shape[0]
    g = torch.Generator().manual_seed(21)
    a, b, c = (torch.randint(0, 400, (k,), generator=g).tolist() for k in (11, 7, 9))
    t1 = a + [pad] * n + b + [pad] * n + c
    s1 = [(len(a), len(a) + n), (len(a) + n + len(b), len(a) + 2 * n + len(b))]
    o1 = re_.generate(t1, TurnOpts(max_new=3, ignore_eos=True, session="s", images=[red, blue], image_pad_id=pad, evict_spans=s1))
    assert len(o1) == 3 and "s" in re_.parked
    seq = next(iter(eng.seqs.values()))
    assert [fp for _, _, fp in seq.images] == [red[2], blue[2]] and all(f % 16 == 0 for f, _, _ in seq.images)
    pages1 = len(seq.pages)
    # turn 2: red is gone, a new (green) screenshot follows the history
    d = [5, 6, 7]
    t2 = a + b + [pad] * n + c + o1 + d + [pad] * n + [8]
    lo = len(a) + len(b) + n + len(c) + len(o1) + len(d)
    o2 = re_.generate(t2, TurnOpts(max_new=3, ignore_eos=True, session="s", images=[blue, green], image_pad_id=pad,
                                   evict_spans=[(len(a) + len(b), len(a) + len(b) + n), (lo, lo + n)]))
    assert re_.resumed == 1 and re_.gap_drops == 1 and len(o2) == 3
    assert [fp for _, _, fp in seq.images] == [blue[2], green[2]] and seq.images[1][0] % 16 == 0
    assert seq.pos3.shape[1] >= seq.images[1][0] + n
    p = seq.pos3[:, seq.images[1][0]:seq.images[1][0] + n]
    assert int(p[0].max()) == int(p[0].min()) and int(p[1].max() - p[1].min()) == 1 and int(p[2].max() - p[2].min()) == 2
    assert int(seq.pos3[0, seq.images[1][0] - 1]) < int(p[0].min())            # the block starts after everything before it
    assert len(seq.tokens) + seq.rope_delta > int(seq.pos3.max())               # decode positions continue past every used id
    # turn 3: blue is gone as well
    t3 = a + b + c + o1 + d + [pad] * n + [8] + o2 + [9]
    lo3 = len(a) + len(b) + len(c) + len(o1) + len(d)
    o3 = re_.generate(t3, TurnOpts(max_new=2, ignore_eos=True, session="s", images=[green], image_pad_id=pad, evict_spans=[(lo3, lo3 + n)]))
    assert re_.resumed == 2 and re_.gap_drops == 2 and len(o3) == 2
    assert [fp for _, _, fp in seq.images] == [green[2]] and len(seq.pages) <= pages1 + 2
    # same-sized image with other content in the kept slot is NOT a continuation
    t4 = [x for x in t3]
    re_.generate(t4 + o3 + [1], TurnOpts(max_new=1, ignore_eos=True, session="s", images=[red], image_pad_id=pad))
    assert re_.resumed == 2
    # droppable marks while sessions are not parked are refused
    with pytest.raises(ValueError):
        RunningEngine(eng, max_batch=2).submit(a, TurnOpts(evict_spans=[(0, 4)]))


@pytest.mark.parametrize("kv_dtype", ["int8", "bf16"])
def test_kv_selection_index_over_int8_and_16bit_pools(kv_dtype):
    """KV selection with the other pool formats: the block index is the mean of the de-rotated keys AS STORED (int8 values times
    their token scale; fp16 words), and a bounded view is selected and attended to."""
    from dataclasses import replace

    from owl_engine_b200.store import select as S

    g = torch.Generator().manual_seed(5)
    base = EngineConfig(model="test-hybrid", snap_cut=True, n_pages=128, n_slots=4, n_snap_rows=2, max_seqs=4, max_seq=512,
                        prefill_chunk=64, kv_dtype=kv_dtype)
    prompt = torch.randint(0, 512, (150,), generator=g).tolist()
    eng = Engine(replace(base, kvmem_budget=96, kvmem_sink=1, kvmem_recent=2))
    sid = eng.add_sequence(prompt)
    eng.prefill(sid)
    out = [eng.decode_step([sid])[0] for _ in range(8)]
    seq = eng.seqs[sid]
    assert seq.view is not None and len(seq.view) == 6 and all(0 <= t < eng.spec.vocab for t in out)
    fi = eng.spec.n_full - 1
    page = seq.pages[2]
    if kv_dtype == "int8":
        k = eng.pool.k_pool[fi][page].view(torch.int8).float().cpu() * eng.pool.k_scale[fi][page].cpu()[..., None]
    else:
        k = eng.pool.k_pool[fi][page].float().cpu()
    inv = eng.runner.inv_freq.cpu()
    ang = torch.arange(32, 48).float()[:, None] * inv[None]
    want = S.mean_k_index(S.derope(k, ang.cos(), ang.sin())[None])[0]
    assert torch.allclose(seq.meank[2].cpu(), want, atol=2e-3, rtol=1e-3)
    eng.free_sequence(sid, publish=False)
