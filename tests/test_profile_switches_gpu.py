"""What the profile's switches select on the GPU: eager steps against captured graphs, launch synchronisation, the YaRN
rope against the fp32 reference model, the pinned upload stager, the query window of KV selection."""
from dataclasses import replace

import pytest
import torch

from owl_engine_b200.engine.core import Engine, EngineConfig
from owl_engine_b200.models import hybrid as H
from owl_engine_b200.models.reference import RefModel, init_weights
from owl_engine_b200.models.spec import test_hybrid as make_spec
from owl_engine_b200.ops import kernels as K

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(autouse=True)
def uniform_tail(monkeypatch):
    """A resumed prefill cuts its chunks elsewhere than a cold one; token-for-token comparisons need every chunk length on
    the same GEMM arithmetic (few-row chunks would otherwise take the integer-activation weight-streaming kernel)."""
    from owl_engine_b200.ops import linear

    monkeypatch.setattr(linear, "SKINNY_UPTO", 0)


def cfg(**kw):
    base = dict(model="test-hybrid", snap_cut=True, n_pages=128, n_slots=4, n_snap_rows=4, max_seqs=4, max_seq=1024, prefill_chunk=64)
    base.update(kw)
    return EngineConfig(**base)


def toks(n, seed=0, vocab=500):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def test_eager_steps_emit_the_tokens_of_the_captured_graphs():
    p = toks(90, 1)
    want = Engine(cfg()).generate(p, 24)
    e = Engine(cfg(cuda_graph=False))
    assert e.generate(p, 24) == want
    assert all(isinstance(g, H._EagerStep) for g in e.runner.graphs.values()) and e.runner.graphs


def test_launch_sync_runs_every_launch_to_completion():
    p = toks(70, 2)
    want = Engine(cfg()).generate(p, 8)
    K.LAUNCH_SYNC = True
    try:
        assert Engine(cfg(cuda_graph=False)).generate(p, 8) == want
    finally:
        K.LAUNCH_SYNC = False


def test_message_and_generation_snapshots_on_the_device():
    mark = (497, 498)
    system = list(mark) + toks(150, 3, 400)
    a, b = system + list(mark) + toks(40, 4, 400), system + list(mark) + toks(55, 5, 400)
    kw = dict(msg_open_ids=mark, snap_msg_min_gap=32, snap_msg_recent=2, snap_decode_stride=1)
    want_b = Engine(cfg()).generate(b, 12)
    e = Engine(cfg(**kw))
    ans = e.generate(a, 40)
    sid = e.add_sequence(b)
    reused = e.seqs[sid].reused
    e.free_sequence(sid, publish=False)
    assert reused == len(system) // 16 * 16
    assert e.generate(b, 12) == want_b                      # resumed from the state saved at the message boundary
    follow = a + ans + list(mark) + toks(20, 6, 400)
    sid = e.add_sequence(follow)
    assert e.seqs[sid].reused == (len(a) + 39) // 16 * 16   # behind the answer: the rolling generation snapshot
    e.free_sequence(sid, publish=False)
    assert e.generate(follow, 8) == Engine(cfg()).generate(follow, 8)


def test_recycled_snapshots_return_from_the_host_tier():
    e = Engine(cfg(n_snap_rows=2, snap_host_mb=64))
    prompts = [toks(100, 20 + i) for i in range(5)]
    first = [e.generate(p, 6) for p in prompts]
    f = e.rel.facts()["snapshots"]
    assert f["live"] == 2 and f["host"] == 3
    for p, w in zip(prompts, first):
        sid = e.add_sequence(p)
        assert e.seqs[sid].reused == 96
        e.free_sequence(sid, publish=False)
        assert e.generate(p, 6) == w


def test_yarn_rope_matches_the_reference_model():
    spec = replace(make_spec(n_layers=4), rope_yarn=(4.0, 64, 32.0, 1.0, 1.0))
    dense = init_weights(spec, seed=3, std=0.05)
    hw, equiv = H.weights_from_dense(spec, dense, DEV, group=128)
    pool = H.StatePool(spec, DEV, n_pages=32, n_slots=4)
    run = H.HybridRunner(spec, hw, pool, max_seqs=4, max_blocks=16, prefill_gemm="tc", pdl=True)
    plain = H.HybridRunner(replace(spec, rope_yarn=None), hw, H.StatePool(spec, DEV, n_pages=32, n_slots=4), max_seqs=4, max_blocks=16,
                           prefill_gemm="tc", pdl=True)
    assert run.rope_scale > 1.1 and not torch.equal(run.inv_freq, plain.inv_freq)
    ref = RefModel(spec, equiv, kv_fp8=True)
    prompt = torch.randint(0, spec.vocab, (150,), generator=torch.Generator().manual_seed(0))
    for r in (run, plain):
        r.block_table[1, :12] = torch.arange(3, 15, dtype=torch.int32, device=DEV)
        r.prefill_chunk_forward(prompt.to(torch.int32).to(DEV), 0, 1, 2)
    torch.cuda.synchronize()
    want = ref.logits(ref.forward(prompt, ref.new_state())[-1:])
    err = lambda r: ((r.logits[:1].float().cpu() - want).norm() / want.norm()).item()
    assert err(run) < 0.05
    assert err(plain) > err(run)          # the runner without the extension is further from the extended reference


def test_stager_uploads_in_pinned_slices():
    from owl_engine_b200.formats.loader import Stager

    st = Stager(DEV, staging_mb=1)
    t = torch.randn(3, 1 << 18)                        # 3 MiB through a 1 MiB buffer
    out = st(t)
    assert out.device.type == "cuda" and torch.equal(out.cpu(), t) and st.slices == 3
    assert torch.equal(st(torch.arange(10)).cpu(), torch.arange(10))


def test_kv_selection_scores_with_the_query_window():
    kw = dict(n_pages=256, max_seq=2048, kvmem_budget=256, kvmem_sink=1, kvmem_recent=2)
    p = toks(600, 7)
    one = Engine(cfg(**kw, kvmem_query_tokens=1)).generate(p, 40)
    e = Engine(cfg(**kw, kvmem_query_tokens=8, kvmem_recall_every=2))
    many = e.generate(p, 40)
    assert len(many) == 40 and len(one) == 40
    sid = e.add_sequence(p, reuse=False)
    e.prefill(sid)
    for _ in range(20):
        e.decode_step([sid])
    seq = e.seqs[sid]
    assert seq.q_ring is not None and seq.q_ring_n == 20 and seq.q_ring.abs().sum().item() > 0
    assert len(seq.view) <= 256 // 16 + 2 and seq.view[-1] == seq.n_cached // 16


def test_graph_fleet_captures_at_boot_and_meters_into_the_ledger():
    from owl_engine_b200.engine.graph_fleet import GraphFleet

    e = Engine(cfg(spec_rows=2))
    fleet = GraphFleet(e, max_batch=3, spec_depths=(3,), spec_rows=2, ctx_buckets=(512, 1024))
    rep = fleet.assemble()
    assert rep["states"] == {"captured": len(fleet.entries)} and rep["bytes"] >= 0
    assert e.ledger.by_class().get("graphs", 0) == rep["bytes"]
    assert len(e.runner.graphs) >= 2 * 3 + 2 + 2 + 2        # decode x buckets, verify, batched verify, the two folds
    n = len(e.runner.graphs)
    out = e.generate(toks(70, 9), 10)                       # decode replays what the fleet captured: no new graph
    assert len(out) == 10 and len(e.runner.graphs) == n


def _server_proc(profile, q):
    import os

    for k in ("WORLD_SIZE", "RANK", "LOCAL_RANK"):
        os.environ.pop(k, None)
    from owl_engine_b200.server import main as M

    q.put(M.main(["-p", profile, "--log-level", "info"]))


def test_server_main_boots_a_profile_that_uses_the_switches(tmp_path):
    """The product's entry point on one GPU with a profile that turns the optional machinery on: message / generation
    snapshots, LRFU eviction, lookup drafting (so the boot captures verify and fold graphs too), checkpoint verification with a
    1 MiB upload stager, request dumps, step profile. Two conversations share a system prompt: the second is served from the
    snapshot at the message boundary."""
    import http.client
    import json
    import multiprocessing as mp
    import os
    import sys
    import time

    sys.path.insert(0, os.path.dirname(__file__))
    from test_tp_gpu import _free_port, _shutdown, _write_checkpoint

    ckpt, port = str(tmp_path / "ckpt"), _free_port()
    _write_checkpoint(ckpt)
    root = os.path.abspath(os.path.join(os.path.dirname(__file__), "..", "configs", "full.toml"))
    prof = tmp_path / "p.toml"
    prof.write_text(f'''extends = ["{root}"]
[server]
bind = "127.0.0.1:{port}"
request_dump_dir = "{tmp_path / 'dumps'}"
[model]
name = "test-hybrid"
path = "{ckpt}"
format = "safetensors"
[runtime]
max_seq = 1024
prefill_chunk = 64
max_batch = 3
default_max_new = 16
[store]
evict_policy = "lrfu:0.1"
snap_host_mb = 64
[store.gdn]
gdn_slots = 3
snap_max = 4
snap_msg_min_gap = 32
[spec]
lookup = true
depth = 3
[load]
verify = true
staging_mb = 1
[probes]
step_profile = true
prompt_dump = true
[cuda]
trace_ring = 128
[kernel]
selfcheck = false
''')
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_server_proc, args=(str(prof), q))
    p.start()

    def post(body, timeout=180.0):
        t0 = time.time()
        while True:
            try:
                c = http.client.HTTPConnection("127.0.0.1", port, timeout=120)
                c.request("POST", "/v1/chat/completions", json.dumps(body), {"Content-Type": "application/json"})
                r = c.getresponse()
                raw = r.read().decode()
                c.close()
                assert r.status == 200, raw
                return json.loads(raw)
            except (ConnectionRefusedError, ConnectionResetError):
                if time.time() - t0 > timeout or not p.is_alive():
                    raise
                time.sleep(0.5)
    try:
        system = "You are a careful assistant. " * 12
        outs = [post({"messages": [{"role": "system", "content": system}, {"role": "user", "content": u}], "max_tokens": 20,
                      "ignore_eos": True}) for u in ("first question", "another, longer second question")]
        c = http.client.HTTPConnection("127.0.0.1", port, timeout=30)
        c.request("GET", "/debug/launches/8")
        dbg = json.loads(c.getresponse().read())
        c.close()
    finally:
        try:
            _shutdown(port)
        except Exception:   # noqa: BLE001
            pass
        p.join(timeout=120)
    assert p.exitcode == 0 and q.get(timeout=10) == 0
    cached = [o["usage"].get("prompt_tokens_details", {}).get("cached_tokens", o["usage"].get("cached_tokens", 0)) for o in outs]
    assert cached[0] == 0 and cached[1] >= 256 and cached[1] % 16 == 0
    assert all(o["usage"]["completion_tokens"] == 20 for o in outs)
    fleet = dbg["fleet"]
    assert fleet and fleet["states"].get("captured", 0) >= 3 and any("verify" in e["name"] for e in fleet["entries"])
    assert len(dbg["launches"]) == 8 and len(os.listdir(tmp_path / "dumps")) == 2
    used = [g for g in dbg["graph_manifest"] if g["replays"] > 0]
    assert used and all(g["launches_per_replay"] > 0 and sum(g["entries"].values()) == g["launches_per_replay"] for g in used)


def test_coverage_probe_reads_the_pool_and_the_last_query():
    e = Engine(cfg(n_pages=256, max_seq=2048))
    sid = e.add_sequence(toks(400, 11), reuse=False)
    e.prefill(sid)
    for _ in range(3):
        e.decode_step([sid])
    k = e.pool_keys(sid)
    assert k.shape == (e.seqs[sid].n_cached, e.spec.hkv, e.spec.hd) and torch.isfinite(k).all() and k.abs().sum() > 0
    rep = e.coverage_probe(sid, ks=(1, 4, 16))
    assert rep["blocks"] == (e.seqs[sid].n_cached + 15) // 16
    for k_, c in rep["curve"].items():
        assert 0.0 <= c["index"] <= c["oracle"] + 1e-6 <= 1.0 + 1e-6 and c["chance"] == min(k_, rep["blocks"]) / rep["blocks"]


def test_packing_on_the_device_gives_the_records_of_packing_on_the_host(tmp_path):
    import os
    import sys

    sys.path.insert(0, os.path.dirname(__file__))
    from owl_engine_b200.formats import loader
    from test_tp_gpu import _write_checkpoint

    ckpt = str(tmp_path / "ckpt")
    _write_checkpoint(ckpt)
    spec = make_spec(n_layers=4, vocab=512)
    _, a = loader.load_model(ckpt, DEV, spec=spec, repack="cpu")
    _, b = loader.load_model(ckpt, DEV, spec=spec, repack="device", staging_mb=1)
    _, c = loader.load_model(ckpt, DEV, spec=spec)                      # auto = device on a GPU
    for la, lb, lc in zip(a.layers, b.layers, c.layers):
        for nm in ("gate_up", "down", "qkvz", "out_proj", "qkv", "o_proj"):
            ta = getattr(la, nm, None)
            if ta is not None:
                assert torch.equal(ta.records, getattr(lb, nm).records) and torch.equal(ta.records, getattr(lc, nm).records), nm
                assert getattr(lb, nm).records.device.type == "cuda"
    assert torch.equal(a.embed, b.embed) and torch.equal(a.lm_head.records, b.lm_head.records)
