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
    e.runner.uniform_rows = True
    fleet = GraphFleet(e, max_batch=3, spec_depths=(3,), spec_rows=2, ctx_buckets=(512, 1024))
    rep = fleet.assemble()
    assert rep["states"] == {"captured": len(fleet.entries)} and rep["bytes"] >= 0
    assert e.ledger.by_class().get("graphs", 0) == rep["bytes"]
    assert len(e.runner.graphs) >= 2 * 3 + 2 + 2 + 2        # decode x buckets, verify, batched verify, the two folds
    n = len(e.runner.graphs)
    out = e.generate(toks(70, 9), 10)                       # decode replays what the fleet captured: no new graph
    assert len(out) == 10 and len(e.runner.graphs) == n
