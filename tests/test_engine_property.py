"""End-to-end invariant of the host logic on the CPU face: whatever the cache, the snapshots and the tiers did before, a
prompt generates exactly what an engine with no cache generates. The stand-in model makes every token depend on the restored
state row and on a mark in every page of the context, so a wrong page, a stale snapshot or a block recalled into the wrong
place changes the output."""
import shutil
import tempfile

import torch
from hypothesis import given, settings, strategies as st

from owl_engine_b200.engine.core import Engine, EngineConfig

MARK = (7001,)


def _tokens(n, seed):
    return torch.randint(0, 500, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


# a few stems that requests share (system prompts), each ending in a message marker
STEMS = [list(MARK) + _tokens(n, 100 + i) for i, n in enumerate((40, 90, 150))]


@settings(max_examples=25, deadline=None)
@given(st.lists(st.tuples(st.integers(0, 2), st.integers(0, 5), st.integers(1, 70), st.integers(1, 24)), min_size=3, max_size=14),
       st.sampled_from([0, 1, 3]), st.booleans(), st.sampled_from(["lru", "lrfu:0.2"]))
def test_cached_generation_equals_cold_generation(requests, stride, tiers, policy):
    tmp = tempfile.mkdtemp(prefix="owl_prop_")
    try:
        kw = dict(model="test-hybrid", n_slots=3, max_seqs=3, max_seq=1024, prefill_chunk=64, msg_open_ids=MARK,
                  snap_msg_min_gap=32, snap_msg_recent=2, snap_decode_stride=stride, evict_policy=policy)
        cold = Engine(EngineConfig(n_pages=256, n_snap_rows=2, prefix_cache=False, **kw), device="cpu")
        tier_kw = dict(host_cache_mb=1, disk_cache_mb=4, disk_dir=tmp, snap_host_mb=1, snap_disk_mb=2) if tiers else {}
        warm = Engine(EngineConfig(n_pages=40, n_snap_rows=2, **tier_kw, **kw), device="cpu")     # a pool that overflows
        history = []
        for stem, variant, tail, n_new in requests:
            prompt = STEMS[stem] + list(MARK) + _tokens(tail, 1000 * stem + variant)
            if history and variant == 5:
                prev_prompt, prev_out = history[-1]
                prompt = prev_prompt + prev_out + list(MARK) + _tokens(tail, 7)          # the next turn of the last conversation
            want = cold.generate(prompt, n_new)
            got = warm.generate(prompt, n_new)
            assert got == want, (len(prompt), warm.last_recall)
            history.append((prompt, got))
        st_ = warm.kv.stats()
        assert warm.kv.free_pages + st_["device_nodes"] == warm.cfg.n_pages              # no page leaked, none counted twice
        assert not warm.seqs and len(warm.states.free_rows) == 3
        warm.close()
    finally:
        shutil.rmtree(tmp, ignore_errors=True)


@settings(max_examples=20, deadline=None)
@given(st.lists(st.one_of(
    st.tuples(st.just("submit"), st.integers(0, 2), st.integers(0, 3), st.integers(1, 60), st.integers(1, 16), st.sampled_from([None, None, "a", "b"])),
    st.tuples(st.just("pump"), st.integers(1, 12)),
    st.tuples(st.just("cancel"), st.integers(0, 7)),
    st.tuples(st.just("follow"), st.integers(1, 30), st.integers(1, 12))), min_size=4, max_size=24),
    st.booleans(), st.sampled_from(["queue", "reject"]), st.booleans())
def test_running_engine_under_random_traffic_serves_what_a_cold_engine_serves(ops, park, on_full, spec):
    """Concurrent turns, parked and nameless sessions, cancellations, a pool that overflows: every turn that completes
    carries the tokens of a cold engine, rejected turns say why, and nothing is left allocated afterwards."""
    from owl_engine_b200.engine.running import RunningEngine, TurnOpts

    kw = dict(model="test-hybrid", n_slots=3, max_seqs=3, max_seq=1024, prefill_chunk=64, msg_open_ids=MARK, snap_msg_min_gap=32,
              snap_msg_recent=2, snap_decode_stride=1, snap_spec_rollback=True)
    cold = Engine(EngineConfig(n_pages=256, n_snap_rows=2, prefix_cache=False, **kw), device="cpu")
    from owl_engine_b200.engine.spec import LookupDraft, SpecRunner

    e = Engine(EngineConfig(n_pages=48, n_snap_rows=3, spec_rows=2, **kw), device="cpu")
    runner = SpecRunner(LookupDraft(1, 6), depth=3, degrade_after=3, probe_every=4) if spec else None      # speculative rounds too
    re_ = RunningEngine(e, max_batch=2, on_full=on_full, park_sessions=park, max_parked=2, auto_sessions=park, prefill_every=2,
                        spec_runner=runner)
    live, done, last = {}, [], None

    def drain():
        for tid, (t, prompt, n_new) in list(live.items()):
            out, end = t.setdefault("out", []), None
            while not t["sink"].empty():
                ev = t["sink"].get()
                if ev[0] == "token":
                    out.append(ev[2])
                elif ev[0] in ("completed", "failed"):
                    end = ev
            if end is not None:
                del live[tid]
                done.append((prompt, n_new, out, end))

    def submit(prompt, n_new, session):
        tid = re_.submit(prompt, TurnOpts(max_new=n_new, ignore_eos=True, session=session))
        live[tid] = ({"sink": re_.turns[tid].sink}, prompt, n_new)

    for op in ops:
        if op[0] == "submit":
            _, stem, variant, tail, n_new, session = op
            submit(STEMS[stem] + list(MARK) + _tokens(tail, 1000 * stem + variant), n_new, session)
        elif op[0] == "follow" and done:
            prompt, _, out, end = done[-1]
            if end[0] == "completed":
                submit(prompt + out + list(MARK) + _tokens(op[1], 5), op[2], None)
        elif op[0] == "pump":
            for _ in range(op[1]):
                re_.pump()
        elif op[0] == "cancel" and live:
            re_.cancel_turn(sorted(live)[op[1] % len(live)])
        drain()
    re_.run_until_idle(max_steps=5000)
    drain()
    assert not live and re_.idle()
    for prompt, n_new, out, end in done:
        if end[0] == "completed" and end[2] in ("length", "stop"):
            assert out == cold.generate(prompt, n_new), (len(prompt), n_new, end)
        elif end[0] == "completed":
            assert end[2] == "cancelled" and out == cold.generate(prompt, n_new)[:len(out)]      # what was emitted was right
        else:
            assert "rejected (" in end[2] and "retry_after_ms=" in end[2]
    for name in list(re_.parked):
        re_._release_parked(name)
    st_ = e.kv.stats()
    assert not e.seqs and e.kv.free_pages + st_["device_nodes"] == e.cfg.n_pages and len(e.states.free_rows) == 3
    assert re_.reservations.outstanding == 0


@settings(max_examples=12, deadline=None)
@given(st.lists(st.one_of(
    st.tuples(st.just("submit"), st.integers(0, 2), st.integers(0, 3), st.integers(1, 60), st.integers(1, 12), st.sampled_from([None, "a"])),
    st.tuples(st.just("pump"), st.integers(1, 10)),
    st.tuples(st.just("cancel"), st.integers(0, 7))), min_size=4, max_size=18), st.booleans(), st.booleans())
def test_follower_rank_ends_in_the_leaders_state(ops, park, spec):
    """Tensor-parallel serving keeps its ranks in lockstep by mirroring the leader's engine calls over the step ring and
    relying on the engine's host logic being a function of its call sequence. Random traffic through a leader (scheduler,
    parked sessions, cancellations, an overflowing pool with a host tier) and a follower that only replays the ring: both
    engines must end with the same pages, tree, snapshots and token streams."""
    import os
    import threading

    from owl_engine_b200.engine import tp_serve as T
    from owl_engine_b200.engine.running import RunningEngine, TurnOpts
    from owl_engine_b200.parallel.ring import StepRing

    from owl_engine_b200.engine.spec import LookupDraft, SpecRunner

    kw = dict(model="test-hybrid", n_pages=40, n_slots=3, n_snap_rows=2, spec_rows=2, max_seqs=3, max_seq=1024, prefill_chunk=64,
              msg_open_ids=MARK, snap_msg_min_gap=32, snap_msg_recent=2, snap_decode_stride=1, snap_spec_rollback=True, host_cache_mb=1,
              snap_host_mb=1)
    lead, foll = Engine(EngineConfig(**kw), device="cpu"), Engine(EngineConfig(**kw), device="cpu")
    name = f"/owl_prop_tp_{os.getpid()}_{abs(hash(str(ops))) % 10 ** 8}"
    ring = StepRing.create(name, 1, capacity=8 << 20)
    rd = StepRing.open(name, 0, 20.0)
    applied = {}
    make_spec = lambda: SpecRunner(LookupDraft(1, 6), depth=3, degrade_after=3, probe_every=4) if spec else None
    foll_spec = make_spec()
    th = threading.Thread(target=lambda: applied.setdefault("n", T.follower_loop(foll, rd, foll_spec, idle_timeout_s=20.0)))
    th.start()
    me = T.MirroredEngine(lead, ring)
    lead_spec = T.MirroredSpec(make_spec(), ring) if spec else None      # speculative rounds are mirrored as whole calls
    re_ = RunningEngine(me, max_batch=2, on_full="queue", park_sessions=park, max_parked=2, auto_sessions=park, prefill_every=2,
                        spec_runner=lead_spec)
    live = []
    try:
        for op in ops:
            if op[0] == "submit":
                _, stem, variant, tail, n_new, session = op
                live.append(re_.submit(STEMS[stem] + list(MARK) + _tokens(tail, 1000 * stem + variant),
                                       TurnOpts(max_new=n_new, ignore_eos=True, session=session)))
            elif op[0] == "pump":
                for _ in range(op[1]):
                    re_.pump()
            elif op[0] == "cancel" and live:
                re_.cancel_turn(live[op[1] % len(live)])
        re_.run_until_idle(max_steps=5000)
        for nm in list(re_.parked):
            re_._release_parked(nm)
    finally:
        me.shutdown()
        th.join(30)
        rd.free()
        ring.free()
    assert "n" in applied and not th.is_alive()
    a, b = lead.kv.stats(), foll.kv.stats()
    assert a == b and lead.kv.free_pages == foll.kv.free_pages
    assert sorted(lead.kv.list()) == sorted(foll.kv.list())
    snaps = lambda e: {h: (s.row, s.n_tokens, s.klass) for h, s in e.states.snaps.items()}
    assert snaps(lead) == snaps(foll)
    assert sorted(lead.states.lower) == sorted(foll.states.lower) and lead.rel.facts()["demoted"] == foll.rel.facts()["demoted"]
    assert lead.runner.launches == foll.runner.launches and not foll.seqs and not lead.seqs
    if spec:
        assert vars(lead_spec.stats) == vars(foll_spec.stats)                 # the same rounds, drafts, folds on both ranks
    assert torch.equal(lead.pool.conv_state, foll.pool.conv_state) and torch.equal(lead.pool.k_pool, foll.pool.k_pool)
