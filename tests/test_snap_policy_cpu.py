"""Recurrent-state snapshot policy: where snapshots are taken, their eviction classes, the per-session cap, the host / disk
tiers for snapshots whose row was recycled, and the LRFU victim order of the prefix tree. Engine cases run on the CPU face,
whose stand-in model makes a continuation depend on the restored state row and on every page of the context."""

import pytest
import torch

from owl_engine_b200.engine.core import Engine, EngineConfig
from owl_engine_b200.store import snap_policy as P
from owl_engine_b200.store.kv import KvStore
from owl_engine_b200.store.state import StateStore

MARK = (7001, 7002)          # the message-open marker of these tests (two tokens)


# -- pure functions ------------------------------------------------------------------------------------------------------
def test_message_points_page_align_dedupe_and_first_is_kept():
    # golden vectors of the reference's unit tests (crates/engine/src/serve/msg_boundary.rs:129-190), page = 4
    prompt = [9, 9, 1, 2, 10, 11, 1, 2, 20, 21, 1, 2, 30, 31, 1, 2, 40]
    assert P.message_points(prompt, [1, 2], 4, 0, 0) == [4, 8, 12]
    assert P.message_points(prompt, [1, 2], 4, 4, 0) == [4, 8, 12]
    assert P.message_points(prompt, [1, 2], 4, 5, 0) == [4, 12]
    assert P.message_points(prompt, [1, 2], 4, 9, 0) == [4]
    assert P.message_points([9, 9, 9, 9, 1, 0, 9, 9, 9, 9, 1, 0], [1], 4, 0, 0) == [4, 8]
    assert P.message_points(prompt, [], 4, 0, 0) == [] and P.message_points(prompt, [1, 2], 0, 0, 0) == []


def test_message_points_dense_tail_ignores_the_gap():
    prompt = [9, 9, 1, 2, 10, 11, 1, 2, 20, 21, 1, 2, 30, 31, 1, 2, 40, 41, 1, 2, 50]
    assert P.message_points(prompt, [1, 2], 4, 100, 0) == [4]
    assert P.message_points(prompt, [1, 2], 4, 100, 1) == [4, 16]
    assert P.message_points(prompt, [1, 2], 4, 100, 2) == [4, 12, 16]
    assert P.message_points(prompt, [1, 2], 4, 100, 3) == [4, 8, 12, 16]
    assert P.message_points(prompt, [1, 2], 4, 100, 9) == [4, 8, 12, 16]


def test_classes_dense_tail_binary_ladder_and_extras():
    pts = [64, 128, 256, 512, 640, 1024, 1536, 1920]
    cls = P.classify(pts, 2048, 2)
    assert cls[-2:] == [("dense", 0), ("dense", 0)]
    assert cls[5] == ("binary", 1)                      # nearest point at or below 2048 / 2
    assert cls[3] == ("binary", 2) and cls[2] == ("binary", 3) and cls[1] == ("binary", 4) and cls[0] == ("binary", 5)
    assert cls[4] == ("extra", 0)
    # eviction order: extras, then the ladder from its oldest rung, then the dense tail
    order = sorted(range(len(pts)), key=lambda i: P.order_key(*cls[i], 0.0))
    assert order[0] == 4 and order[1] == 0 and order[-2:] == [6, 7]


def test_decode_boundary_takes_the_largest_boundary_on_the_stride():
    assert P.decode_boundary(30, 33, 16, 1) == 32
    assert P.decode_boundary(32, 35, 16, 1) is None           # nothing crossed
    assert P.decode_boundary(30, 33, 16, 4) is None           # page 2 is not on a stride of 4
    assert P.decode_boundary(60, 66, 16, 4) == 64
    assert P.decode_boundary(30, 33, 16, 0) is None and P.decode_boundary(30, 33, 0, 1) is None


def test_session_cap_replaces_the_lowest_rank_and_bounds_extras():
    ss = StateStore(2, 8, cap=P.SessionCap(cap=4, reserve=2))
    assert ss.snapshot(1, 16, "extra", session="a") is not None
    assert ss.snapshot(2, 32, "extra", session="a") is not None
    r = ss.snapshot(3, 48, "extra", session="a")               # extras may hold cap - reserve = 2: the older extra leaves
    assert r is not None and 1 not in ss.snaps and {2, 3} <= set(ss.snaps)
    ss.snapshot(4, 64, "dense", session="a")
    ss.snapshot(5, 80, "durable", session="a")                  # 4 held = cap
    ss.snapshot(6, 96, "dense", session="a")                    # replaces an extra
    assert len(ss.of_session("a")) == 4 and sum(s.klass == "extra" for s in ss.of_session("a")) == 1
    ss.snapshot(7, 112, "durable", session="a")
    ss.snapshot(8, 128, "durable", session="a")
    assert ss.snapshot(9, 144, "extra", session="a") is None or len(ss.of_session("a")) == 4
    held = {s.klass for s in ss.of_session("a")}
    assert "extra" not in held or len(ss.of_session("a")) == 4
    # a newcomer that ranks below everything held is refused; another session is not affected
    ss2 = StateStore(2, 8, cap=P.SessionCap(cap=2, reserve=0))
    ss2.snapshot(1, 16, "durable", session="s")
    ss2.snapshot(2, 32, "dense", session="s")
    assert ss2.snapshot(3, 48, "binary", 3, session="s") is None and ss2.skipped == 1
    assert ss2.snapshot(4, 64, "binary", 3, session="t") is not None


def test_eviction_follows_the_class_order():
    ss = StateStore(1, 3)
    ss.snapshot(1, 16, "dense")
    ss.snapshot(2, 32, "extra")
    ss.snapshot(3, 48, "binary", 4)
    ss.snapshot(4, 64, "durable")                                # rows full: the extra goes
    assert 2 not in ss.snaps
    ss.snapshot(5, 80, "binary", 1)                              # then the oldest rung of the ladder
    assert 3 not in ss.snaps and {1, 4, 5} == set(ss.snaps)


def test_lrfu_keeps_the_block_that_is_hit_often():
    def run(policy):
        kv = KvStore(8, 16)
        kv.set_policy(policy)
        chains = [kv.chain(list(range(i * 100, i * 100 + 16))) for i in range(3)]
        for c in chains:
            pages = kv.alloc(1)
            kv.publish(c, pages)
            kv.unref(pages)
        for _ in range(6):                                   # block 0 is popular ...
            m, pg, _ = kv.match(chains[0])
            kv.unref(pg)
        for c in chains[1:]:                                 # ... but the other two were used last
            m, pg, _ = kv.match(c)
            kv.unref(pg)
        _, victims = kv.evict(need_free=kv.free_pages + 1)
        return [int(v) for v in victims], [int(c[0]) for c in chains]
    v, c = run("lru")
    assert v == [c[0]]                                       # plain recency drops the popular block
    v, c = run("lrfu:0.05")
    assert v == [c[1]]                                       # LRFU drops the colder of the two recent ones
    with pytest.raises(ValueError):
        KvStore(4, 16).set_policy("mru")


# -- the engine on the CPU face ----------------------------------------------------------------------------------------------
def cfg(**kw):
    base = dict(model="test-hybrid", n_pages=256, n_slots=4, n_snap_rows=6, max_seqs=4, max_seq=2048, prefill_chunk=64,
                msg_open_ids=MARK, snap_msg_min_gap=64, snap_msg_recent=1)
    base.update(kw)
    return EngineConfig(**base)


def toks(n, seed=0):
    return torch.randint(0, 500, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def msg(n, seed):
    return list(MARK) + toks(n, seed)


def test_sessions_sharing_a_system_prompt_reuse_it_at_the_message_boundary():
    system = msg(150, 1)
    a, b = system + msg(40, 2), system + msg(55, 3)
    fresh = Engine(cfg(), device="cpu")
    want_b = fresh.generate(b, 10)
    e = Engine(cfg(), device="cpu")
    e.generate(a, 10)
    sid = e.add_sequence(b)
    reused = e.seqs[sid].reused
    e.free_sequence(sid, publish=False)
    assert reused == len(system) // 16 * 16 and reused > 0            # up to the page boundary below the second marker
    assert e.generate(b, 10) == want_b
    off = Engine(cfg(msg_open_ids=()), device="cpu")                    # without message snapshots the shared prefix is lost
    off.generate(a, 10)
    sid = off.add_sequence(b)
    assert off.seqs[sid].reused == 0


def test_prefill_plan_cuts_only_where_two_points_fall_into_one_chunk():
    e = Engine(cfg(prefill_chunk=256, snap_msg_min_gap=0, snap_msg_recent=8), device="cpu")
    prompt = msg(60, 1) + msg(60, 2) + msg(60, 3) + msg(300, 4)
    sid = e.add_sequence(prompt)
    seq = e.seqs[sid]
    pts = sorted(seq.snap_points)
    assert pts[-1] == (len(prompt) - 1) // 16 * 16 and len(pts) == 4
    plan = e.prefill_plan(sid)
    assert plan[0][0] == 0 and plan[-1][1] == len(prompt) and all(a[1] == b[0] for a, b in zip(plan, plan[1:]))
    for lo, hi in plan:
        assert sum(lo < p < hi for p in pts) <= 1                      # one inside (saved by the runner), one at the end
    e.prefill(sid)
    assert {s.n_tokens for s in e.states.snaps.values()} == set(pts)
    e.free_sequence(sid)


def test_generation_snapshots_let_the_next_turn_resume_behind_the_answer():
    prompt = msg(100, 5)
    e = Engine(cfg(snap_decode_stride=1), device="cpu")
    answer = e.generate(prompt, 40)
    follow = prompt + answer + msg(30, 6)
    sid = e.add_sequence(follow)
    reused = e.seqs[sid].reused
    e.free_sequence(sid, publish=False)
    # tokens cached when generation stopped: prompt + 39 (the last sampled token was never fed)
    assert reused == (len(prompt) + 39) // 16 * 16
    assert sum(s.klass == "tail" for s in e.states.snaps.values()) == 1          # rolling: one per sequence
    want = Engine(cfg(), device="cpu").generate(follow, 8)
    assert e.generate(follow, 8) == want
    e2 = Engine(cfg(snap_decode_stride=4), device="cpu")
    e2.generate(prompt, 40)
    sid = e2.add_sequence(follow)
    assert e2.seqs[sid].reused == 128                                             # page 8 is the last one on a stride of 4
    none = Engine(cfg(snap_decode_stride=0), device="cpu")
    none.generate(prompt, 40)
    sid = none.add_sequence(follow)
    assert none.seqs[sid].reused == (len(prompt) - 1) // 16 * 16                  # only the prompt's own boundary


def test_recycled_snapshots_move_to_the_host_and_disk_tiers_and_come_back(tmp_path):
    e = Engine(cfg(n_snap_rows=2, msg_open_ids=(), snap_host_mb=1, snap_disk_mb=8, host_cache_mb=1, disk_cache_mb=8,
                   disk_dir=str(tmp_path)), device="cpu")
    nb = (e.pool.conv_state[:, 0].numel() + e.pool.rec_state[:, 0].numel()) * 4
    e.rel.snap_host_cap = 2 * nb                        # room for two snapshots on the host: the third goes to disk
    prompts = [toks(100, 20 + i) for i in range(6)]
    first = [e.generate(p, 6) for p in prompts]
    f = e.rel.facts()["snapshots"]
    assert f["live"] == 2 and f["host"] == 2 and f["disk"] == 2 and f["demoted"] == 4 and f["spilled"] == 2
    for p, w in zip(prompts, first):                    # every prompt again: its state comes back from wherever it went
        sid = e.add_sequence(p)
        assert e.seqs[sid].reused == 96
        e.free_sequence(sid, publish=False)
        assert e.generate(p, 6) == w
    assert e.rel.facts()["snapshots"]["recalled"] >= 4
    # without lower tiers the same traffic loses the older prefixes
    bare = Engine(cfg(n_snap_rows=2, msg_open_ids=()), device="cpu")
    for p in prompts:
        bare.generate(p, 6)
    sid = bare.add_sequence(prompts[0])
    assert bare.seqs[sid].reused == 0


def test_snapshot_files_written_under_their_own_budget_survive_a_restart(tmp_path):
    kw = dict(n_snap_rows=2, msg_open_ids=(), snap_host_mb=1, snap_disk_mb=8, host_cache_mb=1, disk_cache_mb=8, disk_dir=str(tmp_path))
    e = Engine(cfg(**kw), device="cpu")
    prompts = [toks(100, 40 + i) for i in range(4)]
    first = [e.generate(p, 5) for p in prompts]
    e.close()                                           # checkpoint: blocks, live and host-tier snapshots, index
    e2 = Engine(cfg(**kw), device="cpu")
    assert e2.adopted["states"] == 4
    for p, w in zip(prompts, first):
        sid = e2.add_sequence(p)
        assert e2.seqs[sid].reused == 96
        e2.free_sequence(sid, publish=False)
        assert e2.generate(p, 5) == w
    e2.close()


def test_prefix_cache_off_and_no_reclaim():
    e = Engine(cfg(prefix_cache=False), device="cpu")
    p = msg(100, 9)
    a = e.generate(p, 6)
    assert e.generate(p, 6) == a and e.prefix_hits == 0 and e.kv.stats()["nodes"] == 0 and not e.states.snaps
    # no_reclaim: published blocks stay; a request that needs their pages fails instead of evicting them
    e = Engine(cfg(n_pages=16, no_reclaim=True, msg_open_ids=()), device="cpu")
    e.generate(toks(150, 1), 4)
    evictions = e.kv.stats()["evictions"]
    with pytest.raises(RuntimeError):
        e.generate(toks(150, 2), 4)
    assert e.kv.stats()["evictions"] == evictions
    sid = e.add_sequence(toks(150, 1))
    assert e.seqs[sid].reused == 144                     # the first prompt's blocks are all still there


def test_generation_snapshots_start_a_chain_for_a_prompt_shorter_than_a_page():
    e = Engine(cfg(snap_decode_stride=1, msg_open_ids=()), device="cpu")
    prompt = toks(9, 77)
    answer = e.generate(prompt, 50)
    follow = prompt + answer + toks(12, 78)
    sid = e.add_sequence(follow)
    assert e.seqs[sid].reused == (9 + 49) // 16 * 16
    e.free_sequence(sid, publish=False)
    assert e.generate(follow, 6) == Engine(cfg(msg_open_ids=()), device="cpu").generate(follow, 6)


def test_running_engine_tags_snapshots_with_the_session_and_respects_its_cap():
    from owl_engine_b200.engine.running import RunningEngine, TurnOpts

    def run(cap):
        e = Engine(cfg(snap_decode_stride=1, snap_session_cap=cap, snap_structural_reserve=1, snap_msg_min_gap=0, snap_msg_recent=8,
                       n_snap_rows=8), device="cpu")
        re_ = RunningEngine(e, max_batch=2)
        history, outs = msg(60, 1), []
        for turn in range(3):
            out = re_.generate(history, TurnOpts(max_new=20, ignore_eos=True, session="s"))
            outs.append(out)
            history = history + out + msg(40, 10 + turn)
        other = re_.generate(msg(50, 99), TurnOpts(max_new=8, ignore_eos=True, session="t"))
        return e, outs, other
    free, outs_free, _ = run(0)
    capped, outs_cap, _ = run(3)
    assert outs_cap == outs_free                                      # a cap changes what is kept, never what is computed
    assert len(free.states.of_session("s")) > 3
    held = capped.states.of_session("s")
    assert 0 < len(held) <= 3 and capped.states.of_session("t")
    assert sum(s.klass == "extra" for s in held) <= 2                  # cap - reserve
    assert any(s.klass in ("durable", "tail", "dense") for s in held)  # what the next turn resumes from survived
