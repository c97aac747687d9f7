"""The scheduler as a pure function of the turn ledger: admission verdicts, the prefill / decode interleave, batched
speculative steps."""
from owl_engine_b200.engine.scheduler import DECODE, PREFILL, QUEUED, PhaseSched, Scheduler, TurnView


def views(states):
    return [TurnView(i, st, 100, fed=0, need_pages=8, spec=sp, arrival=i) for i, (st, sp) in enumerate(states)]


def test_phase_policy_interleaves_one_chunk_per_n_decode_beats():
    for every in (8, 1, 3):
        ph = PhaseSched(every)
        seq = [ph.pick([1], [2]) for _ in range(4 * (every + 1))]
        assert seq.count("prefill") == 4 and seq.count("decode") == 4 * every
        assert seq[:every + 1] == ["decode"] * every + ["prefill"]
    ph = PhaseSched(8)
    assert ph.pick([1], []) == "prefill"                      # nothing decodes: the prompt runs alone, no slicing
    assert ph.pick([], [1]) == "decode" and ph.pick([], []) == "idle"


def test_admission_hold_reject_and_fifo_order():
    s = Scheduler(max_batch=4, prefill_chunk=64, on_full="queue")
    step, rej = s.schedule(views([(QUEUED, False), (QUEUED, False)]), free_pages=4, evictable=0, outstanding=0, pool_pages=64,
                           free_rows=2)
    assert step.kind == "idle" and not rej                    # held: 8 pages needed, 4 free; the second keeps its place behind it
    step, rej = s.schedule(views([(QUEUED, False)]), free_pages=4, evictable=8, outstanding=0, pool_pages=64, free_rows=2)
    assert step.kind == "begin"
    s2 = Scheduler(max_batch=4, prefill_chunk=64, on_full="reject")
    step, rej = s2.schedule(views([(QUEUED, False)]), free_pages=4, evictable=0, outstanding=0, pool_pages=64, free_rows=2)
    assert rej == [0]
    step, rej = s2.schedule(views([(QUEUED, False)]), free_pages=64, evictable=0, outstanding=0, pool_pages=4, free_rows=2)
    assert rej == [0]                                         # can never fit


def test_speculative_step_covers_all_decoding_turns_up_to_the_scratch_rows():
    s = Scheduler(max_batch=8, prefill_chunk=64, spec_batch=4)
    step, _ = s.schedule(views([(DECODE, True)] * 3), 64, 0, 0, 64, 4)
    assert step.kind == "spec" and step.turns == [0, 1, 2]
    step, _ = s.schedule(views([(DECODE, True)] * 5), 64, 0, 0, 64, 4)
    assert step.kind == "decode" and len(step.turns) == 5      # more turns than scratch rows: a plain batched step
    step, _ = s.schedule(views([(DECODE, True), (DECODE, False)]), 64, 0, 0, 64, 4)
    assert step.kind == "decode"                              # a sampling turn in the batch: plain step for everybody
    step, _ = s.schedule(views([(PREFILL, False)]), 64, 0, 0, 64, 4)
    assert step.kind == "prefill" and step.chunk == (0, 64)


def test_rejections_say_why_and_when_to_retry():
    s = Scheduler(max_batch=4, prefill_chunk=64, on_full="reject")
    s.itl_ms = 10.0
    run = TurnView(9, DECODE, 100, fed=100, need_pages=8, remaining=40)
    q = TurnView(0, QUEUED, 100, need_pages=8)
    _, rej = s.schedule([run, q], free_pages=2, evictable=0, outstanding=0, pool_pages=64, free_rows=2)
    adm = s.take_rejection(rej[0])
    assert rej == [0] and adm.reason == "memory" and adm.retry_after_ms == 400          # 40 tokens to go at 10 ms a beat
    _, rej = s.schedule([run, q], free_pages=64, evictable=0, outstanding=0, pool_pages=64, free_rows=0)
    assert s.take_rejection(rej[0]).reason == "slots"
    _, rej = s.schedule([q], free_pages=4, evictable=0, outstanding=0, pool_pages=4, free_rows=2)
    adm = s.take_rejection(rej[0])
    assert adm.reason == "never_fits" and adm.retry_after_ms == 0                        # retrying cannot help


def test_queue_with_a_time_limit_holds_then_rejects():
    now = [0.0]
    s = Scheduler(max_batch=4, prefill_chunk=64, on_full="queue:500", clock=lambda: now[0])
    q = [TurnView(0, QUEUED, 100, need_pages=8)]
    args = dict(free_pages=2, evictable=0, outstanding=0, pool_pages=64, free_rows=2)
    step, rej = s.schedule(q, **args)
    assert step.kind == "idle" and not rej and 0 in s.held_since
    now[0] = 0.4
    assert s.schedule(q, **args)[1] == []
    now[0] = 0.6
    step, rej = s.schedule(q, **args)
    assert rej == [0] and s.take_rejection(0).reason == "queue_timeout" and 0 not in s.held_since
    # room appears in time: admitted, the hold is forgotten
    s.schedule(q, **args)
    now[0] = 0.7
    step, _ = s.schedule(q, free_pages=20, evictable=0, outstanding=0, pool_pages=64, free_rows=2)
    assert step.kind == "begin" and 0 not in s.held_since


def test_prefill_goes_to_the_turn_owed_most_and_decode_rotates_past_the_batch_width():
    s = Scheduler(max_batch=2, prefill_chunk=64)
    pf = [TurnView(0, PREFILL, 500, fed=128), TurnView(1, PREFILL, 500, fed=0), TurnView(2, PREFILL, 500, fed=64)]
    step, _ = s.schedule(pf, 64, 0, 0, 64, 4)
    assert step.kind == "prefill" and step.turns == [1] and step.chunk == (0, 64)
    dec = [TurnView(i, DECODE, 100, fed=100, remaining=10) for i in range(5)]
    seen = []
    for _ in range(5):
        step, _ = s.schedule(dec, 64, 0, 0, 64, 4)
        assert step.kind == "decode" and len(step.turns) == 2
        seen += step.turns
    assert sorted(seen) == [0, 0, 1, 1, 2, 2, 3, 3, 4, 4]          # ten rows over five beats: every turn ran twice
