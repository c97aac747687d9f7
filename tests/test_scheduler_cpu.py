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
