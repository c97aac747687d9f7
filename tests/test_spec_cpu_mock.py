"""Speculative decoding on the CPU face: the round machine (propose, verify as one multi-row step, accept, restore + fold)
over the stand-in model, whose recurrent state and per-page marks make a wrong rollback visible in the next token."""
import torch

from owl_engine_b200.engine.core import Engine, EngineConfig
from owl_engine_b200.engine.running import RunningEngine, TurnOpts
from owl_engine_b200.engine.spec import LookupDraft, OracleDraft, SpecRunner, generate_spec


def cfg(**kw):
    base = dict(model="test-hybrid", n_pages=128, n_slots=4, n_snap_rows=3, spec_rows=4, max_seqs=4, max_seq=1024, prefill_chunk=64)
    base.update(kw)
    return EngineConfig(**base)


def toks(n, seed=0):
    return torch.randint(0, 500, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def test_forced_acceptance_lengths_reproduce_plain_decoding():
    prompt = toks(70, 1)
    want = Engine(cfg(), device="cpu").generate(prompt, 40)
    for accept in (0, 1, 3, 7):
        e = Engine(cfg(), device="cpu")
        spec = SpecRunner(OracleDraft(want, len(prompt), accept, 512), depth=7, degrade_below=-1.0)
        got = generate_spec(e, prompt, 40, spec)
        assert got == want, accept
        st = spec.stats
        assert st.rounds > 0 and (st.accepted / st.rounds >= min(accept, 6.0) - 1.01 or accept == 0)
        assert (st.folds > 0) == (accept < 7)                    # a rejected row means: restore the state, replay the accepted rows
        assert e.kv.free_pages + e.kv.stats()["device_nodes"] == e.cfg.n_pages


def test_batched_rounds_through_the_running_engine():
    """Three turns decode together: the scheduler hands all of them to one speculative step, the target verifies them as
    one (3, T) step, sequences with rejected rows are folded together; every stream equals plain decoding."""
    prompts = [toks(40 + 7 * i, 10 + i) for i in range(3)]
    plain = Engine(cfg(), device="cpu")
    want = [plain.generate(p, 60) for p in prompts]
    e = Engine(cfg(), device="cpu")
    spec = SpecRunner(LookupDraft(2, 8), depth=3, degrade_below=-1.0)
    # sequence ids are handed out in admission order: each turn drafts from its own recorded continuation, 2 right then 1 wrong
    spec.per_sid = {i: OracleDraft(want[i], len(prompts[i]), 2, 512) for i in range(3)}
    re_ = RunningEngine(e, max_batch=4, spec_runner=spec, prefill_every=1)      # prompts join the decoding turns at once
    tids = [re_.submit(p, TurnOpts(max_new=60, ignore_eos=True)) for p in prompts]
    sinks = [re_.turns[t].sink for t in tids]
    re_.run_until_idle()
    got = []
    for s in sinks:
        out = []
        while not s.empty():
            ev = s.get()
            if ev[0] == "token":
                out.append(ev[2])
        got.append(out)
    assert got == want
    st = spec.stats
    assert st.rounds >= 20 and st.accepted >= 2 * (st.rounds - 6) and st.folds > 0
    assert ("foldb", 3, 4) in e.runner.graphs                     # the batched fold ran for the three of them


def test_batched_rounds_save_the_boundaries_they_step_over():
    prompts = [toks(40 + 7 * i, 20 + i) for i in range(3)]
    plain = Engine(cfg(), device="cpu")
    want = [plain.generate(p, 70) for p in prompts]
    e = Engine(cfg(snap_decode_stride=1, snap_spec_rollback=True, n_snap_rows=16), device="cpu")        # rows enough that nothing is evicted in this test
    spec = SpecRunner(LookupDraft(2, 8), depth=3, degrade_below=-1.0)
    spec.per_sid = {i: OracleDraft(want[i], len(prompts[i]), 2, 512) for i in range(3)}
    sids = [e.add_sequence(p) for p in prompts]
    outs = [[e.prefill(s)] for s in sids]
    for s in sids:
        spec.after_prefill(e, s)
    while min(len(o) for o in outs) < 60:
        for o, em in zip(outs, spec.round_batch(e, sids)):
            o.extend(em)
    for i, s in enumerate(sids):
        seq = e.seqs[s]
        assert outs[i] == want[i][:len(outs[i])]
        tail = e.states.snaps[seq.tail_hash]
        assert tail.klass == "tail" and tail.n_tokens == seq.n_cached // 16 * 16        # never a whole page behind
    n_cached = [e.seqs[s].n_cached for s in sids]
    for s in sids:
        e.free_sequence(s)
    for i, p in enumerate(prompts):                                # the next turn of each resumes at its rolling snapshot
        follow = p + outs[i][:n_cached[i] - len(p) + 1] + toks(9, 30 + i)
        sid = e.add_sequence(follow)
        assert e.seqs[sid].reused == n_cached[i] // 16 * 16
        e.free_sequence(sid, publish=False)
        assert e.generate(follow, 5) == Engine(cfg(), device="cpu").generate(follow, 5)


def test_lookup_finds_a_repeat_and_its_rejected_drafts_are_rolled_back():
    base = toks(23, 2)
    prompt = base * 3 + base[:9]
    want = Engine(cfg(), device="cpu").generate(prompt, 12)
    e = Engine(cfg(), device="cpu")
    spec = SpecRunner(LookupDraft(1, 8), depth=3, degrade_below=-1.0)
    sid = e.add_sequence(prompt)
    first = e.prefill(sid)
    spec.after_prefill(e, sid)
    e.seqs[sid].tokens[-1] = base[9]                              # pretend the model continued the repeat: the lookup now has a suffix
    out = spec.round(e, sid)
    assert spec.draft.hits == 1 and spec.stats.rounds == 1 and len(out) >= 1
    assert first == want[0]


def test_degrade_after_a_streak_of_rounds_without_an_accepted_draft():
    prompt = toks(60, 3)
    want = Engine(cfg(), device="cpu").generate(prompt, 40)
    e = Engine(cfg(), device="cpu")
    spec = SpecRunner(OracleDraft(want, len(prompt), 0, 512), depth=3, degrade_below=-1.0, degrade_after=4, probe_every=6)
    assert generate_spec(e, prompt, 40, spec) == want
    assert spec.stats.degraded_steps >= 6                         # plain steps while drafting is switched off
    assert spec.stats.rounds >= 4 and spec.stats.accepted == 0


def test_forced_acceptance_harness_emits_the_drafts():
    prompt = toks(50, 4)
    e = Engine(cfg(), device="cpu")
    want = Engine(cfg(), device="cpu").generate(prompt, 30)
    wrong = [(t + 1) % 512 for t in want]                         # drafts that the target would reject
    spec = SpecRunner(OracleDraft(wrong, len(prompt), 7, 512), depth=3, degrade_below=-1.0, force_accept=2)
    out = generate_spec(e, prompt, 12, spec)
    assert len(out) == 12 and spec.stats.accepted == 2 * spec.stats.rounds
    assert out != want[:12]                                       # a throughput harness: the text is the drafts', not the target's


def test_generation_snapshots_are_taken_when_a_round_lands_on_a_page_boundary():
    prompt = toks(60, 5)
    want = Engine(cfg(), device="cpu").generate(prompt, 80)
    e = Engine(cfg(snap_decode_stride=1, snap_spec_rollback=True), device="cpu")
    spec = SpecRunner(OracleDraft(want, len(prompt), 2, 512), depth=3, degrade_below=-1.0)
    sid = e.add_sequence(prompt)
    out = [e.prefill(sid)]
    spec.after_prefill(e, sid)
    while len(out) < 80:
        out.extend(spec.round(e, sid))
    seq = e.seqs[sid]
    assert out[:80] == want and seq.tail_hash is not None
    tails = [s for s in e.states.snaps.values() if s.klass == "tail"]
    # rounds of three tokens step over most page boundaries in mid-round: the state is rolled back to the boundary and saved,
    # so the rolling snapshot never trails the sequence by a whole page
    assert len(tails) == 1 and tails[0].n_tokens == seq.n_cached // 16 * 16 and tails[0].n_tokens > len(prompt)
    e.free_sequence(sid)
    follow = prompt + out[:70] + toks(9, 6)
    sid = e.add_sequence(follow)
    assert e.seqs[sid].reused == tails[0].n_tokens                 # the next turn resumes at the rolling snapshot
    e.free_sequence(sid, publish=False)
    assert e.generate(follow, 6) == Engine(cfg(), device="cpu").generate(follow, 6)


def test_the_engines_own_token_edits_reach_the_lookups_history():
    """Replacing the newest token and excising a page range both edit the history in place; the lookup's array follows."""
    from owl_engine_b200.engine.core import PAGE
    from owl_engine_b200.engine.spec import suffix_lookup

    e = Engine(cfg(), device="cpu")
    lk = LookupDraft(1, 4)
    base = toks(PAGE, 5)
    sid = e.add_sequence(base * 3 + base[:5], reuse=False)
    e.prefill(sid)
    seq = e.seqs[sid]
    assert lk.find(e, sid, 3) == suffix_lookup(seq.tokens, 3, 1, 4)
    ep = seq.tokens_epoch
    e.set_last_token(sid, (seq.tokens[-1] + 1) % 50)
    assert seq.tokens_epoch == ep + 1 and lk.find(e, sid, 3) == suffix_lookup(seq.tokens, 3, 1, 4)
    n = len(seq.tokens)
    e.drop_ranges(sid, [(PAGE, 2 * PAGE)])
    seq.tokens.extend(base[:PAGE])                                 # back to the old length before the next lookup
    assert len(seq.tokens) == n and seq.tokens_epoch == ep + 2
    assert lk.find(e, sid, 3) == suffix_lookup(seq.tokens, 3, 1, 4)
