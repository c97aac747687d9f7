"""Speculative decoding: greedy output is identical to plain decoding for every draft source and
acceptance length; rollback folds run; the MTP head's device chain works."""
import pytest
import torch

from owl_engine_b200.engine.core import Engine, EngineConfig
from owl_engine_b200.engine.spec import LookupDraft, MtpDraft, OracleDraft, SpecRunner, generate_spec
from owl_engine_b200.models.mtp import MtpHead

pytestmark = pytest.mark.gpu


def make_engine():
    eng = Engine(EngineConfig(model="test-hybrid", snap_cut=True, n_pages=128, n_slots=4, n_snap_rows=2, max_seqs=4, max_seq=512,
                              prefill_chunk=64))
    # the plain baseline uses the same row-count-independent arithmetic a speculating engine switches to
    eng.runner.uniform_rows = True
    return eng


def prompt(n=41, seed=0, vocab=512):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


@pytest.mark.parametrize("accept", [0, 1, 2, 3])
def test_forced_acceptance_equals_plain_decoding(accept):
    eng = make_engine()
    p = prompt()
    plain = eng.generate(p, 28)
    spec = SpecRunner(OracleDraft(plain, len(p), accept, eng.spec.vocab), depth=3, degrade_below=-1.0)
    got = generate_spec(eng, p, 28, spec)
    assert got == plain
    st = spec.stats
    assert st.rounds > 0 and st.mean_accept == pytest.approx(min(accept, 3), abs=0.35)
    if accept < 3:
        assert st.folds > 0          # a rejected row forces restore + fold
    if accept == 3:
        assert st.emitted / st.rounds > 3.5


def test_mtp_head_and_lookup_drafts_keep_the_output():
    eng = make_engine()
    p = prompt(seed=2)
    plain = eng.generate(p, 24)
    head = MtpHead(eng.runner, seed=5)
    spec = SpecRunner(MtpDraft(head), depth=3, degrade_below=-1.0)
    assert generate_spec(eng, p, 24, spec) == plain
    assert spec.stats.rounds > 0 and spec.stats.drafted >= 3 * spec.stats.rounds - 3
    # suffix lookup on a periodic prompt: the model output need not be periodic, the invariant must hold
    rep = (prompt(7, seed=3) * 6)[:40]
    plain2 = eng.generate(rep, 16)
    spec2 = SpecRunner(LookupDraft(min_match=2), depth=3, degrade_below=-1.0)
    assert generate_spec(eng, rep, 16, spec2) == plain2


def test_degrade_after_low_acceptance():
    eng = make_engine()
    p = prompt(seed=4)
    plain = eng.generate(p, 40)
    spec = SpecRunner(OracleDraft(plain, len(p), 0, eng.spec.vocab), depth=2, window=4, degrade_below=0.5, cooldown=8)
    assert generate_spec(eng, p, 40, spec) == plain
    assert spec.stats.degraded_steps >= 8


@pytest.mark.parametrize("depth,accepts", [(3, [3, 1, 0]), (7, [3, 3, 7])])
def test_batched_rounds_equal_plain_decoding_per_sequence(depth, accepts):
    """Several sequences share one (B, T) verify step and one batched fold per round; every sequence's output equals its
    plain greedy continuation, whatever its acceptance length."""
    eng = Engine(EngineConfig(model="test-hybrid", snap_cut=True, n_pages=192, n_slots=4, n_snap_rows=2, spec_rows=4, max_seqs=4,
                              max_seq=512, prefill_chunk=64))
    eng.runner.uniform_rows = True
    n_new = 26
    prompts = [prompt(33 + 5 * i, seed=10 + i) for i in range(len(accepts))]
    plains = [eng.generate(p, n_new) for p in prompts]
    spec = SpecRunner(None, depth=depth, degrade_below=-1.0)
    spec.per_sid = {}
    sids, outs = [], []
    for p, plain, acc in zip(prompts, plains, accepts):
        sid = eng.add_sequence(p, reuse=False)
        outs.append([eng.prefill(sid)])
        spec.per_sid[sid] = OracleDraft(plain, len(p), acc, eng.spec.vocab)
        spec.after_prefill(eng, sid)
        sids.append(sid)
    while any(len(o) < n_new for o in outs):
        live = [i for i, o in enumerate(outs) if len(o) < n_new]
        for i, toks in zip(live, spec.round_batch(eng, [sids[i] for i in live])):
            outs[i].extend(toks)
    for o, plain in zip(outs, plains):
        assert o[:n_new] == plain
    assert spec.stats.folds > 0 and spec.stats.rounds > len(accepts)
    # the verify steps were batched: fewer (B, T) graphs than rounds
    assert any(isinstance(k, tuple) and len(k) > 2 and isinstance(k[0], int) and k[0] > 1 and k[1] > 1 for k in eng.runner.graphs)
