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
