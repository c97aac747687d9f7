"""The store on the host: chain hashes and the prefix tree, budgets and admission, state rows, selection, the coverage probe."""
import numpy as np
import pytest
import torch

from owl_engine_b200.store import budget as B
from owl_engine_b200.store import select as S
from owl_engine_b200.store.kv import DEVICE, HOST, KvStore
from owl_engine_b200.store.state import SessionTable, StateStore
from owl_engine_b200.store.tiers import DiskTier, HostTier


def test_chain_hash_is_prefix_stable_and_tag_sensitive():
    st = KvStore(8, 4)
    a = st.chain(list(range(12)))
    b = st.chain(list(range(12)) + [99, 98, 97, 96])
    assert len(a) == 3 and np.array_equal(a, b[:3]) and len(set(b.tolist())) == 4
    c = st.chain(list(range(12)), tags=[0, 7, 0])
    assert c[0] == a[0] and c[1] != a[1] and c[2] != a[2]


def test_publish_match_refcounts_and_lru_eviction():
    st = KvStore(6, 4)
    toks = list(range(16))
    ch = st.chain(toks)
    pages = st.alloc(4)
    assert st.publish(ch, pages) == 4 and all(st.refcount(p) == 2 for p in pages)
    st.unref(pages)                                      # the sequence is done; the tree keeps them
    m, pg, carr = st.match(st.chain(toks[:8] + [5, 5, 5, 5]))
    assert m == 2 and pg == pages[:2] and carr == [DEVICE, DEVICE]
    # matched pages are pinned: eviction may only take the two unpinned deepest blocks (leaf first)
    vp, vh = st.evict(need_free=6)
    assert vp == [pages[3], pages[2]] and st.free_pages == 4
    st.unref(pg)
    vp, _ = st.evict(need_free=6)
    assert vp == [pages[1], pages[0]] and st.free_pages == 6 and st.stats()["nodes"] == 0


def test_demote_keeps_chain_and_promote_restores():
    st = KvStore(4, 4)
    ch = st.chain(list(range(8)))
    pages = st.alloc(2)
    st.publish(ch, pages)
    st.unref(pages)
    vp, vh = st.evict(need_free=4, demote=True)
    assert len(vp) == 2 and st.stats()["nodes"] == 2 and st.stats()["device_nodes"] == 0
    st.set_carrier(vh[0], HOST, 11)
    m, pg, carr = st.match(ch)
    assert m == 2 and carr.count(HOST) == 2
    new = st.alloc(1)
    st.set_carrier(int(ch[0]), DEVICE, new[0])
    assert st.node(int(ch[0]))["carrier"] == DEVICE and st.refcount(new[0]) == 2


def test_budget_plan_admission_pressure():
    plan = B.MemoryPlan(total=180 << 30, budget_frac=0.95, reserve=1 << 30, weights=15 << 30, gdn_rows=2 << 30,
                        workspace=3 << 30, page_bytes=512 << 10)
    plan.check()
    assert plan.kv_pages > 250_000
    with pytest.raises(B.BudgetError):
        B.MemoryPlan(16 << 30, 0.9, 1 << 30, 15 << 30, 0, 0, 512 << 10).check()
    assert B.check_admission(100, 50, 60, 0, 1000, 1) == B.ADMIT
    assert B.check_admission(100, 50, 60, 20, 1000, 1) == B.REJECT
    assert B.check_admission(100, 50, 60, 20, 1000, 1, "queue:500") == B.HOLD
    assert B.check_admission(2000, 50, 60, 0, 1000, 1, "queue") == B.REJECT
    pp = B.PressurePolicy()
    assert pp.target(200, 1000) == 0 and pp.target(100, 1000) == 150
    v = B.plan_capacity(need=30, free_pages=10, evictable=50, host_free=5, disk_free=100)
    assert (v.evict_pages, v.sink, v.satisfied) == (20, "disk", True)
    led = B.Ledger()
    led.record("weights", "weights", 10); led.record("kv", "pool", 20)
    view = led.view(100, 60)
    assert sum(view["buckets"].values()) == 100


def test_selection_keeps_sink_recent_and_best():
    torch.manual_seed(0)
    nb, hkv, hd = 40, 2, 16
    index = torch.randn(nb, hkv, hd)
    q = index[17].repeat_interleave(2, 0)[None] * 3      # queries aligned with block 17
    scores = S.score_blocks(q, index)
    kept = S.select(scores, nb, budget_blocks=8, sink=2, recent=3)
    assert kept == sorted(kept) and {0, 1, 37, 38, 39, 17} <= set(kept) and len(kept) == 8
    k = torch.randn(5, 2, 16); ang = torch.rand(5, 4)
    from owl_engine_b200.ops.reference import apply_rope
    assert torch.allclose(S.derope(apply_rope(k, ang.cos(), ang.sin()), ang.cos(), ang.sin()), k, atol=1e-5)


def test_tiers_and_restart_index(tmp_path):
    host = HostTier(page_bytes=64, capacity_bytes=64 * 5, pin=False)
    s = host.alloc(); host.slot(s).fill_(7)
    assert host.used == 1 and int(host.slot(s)[0]) == 7
    disk = DiskTier(str(tmp_path), 64, 64 * 2)
    assert disk.spill(0xabc, 0, range(16), host.slot(s)) and disk.spill(0xdef, 0xabc, range(16, 32), host.slot(s))
    assert not disk.spill(0x123, 0, range(16), host.slot(s))        # over capacity
    disk.save_index(16)
    d2 = DiskTier(str(tmp_path), 64, 64 * 2)
    assert d2.load_index() == 2 and d2.index[0xdef]["parent"] == 0xabc
    out = torch.zeros(64, dtype=torch.uint8); d2.fill(0xabc, out)
    assert int(out.sum()) == 7 * 64


def test_state_store_and_sessions():
    ss = StateStore(2, 2)
    assert ss.borrow(1) == 0 and ss.borrow(2) == 1 and ss.borrow(3) is None
    ss.give_back(1)
    assert ss.borrow(3) == 0
    r1, r2 = ss.snapshot(100, 64, "transient"), ss.snapshot(200, 128)
    r3 = ss.snapshot(300, 192)                    # evicts the transient one
    assert {r1, r2} == {2, 3} and r3 == r1 and ss.find([100, 200, 999]).n_tokens == 128
    t = SessionTable()
    t.commit("s", [1, 2, 3, 4])
    assert t.common_prefix(t.get_or_create("s").tokens, [1, 2, 9]) == 2


def test_coverage_probe_finds_the_block_the_queries_attend_to():
    """Keys of one block point along the query direction: the true attention mass concentrates there, and the Mean-K index
    must rank that block first (index curve = oracle curve at k = 1, far above chance). A scrambled index falls to chance."""
    import torch

    from owl_engine_b200.ops import reference as R
    from owl_engine_b200.store import coverage as C
    from owl_engine_b200.store import select as S

    g = torch.Generator().manual_seed(0)
    T, block, hq, hkv, hd, rot = 256, 16, 4, 2, 64, 32
    inv = R.rope_inv_freq(rot, 1e4)
    direction = torch.randn(hkv, hd, generator=g)
    k = torch.randn(T, hkv, hd, generator=g) * 0.3
    k[5 * block:6 * block] += 2.0 * direction                        # the needle block (de-rotated space)
    q = (direction.repeat_interleave(hq // hkv, 0) * 1.5 + torch.randn(3, hq, hd, generator=g) * 0.2)
    ang = lambda pos: (pos.float()[:, None] * inv[None, :], )
    kc, ks = ang(torch.arange(T))[0].cos(), ang(torch.arange(T))[0].sin()
    qpos = torch.tensor([T, T + 1, T + 2])
    qc, qs = ang(qpos)[0].cos(), ang(qpos)[0].sin()
    rope = lambda x, c, s: S.derope(x, c, -s)                           # rotating = de-rotating by the negative angle
    rep = C.probe(rope(q, qc, qs), qpos, rope(k, kc, ks), inv, rot, block, ks=(1, 4))
    assert rep["blocks"] == 16
    one = rep["curve"][1]
    assert one["index"] == one["oracle"] and one["index"] > 0.5 and one["chance"] == 1 / 16
    assert rep["spearman"] > 0.3
    mass = C.block_mass(rope(q, qc, qs), rope(k, kc, ks), block)
    assert abs(float(mass.sum()) - 1.0) < 1e-5 and int(mass.argmax()) == 5
    scrambled = C.coverage_curve(mass, torch.arange(16).float(), ks=(1,))[1]      # scores unrelated to the mass
    assert scrambled["index"] < 0.2
