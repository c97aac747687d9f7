"""The relocation facade on the CPU: a small pool of plain tensors goes through pressure (device -> host -> disk -> drop),
recall in its three modes, a checkpoint and the adoption of the disk tier's index by a fresh store, as after a restart."""
import pytest
import torch

from owl_engine_b200.store import budget as B
from owl_engine_b200.store.kv import KvStore
from owl_engine_b200.store.rel import Rel
from owl_engine_b200.store.state import StateStore
from owl_engine_b200.store.tiers import DiskTier, HostTier, Mover, page_bytes
from owl_engine_b200.utils.ledger import BudgetError, DeviceLedger

PAGE = 16


class Pool:
    """Device pool stand-in: two layers, 12 pages; rows of recurrent state."""

    def __init__(self, n_pages=12, rows=6):
        self.device = torch.device("cpu")
        g = torch.Generator().manual_seed(0)
        self.k_pool = torch.randint(0, 255, (2, n_pages, PAGE, 2, 8), dtype=torch.uint8, generator=g)
        self.v_pool = torch.randint(0, 255, (2, n_pages, PAGE, 2, 8), dtype=torch.uint8, generator=g)
        self.k_scale = self.v_scale = None
        self.conv_state = torch.randn(3, rows, 10, 3, generator=g)
        self.rec_state = torch.randn(3, rows, 2, 4, 4, generator=g)


def make(tmp, n_pages=12, host_pages=4, disk_pages=6):
    pool = Pool(n_pages)
    kv, st = KvStore(n_pages, PAGE), StateStore(2, 3)
    pb = page_bytes(pool)
    host = HostTier(pb, host_pages * pb, pin=False)
    disk = DiskTier(str(tmp), pb, disk_pages * pb + 10_000_000)
    rel = Rel(kv, st, pool, host, Mover(pool, host), disk, PAGE, B.PressurePolicy(low=0.3, high=0.5))
    return pool, kv, st, rel


def publish(kv, rel, tokens):
    chain = kv.chain(tokens)
    pages = kv.alloc(len(chain))
    kv.publish(chain, pages)
    rel.note_published(chain, tokens)
    kv.unref(pages)                       # the sequence is gone: only the tree references the pages
    return chain, pages


def page_copy(pool, page):
    return torch.cat([pool.k_pool[:, page].reshape(-1), pool.v_pool[:, page].reshape(-1)]).clone()


def test_pressure_cascade_recall_and_restart(tmp_path):
    pool, kv, st, rel = make(tmp_path)
    toks_a = list(range(100, 100 + 6 * PAGE))
    toks_b = list(range(900, 900 + 6 * PAGE))
    chain_a, pages_a = publish(kv, rel, toks_a)
    want_a = [page_copy(pool, p) for p in pages_a]
    chain_b, pages_b = publish(kv, rel, toks_b)
    assert kv.free_pages == 0
    # need 5 pages: leaves of the older chain go to the host tier (4 slots), one of them on to disk
    rel.make_room(5)
    assert kv.free_pages >= 5 and rel.demoted == 5 and rel.spilled == 1 and rel.dropped == 0
    assert rel.last_verdict.sink in ("host", "disk") and rel.last_verdict.satisfied
    got = kv.alloc(5)
    for p in got:                          # the freed pages get new content
        pool.k_pool[:, p] = 7
        pool.v_pool[:, p] = 9
    kv.unref(got)
    # recall of chain a in the three modes
    m, pages, carr = kv.match(chain_a)
    assert m == 6 and carr[0] == 0 and set(carr) >= {0, 1}
    n_down = sum(c != 0 for c in carr)
    kv.unref([p for p, c in zip(pages, carr) if c == 0])
    first_down = min(i for i, c in enumerate(carr) if c != 0)
    assert rel.promote(chain_a, 6, list(pages), carr, lambda: None, mode="resident") == (first_down, set())
    m, pages, carr = kv.match(chain_a)

    def one_page():
        a = kv.alloc(1)
        if a is None:
            rel.make_room(1)
            a = kv.alloc(1)
        return a[0] if a else None
    usable, promoted = rel.promote(chain_a, 6, pages, carr, one_page, mode="sync")
    assert usable == 6 and len(promoted) == n_down
    for i in range(6):                     # every block of the chain is back on the device with its bytes
        assert torch.equal(page_copy(pool, pages[i]), want_a[i]), i
    kv.unref(pages)
    # a durable snapshot at the end of chain a, then a checkpoint and a "restart"
    row = st.snapshot(int(chain_a[-1]), 6 * PAGE)
    want_state = rel._state_bytes(row).clone()
    facts = rel.checkpoint()
    assert facts["indexed"] >= 6 and facts["states"] == 1
    rel.disk.close()

    pool2, kv2, st2, rel2 = make(tmp_path)
    pool2.conv_state.zero_()
    pool2.rec_state.zero_()
    ad = rel2.adopt()
    assert ad["blocks"] >= 6 and ad["states"] == 1 and ad["refused_blocks"] == 0
    m, pages, carr = kv2.match(kv2.chain(toks_a))
    assert m == 6 and set(carr) == {2}
    snap = rel2.find_snapshot(kv2.chain(toks_a))
    assert snap is not None and snap.n_tokens == 6 * PAGE
    assert torch.equal(rel2._state_bytes(snap.row), want_state)

    def one_page2():
        a = kv2.alloc(1)
        return a[0] if a else None
    usable, promoted = rel2.promote(kv2.chain(toks_a), 6, pages, carr, one_page2, mode="sync")
    assert usable == 6
    for i in range(6):
        assert torch.equal(page_copy(pool2, pages[i]), want_a[i]), i
    rel2.disk.close()


def test_adoption_refuses_a_block_that_does_not_belong_to_its_chain(tmp_path):
    pool, kv, st, rel = make(tmp_path)
    toks = list(range(50, 50 + 3 * PAGE))
    chain, pages = publish(kv, rel, toks)
    rel.checkpoint()
    h = int(chain[1])
    rel.disk.index[h]["tokens"][0] += 1          # the recorded tokens no longer hash to the block's name
    rel.disk.save_index(PAGE)
    rel.disk.close()
    pool2, kv2, st2, rel2 = make(tmp_path)
    ad = rel2.adopt()
    assert ad["refused_blocks"] == 1 and kv2.node(h) is None and kv2.node(int(chain[0])) is not None
    rel2.disk.close()


def test_watermark_relief_and_modes(tmp_path):
    pool, kv, st, rel = make(tmp_path, n_pages=12, host_pages=8)
    publish(kv, rel, list(range(10 * PAGE)))
    assert kv.free_pages == 2                     # under the low watermark (30 % of 12)
    n = rel.relieve()
    assert n > 0 and kv.free_pages >= int(0.5 * 12) - 0 and rel.demoted == n
    assert rel.relieve() == 0                     # above the low mark now
    rel.disk.close()


def test_disk_tier_index_round_trip_with_background_writer(tmp_path):
    d = DiskTier(str(tmp_path), 64, 10_000)
    data = torch.arange(64, dtype=torch.uint8)
    assert d.spill(11, 0, list(range(16)), data, tag=5) and d.spill(12, 11, list(range(16, 32)), data + 1)
    out = torch.zeros(64, dtype=torch.uint8)
    d.fill(12, out)                               # served from the pending copy or the file, whichever exists
    assert torch.equal(out, data + 1)
    assert d.put_state(12, 32, torch.arange(10, dtype=torch.float32))
    assert d.save_index(16) == 2
    d.close()
    e = DiskTier(str(tmp_path), 64, 10_000)
    assert e.load_index() == 2 and e.index[11] == {"parent": 0, "tag": 5, "tokens": list(range(16))}
    assert e.chain_order() == [11, 12] and e.states[12]["n_tokens"] == 32
    assert torch.equal(e.get_state(12).view(torch.float32), torch.arange(10, dtype=torch.float32))
    e.drop(11)
    assert e.load_index() == 1                    # a block whose file is gone is not adopted
    e.close()


def test_ledger_budget_refusal_and_view():
    led = DeviceLedger("cpu", total_bytes=1 << 20, budget_frac=0.5, reserve_bytes=1 << 16, enforce=True)
    a = led.alloc("pool", "kv pool", (1 << 18,), torch.uint8)
    led.track("view of pool", "kv pool", a[:10])                 # same storage: counted once
    assert led.used() == 1 << 18 and led.room() == (1 << 19) - (1 << 16) - (1 << 18)
    with pytest.raises(BudgetError) as e:
        led.alloc("resident copy", "resident copies", (1 << 19,), torch.uint8)
    assert "resident copy" in str(e.value) and "left of the declared budget" in str(e.value) and led.refused == 1

    class Obj:
        def __init__(self):
            self.w = torch.zeros(100)
            self.parts = [torch.zeros(50), {"x": torch.zeros(25)}]
    assert led.track_tree("obj", "weights", Obj()) == 175 * 4
    v = led.view()
    assert v["buckets"]["kv pool"] == 1 << 18 and v["buckets"]["weights"] == 700 and v["tracked"] == (1 << 18) + 700
    led.release("pool")
    assert led.by_class().get("kv pool", 0) == 0


def test_checkpoint_in_beats_writes_a_bounded_amount_and_saves_the_index_last(tmp_path):
    """The idle checkpoint of the serving loop: every call writes about ``budget_bytes`` and says how much is pending; only
    the call that finishes the job saves the restart index; a restarted engine adopts everything."""
    import os

    from owl_engine_b200.engine.core import Engine, EngineConfig

    kw = dict(model="test-hybrid", n_pages=64, n_slots=4, n_snap_rows=3, max_seqs=4, max_seq=512, prefill_chunk=64,
              host_cache_mb=1, disk_cache_mb=8, disk_dir=str(tmp_path))
    e = Engine(EngineConfig(**kw), device="cpu")
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 500, (100,), generator=g).tolist() for _ in range(3)]
    first = [e.generate(p, 4) for p in prompts]
    pb = e.disk.page_bytes
    beats, pend = 0, None
    while True:
        rep = e.checkpoint(budget_bytes=4 * pb)
        beats += 1
        assert rep["bytes"] <= 4 * pb or rep["blocks"] + rep["states"] == 1      # a beat stays within its budget
        if pend is not None:
            assert rep["pending"] < pend                                          # and always makes progress
        pend = rep["pending"]
        if pend:
            assert "indexed" not in rep and not os.path.exists(tmp_path / "chain.idx")
        else:
            assert rep["indexed"] >= 18
            break
    assert beats >= 4
    e.disk.close()
    e2 = Engine(EngineConfig(**kw), device="cpu")
    assert e2.adopted["blocks"] >= 18 and e2.adopted["states"] == 3
    for p, w in zip(prompts, first):
        assert e2.generate(p, 4) == w
    e2.close()
