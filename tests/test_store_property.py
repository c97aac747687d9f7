"""Invariants of the native block ledger and of the leave-gap page arithmetic under random operation sequences."""
import numpy as np
from hypothesis import given, settings, strategies as st

from owl_engine_b200.engine import img_evict as E
from owl_engine_b200.store.kv import DEVICE, KvStore

PAGE = 16


@settings(max_examples=120, deadline=None)
@given(st.lists(st.tuples(st.sampled_from(["new", "free", "match", "evict", "demote"]), st.integers(0, 7), st.integers(1, 5)),
                min_size=5, max_size=60), st.sampled_from(["lru", "lrfu:0.1"]))
def test_pages_are_conserved_and_pinned_pages_are_never_evicted(ops, policy):
    n_pages = 24
    kv = KvStore(n_pages, PAGE)
    kv.set_policy(policy)
    prompts = {i: list(range(i * 1000, i * 1000 + 5 * PAGE)) for i in range(8)}      # eight distinct five-block prompts
    prompts[7] = prompts[0][:2 * PAGE] + prompts[7][2 * PAGE:]                         # one shares a two-block prefix with another
    live: list[tuple[list, int]] = []                                                  # (pages held by a "sequence", prompt id)
    demoted: set = set()

    def check():
        held = sum(len(p) for p, _ in live)
        stats = kv.stats()
        refs = [kv.refcount(p) for p in range(n_pages)]
        assert all(r >= 0 for r in refs)
        assert stats["free_pages"] == sum(1 for r in refs if r == 0)                   # a page is free iff nobody references it
        assert stats["free_pages"] + stats["device_nodes"] + held >= n_pages - held    # every page is free, in the tree or held
        for pages, _ in live:
            assert all(kv.refcount(p) >= 1 for p in pages)

    for op, which, n in ops:
        if op == "new":
            chain = kv.chain(prompts[which][:n * PAGE])
            m, pages, carriers = kv.match(chain)
            keep = [p for p, c in zip(pages, carriers) if c == DEVICE]
            # carriers other than the device do not pin anything; a real engine would promote them first
            usable = 0
            for c in carriers:
                if c != DEVICE:
                    break
                usable += 1
            kv.unref(keep[usable:])
            pages = keep[:usable]
            fresh = kv.alloc(n - usable)
            if fresh is None:
                kv.unref(pages)
            else:
                live.append((pages + fresh, which))
        elif op == "free" and live:
            pages, pid = live.pop(which % len(live))
            chain = kv.chain(prompts[pid][:len(pages) * PAGE])
            kv.publish(chain, pages)
            kv.unref(pages)
        elif op == "match":
            chain = kv.chain(prompts[which][:n * PAGE])
            m, pages, carriers = kv.match(chain)
            assert m <= n and len(pages) == m
            kv.unref([p for p, c in zip(pages, carriers) if c == DEVICE])
        elif op in ("evict", "demote"):
            pinned = {p for pages, _ in live for p in pages}
            victims, hashes = kv.evict(need_free=kv.free_pages + n, demote=op == "demote")
            assert not (set(victims) & pinned)                                         # a page a sequence holds never leaves
            if op == "demote":
                demoted |= {int(h) for h in hashes}
        check()
    for pages, _ in live:
        kv.unref(pages)
    kv.evict(need_free=n_pages)
    assert kv.free_pages == n_pages                                                    # everything comes back in the end


@settings(max_examples=200, deadline=None)
@given(st.lists(st.integers(0, 400), min_size=8, max_size=120), st.lists(st.tuples(st.integers(0, 119), st.integers(1, 30)), max_size=4),
       st.integers(0, 3))
def test_pad_rule_aligns_segments_and_unpad_restores_the_client_view(ids, raw_spans, n_drop):
    spans, cur = [], 0
    for lo, ln in sorted(raw_spans):
        lo = max(lo, cur)
        hi = min(len(ids), lo + ln)
        if hi > lo:
            spans.append((lo, hi))
            cur = hi
    ps = E.pad_rule(ids, spans, PAGE, pad_id=-7)
    assert E.unpad(ps) == list(ids)                                                    # pads are invisible to the client
    assert all(s.start % PAGE == 0 and s.hi % PAGE == 0 for s in ps.spans)             # segment + rear pads = whole pages
    assert E.client_spans(ps) == spans
    again = E.pad_rule(E.unpad(ps), E.client_spans(ps), PAGE, pad_id=-7)
    assert again.ids == ps.ids                                                         # applying the rule again changes nothing
    # the client drops some segments: the server finds exactly those, as page ranges inside the padded sequence
    drop = spans[:n_drop]
    kept = [t for i, t in enumerate(ids) if not any(lo <= i < hi for lo, hi in drop)]
    found = E.detect_deletions(ps, kept + [401, 402])
    if found is not None:
        ranges, suffix = found
        assert all(lo % PAGE == 0 and hi % PAGE == 0 for lo, hi in ranges)
        after = E.apply_deletions(ps, ranges)
        assert E.unpad(after) == kept                                                 # what remains is the client's history


@settings(max_examples=15, deadline=None)
@given(st.lists(st.integers(0, 6000), min_size=1, max_size=80), st.integers(0, 2 ** 31 - 1))
def test_step_ring_delivers_random_sized_messages_intact_and_in_order(sizes, seed):
    import os
    import threading

    from owl_engine_b200.parallel.ring import StepRing

    name = f"/owl_prop_ring_{os.getpid()}_{seed % 100000}"
    ring = StepRing.create(name, 2, capacity=16384)                 # small: the producer keeps running into the readers
    readers = [StepRing.open(name, r, 5.0) for r in range(2)]
    rng = np.random.default_rng(seed)
    msgs = [rng.integers(0, 256, n, dtype=np.uint8).tobytes() for n in sizes]
    got = [[], []]

    def read(i):
        for _ in msgs:
            got[i].append(readers[i].pop_bytes(10.0))
    ts = [threading.Thread(target=read, args=(i,)) for i in range(2)]
    for t in ts:
        t.start()
    for m in msgs:
        ring.push_bytes(m, timeout_s=10.0)
    for t in ts:
        t.join(20)
    for r in readers:
        r.free()
    ring.free()
    assert got[0] == msgs and got[1] == msgs


@settings(max_examples=200, deadline=None)
@given(st.lists(st.integers(0, 5), min_size=0, max_size=400), st.integers(1, 64), st.integers(0, 500), st.integers(0, 6))
def test_message_points_are_page_aligned_ascending_and_keep_the_ends(stream, page, min_gap, recent):
    from owl_engine_b200.store import snap_policy as P

    toks = [9 if x else 1 for x in stream]                          # 1 = the marker
    pts = P.message_points(toks, [1], page, min_gap, recent)
    cand = sorted({i // page * page for i, t in enumerate(toks) if t == 1 and i // page > 0})
    assert pts == sorted(set(pts)) and all(p % page == 0 and p > 0 for p in pts) and set(pts) <= set(cand)
    if cand:
        assert pts[0] == cand[0]                                    # the first boundary is always kept
        tail = cand[max(0, len(cand) - recent):] if recent else []
        assert set(tail) <= set(pts)                                # and the newest `recent`
        middle = [p for p in pts if p not in tail]
        assert all(b - a >= min_gap for a, b in zip(middle, middle[1:]))          # the rest keep their distance
    cls = P.classify(pts, len(toks), recent)
    assert len(cls) == len(pts) and all(c in ("dense", "binary", "extra") for c, _ in cls)
    assert [c for c, _ in cls[max(0, len(cls) - recent):]] == ["dense"] * min(recent, len(cls)) if recent else True
