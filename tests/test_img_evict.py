"""Leave-gap deletion of image segments: padding rule, recognition of deletions, page map, position ledger (host side)."""
from owl_engine_b200.engine import img_evict as E

PAGE, PAD = 16, 999


def _history():
    text = lambda n, base: list(range(base, base + n))
    a, img1, b, img2, c = text(21, 100), [7] * 40, text(9, 200), [8] * 33, text(5, 300)
    ids = a + img1 + b + img2 + c
    spans = [(21, 61), (70, 103)]
    return ids, spans, (a, img1, b, img2, c)


def test_pad_rule_aligns_segments_and_is_invertible():
    ids, spans, _ = _history()
    seq = E.pad_rule(ids, spans, PAGE, PAD)
    for sp in seq.spans:
        assert sp.start % PAGE == 0 and sp.hi % PAGE == 0
        assert seq.ids[sp.lo:sp.start] == [PAD] * sp.pad_before and seq.ids[sp.end:sp.hi] == [PAD] * sp.pad_after
    assert E.unpad(seq) == ids and E.client_spans(seq) == spans
    # the rule is idempotent on the prefix: appending text does not move anything that was already placed
    seq2 = E.pad_rule(ids + [1, 2, 3], spans, PAGE, PAD)
    assert seq2.ids[:len(seq.ids)] == seq.ids and seq2.spans == seq.spans


def test_deletions_are_recognised_and_compiled_to_pages():
    ids, spans, (a, img1, b, img2, c) = _history()
    old = E.pad_rule(ids, spans, PAGE, PAD)
    # drop the first screenshot, append a new turn
    r = E.detect_deletions(old, a + b + img2 + c + [5, 6])
    assert r is not None
    ranges, suffix = r
    sp = old.spans[0]
    assert ranges == [(sp.start, sp.hi)]
    assert suffix == [5, 6]
    after = E.apply_deletions(old, ranges)
    assert E.unpad(after) == a + b + img2 + c and len(after.spans) == 1
    assert after.spans[0].start % PAGE == 0 and after.ids[after.spans[0].start:after.spans[0].end] == img2
    again = E.detect_deletions(after, a + b + c + [1])                              # the other screenshot goes a turn later
    assert again is not None and again[0] == [(after.spans[0].start, after.spans[0].hi)] and again[1] == [1]
    lo, hi = ranges[0]
    assert lo % PAGE == 0 and hi % PAGE == 0
    pages = E.page_map(len(old.ids), ranges, PAGE)
    assert pages == [p for p in range((len(old.ids) + PAGE - 1) // PAGE) if not lo // PAGE <= p < hi // PAGE]
    # both screenshots dropped; nothing dropped; an edit inside the text is not a deletion
    both = E.detect_deletions(old, a + b + c)
    assert both is not None and len(both[0]) == 2 and both[1] == []
    assert E.detect_deletions(old, ids + [9]) == ([], [9])
    assert E.detect_deletions(old, a[:-1] + [0] + img1 + b + img2 + c) is None
    assert E.detect_deletions(old, a + img1[:-1] + b + img2 + c) is None           # a partial image is not a deletion


def test_position_ledger_keeps_holes():
    pos = list(range(100))
    kept, nxt = E.positions_after_splice(pos, [(32, 64)])
    assert kept == list(range(32)) + list(range(64, 100)) and nxt == 100
    kept2, nxt2 = E.positions_after_splice(kept + [100, 101], [(48, 64)])            # a second deletion later on
    assert nxt2 == 102 and len(kept2) == len(kept) + 2 - 16


def test_pad_rule_continues_a_live_sequence_from_its_cache_index():
    """A suffix appended at cache index 37: its droppable segment starts and ends on page boundaries of the SEQUENCE."""
    suffix = list(range(100, 130))
    ps = E.pad_rule(suffix, [(5, 17)], 16, 0, base=37)
    sp = ps.spans[0]
    assert sp.start % 16 == 0 and sp.hi % 16 == 0 and sp.start == 48 and sp.end == 60 and sp.hi == 64
    assert ps.ids[:5] == suffix[:5] and ps.ids[5:11] == [0] * 6 and ps.ids[11:23] == suffix[5:17]
    whole = E.PaddedSeq(list(range(37)) + ps.ids, ps.spans)
    assert E.unpad(whole) == list(range(37)) + suffix
    r, tail = E.detect_deletions(whole, list(range(37)) + suffix[:5] + suffix[17:] + [7])
    assert r == [(48, 64)] and tail == [7]


def test_identity_ids_tell_same_sized_images_apart():
    pad = 9
    ids = [1, 2, pad, pad, pad, 3, pad, pad, pad, 4]
    a = E.identity_ids(ids, pad, [111, 222])
    assert a[0:2] == [1, 2] and a[5] == 3 and a[9] == 4 and len(set(a[2:5])) == 1 and len(set(a[6:9])) == 1 and a[2] != a[6]
    assert all(t < 0 for t in a[2:5] + a[6:9])
    old = E.pad_rule(a, [(2, 5), (6, 9)], 4, 0)
    # the client drops the FIRST image: with plain pad tokens the two histories would also match "second image dropped"
    new = E.identity_ids([1, 2, 3, pad, pad, pad, 4, 5], pad, [222])
    r, tail = E.detect_deletions(old, new)
    assert r == [(old.spans[0].start, old.spans[0].hi)] and tail == [5]
    assert E.identity_ids(ids, None, []) == ids


def test_vision_expand_reports_droppable_spans_with_their_markers():
    import torch

    from owl_engine_b200.cli import png
    from owl_engine_b200.models import vision as V
    from owl_engine_b200.server.http import Vision

    tower = V.VisionTower(V.tiny_vision(out_hidden=64))
    vis = Vision(tower, pad_id=500)
    red, blue = png.encode_png(96, 64, png.RED), png.encode_png(96, 64, png.BLUE)
    ids = [1, 2, 70, 500, 71, 3, 70, 500, 71, 4]
    out, images, spans = vis.expand(ids, [red, blue], [True, False], (70, 71))
    n = images[0][0].shape[0]
    assert out == [1, 2, 70] + [500] * n + [71, 3, 70] + [500] * n + [71, 4] and len(images) == 2
    assert spans == [(2, 2 + n + 2)]
    out2, _, spans2 = vis.expand(ids, [red, blue], [True, True])        # no marker ids known: the pad runs alone
    assert spans2 == [(3, 3 + n), (3 + n + 3, 3 + 2 * n + 3)] and out2 == out
    assert torch.equal(images[0][0], vis.expand(ids, [red, blue])[1][0][0])
