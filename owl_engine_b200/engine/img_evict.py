"""Prefix-transparent deletion of image segments ("leave-gap"): host-side pure functions.

An agent's history interleaves screenshots and text. When the client drops an old screenshot, the KV of everything before it stays
exact, the pages of the dropped segment are unlinked, and everything after it keeps its KV AND its rotary positions: the position
ledger keeps a hole, new tokens continue from ``max_pos + 1``. Nothing is rotated again, so images can be dropped any number of times
without drift. What follows the hole was computed while the image was visible: that is carried memory, not recomputation; what
precedes it is bit-exact.

To make a segment removable by unlinking whole pages, the engine pads it to page boundaries with ``pad_id`` tokens of its own
(the client never sees them). This module holds the padding rule, its inverse, the recognition of deletions between two client
token lists, the page map of a deletion plan and the position ledger; the device side is ``Engine.drop_ranges`` /
``Engine.extend_sequence``.

Reference counterpart: ``crates/engine/src/vision/img_evict.rs:1-60`` (requirements, leave-gap rationale, rebuild rule),
``crates/engine/src/sched/scheduler.rs:1024`` (``plan_image_leave_gap``).
"""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass(frozen=True)
class ImgSpan:
    start: int          # first token of the segment, padded coordinates
    end: int            # one past its last token
    pad_before: int     # pad tokens the engine put in front of it (they end exactly at ``start``)
    pad_after: int      # pad tokens after it (they start exactly at ``end``)

    @property
    def lo(self) -> int:
        return self.start - self.pad_before

    @property
    def hi(self) -> int:
        return self.end + self.pad_after


@dataclass
class PaddedSeq:
    ids: list = field(default_factory=list)
    spans: list = field(default_factory=list)          # ImgSpan, ascending
    pads: list = field(default_factory=list)           # (lo, hi) of pad runs left behind by deleted segments (their front pads)


def pad_rule(ids: list, spans: list, page: int, pad_id: int, base: int = 0) -> PaddedSeq:
    """``spans``: ``(start, end)`` of the removable segments in CLIENT coordinates, ascending and disjoint. Pads go in front
    of a segment so that it starts on a page boundary and behind it so that it ends on one; applying the rule to an
    already padded prefix changes nothing (position differences are whole pages). ``base``: cache index of ``ids[0]`` when
    the tokens continue a live sequence; the returned spans are then in the sequence's coordinates (``ids`` stay relative)."""
    out, res, cur = [], [], 0
    for s, e in spans:
        assert cur <= s < e <= len(ids)
        out.extend(ids[cur:s])
        before = (-(base + len(out))) % page
        out.extend([pad_id] * before)
        start = base + len(out)
        out.extend(ids[s:e])
        end = base + len(out)
        after = (-end) % page
        out.extend([pad_id] * after)
        res.append(ImgSpan(start, end, before, after))
        cur = e
    out.extend(ids[cur:])
    return PaddedSeq(out, res)


def identity_ids(ids: list, image_pad_id, fingerprints: list) -> list:
    """Token list in which the k-th run of image-pad tokens is replaced by a marker of that image's content fingerprint
    (a negative number: no vocabulary id), so that two screenshots of the same size are different segments when two client
    histories are compared."""
    if image_pad_id is None or not fingerprints:
        return list(ids)
    out, k, prev = [], -1, None
    for t in ids:
        if t == image_pad_id:
            if prev != image_pad_id:
                k += 1
            out.append(-1 - (int(fingerprints[min(k, len(fingerprints) - 1)]) & 0x7FFFFFFF))
        else:
            out.append(t)
        prev = t
    return out


def _pad_runs(seq: PaddedSeq) -> list:
    runs = list(seq.pads)
    for sp in seq.spans:
        if sp.pad_before:
            runs.append((sp.lo, sp.start))
        if sp.pad_after:
            runs.append((sp.end, sp.hi))
    return sorted(runs)


def unpad(seq: PaddedSeq) -> list:
    """The token list the client sees."""
    out, cur = [], 0
    for lo, hi in _pad_runs(seq):
        out.extend(seq.ids[cur:lo])
        cur = hi
    out.extend(seq.ids[cur:])
    return out


def client_spans(seq: PaddedSeq) -> list:
    """The segments in client coordinates."""
    runs = _pad_runs(seq)
    out = []
    for sp in seq.spans:
        shift = sum(hi - lo for lo, hi in runs if hi <= sp.start)
        out.append((sp.start - shift, sp.end - shift))
    return out


def apply_deletions(old: PaddedSeq, ranges: list) -> PaddedSeq:
    """The padded sequence after unlinking ``ranges`` (each the ``[start, hi)`` of a segment): survivors keep their order, the
    front pads of a deleted segment stay behind as a bare pad run."""
    gone = sorted(ranges)
    shift_at = lambda x: sum(hi - lo for lo, hi in gone if hi <= x)
    ids, cur = [], 0
    for lo, hi in gone:
        ids.extend(old.ids[cur:lo])
        cur = hi
    ids.extend(old.ids[cur:])
    spans, pads = [], [(lo - shift_at(lo), hi - shift_at(lo)) for lo, hi in old.pads]
    for sp in old.spans:
        if (sp.start, sp.hi) in gone:
            if sp.pad_before:
                pads.append((sp.lo - shift_at(sp.lo), sp.start - shift_at(sp.lo)))
        else:
            d = shift_at(sp.start)
            spans.append(ImgSpan(sp.start - d, sp.end - d, sp.pad_before, sp.pad_after))
    return PaddedSeq(ids, spans, sorted(pads))


def detect_deletions(old: PaddedSeq, new_client_ids: list):
    """If the new client token list is the old one with some WHOLE segments removed (plus anything appended), return
    ``(ranges, suffix)``: the padded ranges ``[start, hi)`` to unlink (each segment with its rear pads: whole pages; the
    front pads stay in the partially filled page before it) and the client
    tokens that follow the old content. ``None`` when the lists differ in any other way."""
    old_client, cs = unpad(old), client_spans(old)

    def walk(i_span: int, pos_old: int, pos_new: int, dropped: tuple):
        # compare up to the next segment, then branch: kept or dropped
        nxt = cs[i_span][0] if i_span < len(cs) else len(old_client)
        n = nxt - pos_old
        if old_client[pos_old:nxt] != new_client_ids[pos_new:pos_new + n]:
            return None
        if i_span == len(cs):
            return dropped, new_client_ids[pos_new + n:]
        s, e = cs[i_span]
        seg = old_client[s:e]
        if new_client_ids[pos_new + n:pos_new + n + len(seg)] == seg:               # kept
            r = walk(i_span + 1, e, pos_new + n + len(seg), dropped)
            if r is not None:
                return r
        return walk(i_span + 1, e, pos_new + n, dropped + (i_span,))               # dropped

    r = walk(0, 0, 0, ())
    if r is None:
        return None
    dropped, suffix = r
    return [(old.spans[i].start, old.spans[i].hi) for i in dropped], suffix


def page_map(n_tokens: int, ranges: list, page: int) -> list:
    """Old page numbers that survive the deletion of the page-aligned ``ranges``, in order."""
    gone = set()
    for lo, hi in ranges:
        assert lo % page == 0 and hi % page == 0 and lo < hi
        gone.update(range(lo // page, hi // page))
    return [p for p in range((n_tokens + page - 1) // page) if p not in gone]


def positions_after_splice(positions: list, ranges: list) -> tuple:
    """Position ledger after the deletion: the survivors keep their positions; returns ``(positions, next_position)`` with
    ``next_position = max over ALL old positions + 1`` (holes are never refilled)."""
    keep = [True] * len(positions)
    for lo, hi in ranges:
        for i in range(lo, min(hi, len(positions))):
            keep[i] = False
    nxt = (max(positions) + 1) if positions else 0
    return [p for p, k in zip(positions, keep) if k], nxt
