"""Speculative decoding: propose -> verify -> accept -> fold.

One round for one sequence whose last token (the *anchor*) has not been fed yet:

1. **propose**: ``depth`` draft tokens from the draft source -- the MTP head (device chain), a
   suffix lookup in the sequence's own history (host), or an oracle that replays a recorded
   continuation (forced-acceptance harness for throughput studies and tests);
2. **verify**: the target runs ``T = 1 + depth`` rows (anchor + drafts) in one step, causal inside
   the rows, with every GDN layer's inputs kept; its GDN state rows were copied to the sequence's
   scratch state row first;
3. **accept**: greedy -- the longest prefix where draft i equals the target's argmax of row i-1;
   sampling -- exact rejection sampling ``min(1, p/q)`` with a residual resample (``accept_rejection``);
   ``m`` accepted drafts emit ``m + 1`` tokens (the target's token after the last accepted row);
4. **fold**: if some rows were rejected the GDN state is restored from the scratch row and only the
   recurrence of the accepted ``m + 1`` rows is replayed (``HybridRunner.fold``), so the state equals
   plain decoding. KV entries of rejected rows stay in their pages but are beyond the context
   length and are overwritten by the next rows.

Greedy speculative output is bit-identical to plain greedy decoding (same kernels, same per-row
arithmetic), which the tests assert. A window of acceptance lengths drives degrade / restore:
after ``window`` rounds with a mean accepted length below ``degrade_below`` the runner falls back
to plain decoding for ``cooldown`` steps.

Reference counterpart: ``crates/engine/src/exec/spec.rs:152,1104,1377``, ``exec/draft.rs``,
``exec/lookup.rs:1-40``, ``exec/proposal_q.rs:417``, constants ``exec/mod.rs:17-90``.
"""
from __future__ import annotations

import random
from dataclasses import dataclass, field

import numpy as np
import torch

from ..models import hybrid as H
from .core import PAGE, Engine


# ---- acceptance rules -------------------------------------------------------------------------
def accept_greedy(drafts: list[int], target: list[int]) -> int:
    """``target[i]`` = the target's argmax after row i (row 0 = anchor). Number of accepted drafts."""
    m = 0
    while m < len(drafts) and drafts[m] == target[m]:
        m += 1
    return m


def accept_rejection(drafts: list[int], q: list[dict], p: list[dict], rng: random.Random) -> tuple[int, int]:
    """Exact speculative sampling. ``q[i]`` / ``p[i]``: proposal / target distributions (token -> prob) for
    draft i; ``p`` has one more entry (the distribution after the last draft). Returns ``(m, next_token)``:
    ``m`` accepted drafts and the token that follows them, distributed exactly as target sampling."""
    for i, d in enumerate(drafts):
        pi, qi = p[i].get(d, 0.0), q[i].get(d, 0.0)
        if qi > 0.0 and rng.random() < min(1.0, pi / qi):
            continue
        # rejected: resample from the residual max(0, p - q), renormalised
        res = {t: max(0.0, pv - q[i].get(t, 0.0)) for t, pv in p[i].items()}
        z = sum(res.values())
        dist = res if z > 0.0 else p[i]
        return i, _draw(dist, rng)
    return len(drafts), _draw(p[len(drafts)], rng)


def _draw(dist: dict, rng: random.Random) -> int:
    z = sum(dist.values())
    u, acc = rng.random() * z, 0.0
    for t, v in dist.items():
        acc += v
        if u <= acc:
            return t
    return next(reversed(dist))


# ---- draft sources ----------------------------------------------------------------------------
def suffix_lookup(hist, k: int, nmin: int, nmax: int):
    """Where did the current suffix occur before, and what followed it? ``hist`` (array of token ids) ends with the token
    fed last. A candidate is any earlier end position ``e`` whose last ``nmin`` tokens equal the last ``nmin`` tokens of
    ``hist``; the match is extended towards older tokens up to ``nmax``; the longest match wins, the more recent one on a
    tie; candidate and suffix may overlap (periodic text). Returns ``(follow, match_len)`` with up to ``k`` tokens that
    followed the match, or None."""
    h = np.asarray(hist)
    n = len(h)
    if nmin < 1 or n < nmin + 1 or k < 1:
        return None
    ends = np.arange(nmin - 1, n - 1)                          # e < n - 1: something must follow the match
    ok = np.ones(len(ends), dtype=bool)
    for j in range(nmin):
        ok &= h[ends - j] == h[n - 1 - j]
    cand = ends[ok]
    if len(cand) == 0:
        return None
    best_e, best_len = -1, 0
    for e in cand[::-1]:                                       # most recent first: on equal length the earlier pick stays
        m = nmin
        while m < nmax and e - m >= 0 and h[e - m] == h[n - 1 - m]:
            m += 1
        if m > best_len:
            best_e, best_len = int(e), m
            if m >= nmax:
                break
    follow = h[best_e + 1:best_e + 1 + k].tolist()
    return follow, best_len


def fuse_lookup(draft: list, follow: list, match_len: int, nmin: int, nstrong: int, agree_min: int) -> list:
    """Lookup-augmented drafting: the looked-up continuation replaces the head of the model's draft when the match is
    strong (``match_len >= nstrong``) or when it is at least ``nmin`` long and agrees with the draft on its first
    ``agree_min`` tokens; positions the lookup does not reach keep the model's tokens."""
    if not follow or match_len < nmin:
        return list(draft)
    agree = 0
    while agree < min(len(draft), len(follow)) and draft[agree] == follow[agree]:
        agree += 1
    if match_len >= nstrong or agree >= agree_min:
        return list(follow) + list(draft[len(follow):])
    return list(draft)


class LookupDraft:
    """Suffix lookup in the sequence's own history (host side): if the last tokens occurred earlier, propose what followed
    (``suffix_lookup``). Alone it is a draft source; next to a draft model it overrides the head of the model's draft
    (``fuse``). The history is kept as a growing array per sequence, so a round costs a few vector compares, not a copy
    of the history."""

    def __init__(self, min_match: int = 2, max_match: int = 8, nstrong: int | None = None, agree: int = 0):
        self.min_match, self.max_match = min_match, max_match
        self.nstrong = min_match if nstrong is None else nstrong
        self.agree = agree
        self._hist: dict = {}          # sid -> (array with spare room, valid length, epoch)
        self.hits = self.lookups = 0

    def _array(self, sid: int, toks: list, epoch: int = 0):
        """The history as an array. Between two calls the list may have grown or been cut at its end; every other edit
        (tokens removed from the middle, the newest token replaced) is announced by a new ``epoch`` and rebuilds the array.
        The last few tokens of the part already held are compared as well, so an unannounced edit near the end is caught."""
        buf, n, ep = self._hist.get(sid, (None, 0, 0))
        m = len(toks)
        g = min(n, 8)
        if buf is None or ep != epoch or m < n or m > len(buf) or (g and buf[n - g:n].tolist() != list(toks[n - g:n])):
            buf = np.empty(max(1024, 2 * m), dtype=np.int64)
            buf[:m] = toks
        elif m > n:
            buf[n:m] = toks[n:m]
        self._hist[sid] = (buf, m, epoch)
        if len(self._hist) > 64:
            self._hist.pop(next(iter(self._hist)))
        return buf[:m]

    def find(self, engine: Engine, sid: int, depth: int):
        self.lookups += 1
        seq = engine.seqs[sid]
        r = suffix_lookup(self._array(sid, seq.tokens, getattr(seq, "tokens_epoch", 0)), depth, self.min_match, self.max_match)
        if r is not None:
            self.hits += 1
        return r

    def propose(self, engine: Engine, sid: int, depth: int) -> list[int]:
        r = self.find(engine, sid, depth)
        return r[0] if r is not None else []

    def fuse(self, draft: list, found) -> list:
        if found is None:
            return list(draft)
        return fuse_lookup(draft, found[0], found[1], self.min_match, self.nstrong, self.agree)

    def observe(self, engine, sid, n_rows, emitted, row0=0):
        pass


class OracleDraft:
    """Replays a recorded continuation with a fixed number of correct drafts per round, then a wrong
    one: the forced-acceptance harness (acceptance length is an input, not a model property)."""

    def __init__(self, continuation: list[int], n_prompt: int, accept: int, vocab: int):
        self.cont, self.n_prompt, self.accept, self.vocab = continuation, n_prompt, accept, vocab

    def propose(self, engine: Engine, sid: int, depth: int) -> list[int]:
        seq = engine.seqs[sid]
        i = len(seq.tokens) - self.n_prompt          # index into the continuation of the NEXT token
        good = self.cont[i:i + min(self.accept, depth)]
        out = list(good)
        if len(out) < depth and i + len(out) < len(self.cont):
            out.append((self.cont[i + len(out)] + 1) % self.vocab)     # a deliberately wrong draft
        return out

    def observe(self, engine, sid, n_rows, emitted, row0=0):
        pass


class MtpDraft:
    """The MTP head as draft source (``models/mtp.py``); optionally overridden by a suffix lookup."""

    def __init__(self, head, lookup: LookupDraft | None = None, window: int = 8192):
        self.head, self.lookup, self.window = head, lookup, window
        self.ready: dict = {}        # sid -> True once the head has absorbed the row before the anchor
        self._chunks: list = []      # (pos0, t, last-layer hiddens) of the prompt chunks just prefetched
        t = head.target
        self._tap = t.spec.n_layers - 1
        if t.taps is None:
            t.taps = {}
        t.taps.setdefault("prefill", {})
        t.taps.setdefault(self._tap, torch.zeros(t.MAX_ROWS, t.spec.hidden, dtype=torch.bfloat16, device=t.device))
        t.tap_sink = self._on_chunk
        t.graphs.clear()

    def _on_chunk(self, pos0: int, t: int, taps: dict) -> None:
        """Keep the target's final hiddens of the prompt chunks (the most recent ``window`` positions)."""
        self._chunks.append((pos0, t, taps[self._tap]))
        while len(self._chunks) > 1 and sum(c[1] for c in self._chunks[1:]) >= self.window:
            self._chunks.pop(0)

    def after_prefill(self, engine: Engine, sid: int) -> None:
        """Fill the head's KV for the prompt (every row but the last, chunk by chunk on the GEMM path), then absorb the
        last prompt row: (first generated token, hidden of the last prompt position)."""
        seq = engine.seqs[sid]
        for pos0, t, h in self._chunks:
            n = t - 1 if pos0 + t >= seq.n_cached else t
            if n > 0 and pos0 + n < len(seq.tokens):
                nxt = torch.tensor(seq.tokens[pos0 + 1:pos0 + n + 1], dtype=torch.int32, device=engine.device)
                self.head.absorb_prefill(nxt, h[:n], pos0, seq.row)
        self._chunks.clear()
        q = seq.n_cached - 1
        self.head.absorb([seq.tokens[-1]], engine.runner.h[:1], q, seq.row, seq.pages)
        self.ready[sid] = True

    def propose(self, engine: Engine, sid: int, depth: int) -> list[int]:
        found = self.lookup.find(engine, sid, depth) if self.lookup is not None else None
        if found is not None and len(found[0]) >= depth and found[1] >= self.lookup.nstrong:
            return found[0]                        # a strong match covers the whole draft: the head need not run
        if not self.ready.get(sid):
            return found[0] if found is not None else []
        draft = self.head.chain(depth).tolist()
        return self.lookup.fuse(draft, found) if self.lookup is not None else draft

    def observe(self, engine: Engine, sid: int, n_rows: int, emitted: list[int], row0: int = 0) -> None:
        """After a verify step: its rows row0..row0+n_rows-1 (this sequence's accepted rows) feed the head, with the
        target's hiddens."""
        seq = engine.seqs[sid]
        q0 = seq.n_cached - n_rows
        self.head.absorb(emitted, engine.runner.h[row0:row0 + n_rows], q0, seq.row, seq.pages)
        self.ready[sid] = True


class DFlash2Draft:
    """The DFlash2 block draft as draft source (``models/dflash2.py``): the target's tap hiddens of every prompt chunk
    and of every accepted row are encoded into the draft's ring KV; a proposal is one captured forward of the 8-row
    block. One sequence at a time (the ring belongs to the sequence that was prefetched last)."""

    def __init__(self, draft, runner, lookup: LookupDraft | None = None):
        self.draft, self.lookup, self.sid = draft, lookup, None
        dev, H = runner.device, runner.spec.hidden
        runner.taps = {i: torch.zeros(runner.MAX_ROWS, H, dtype=torch.bfloat16, device=dev) for i in draft.spec.taps}
        runner.taps["prefill"] = {}
        runner.tap_sink = self._on_chunk
        runner.graphs.clear()
        self.runner = runner

    def _on_chunk(self, pos0: int, t: int, taps: dict) -> None:
        if pos0 < self.draft.n_seen or pos0 == 0:
            self.draft.reset()
        cat = torch.cat([taps[i] for i in self.draft.spec.taps], dim=1)
        for o in range(0, t, self.draft.max_encode):
            self.draft.encode(cat[o:o + self.draft.max_encode], pos0 + o)

    def after_prefill(self, engine: Engine, sid: int) -> None:
        self.sid = sid
        if self.draft.graph is None:
            self.draft.capture()

    def propose(self, engine: Engine, sid: int, depth: int) -> list[int]:
        found = self.lookup.find(engine, sid, depth) if self.lookup is not None else None
        if found is not None and len(found[0]) >= depth and found[1] >= self.lookup.nstrong:
            return found[0]                        # a strong match covers the whole draft: the draft model need not run
        if sid != self.sid:
            return found[0] if found is not None else []
        seq = engine.seqs[sid]
        draft = self.draft.propose(seq.tokens[-1], seq.n_cached, depth)
        return self.lookup.fuse(list(draft), found) if self.lookup is not None else draft

    def observe(self, engine: Engine, sid: int, n_rows: int, emitted: list[int], row0: int = 0) -> None:
        if sid != self.sid:
            return
        seq = engine.seqs[sid]
        cat = torch.cat([self.runner.taps[i][row0:row0 + n_rows] for i in self.draft.spec.taps], dim=1)
        self.draft.encode(cat, seq.n_cached - n_rows)


class DFlash2Pool:
    """DFlash2 for several live sequences: one draft instance (ring KV, block buffers, captured proposal) per sequence over
    ONE shared set of draft weights. ``bind(sid)`` before the sequence's prefill routes the prompt's tap hiddens to its
    instance; ``release(sid)`` returns the instance. The draft forward itself still runs once per sequence and round (an
    8-row block each); the target's verify and fold are batched by ``SpecRunner.round_batch``."""

    def __init__(self, make_draft, n: int, runner, lookup: LookupDraft | None = None):
        self.members = [DFlash2Draft(make_draft(), runner, lookup) for _ in range(n)]
        self.free = list(range(n))
        self.of: dict = {}
        self.runner = runner
        runner.tap_sink = self._on_chunk
        self._cur = None

    def bind(self, sid: int) -> None:
        if not self.free:
            raise RuntimeError("no free draft instance")
        self.of[sid] = self._cur = self.members[self.free.pop()]
        self._cur.draft.reset()

    def release(self, sid: int) -> None:
        m = self.of.pop(sid, None)
        if m is not None:
            self.free.append(self.members.index(m))

    def _on_chunk(self, pos0: int, t: int, taps: dict) -> None:
        if self._cur is not None:
            self._cur._on_chunk(pos0, t, taps)

    def after_prefill(self, engine: Engine, sid: int) -> None:
        self.of[sid].after_prefill(engine, sid)

    def propose(self, engine: Engine, sid: int, depth: int) -> list[int]:
        m = self.of.get(sid)
        return m.propose(engine, sid, depth) if m is not None else []

    def observe(self, engine: Engine, sid: int, n_rows: int, emitted: list[int], row0: int = 0) -> None:
        m = self.of.get(sid)
        if m is not None:
            m.observe(engine, sid, n_rows, emitted, row0)


# ---- the round machine ------------------------------------------------------------------------
@dataclass
class SpecStats:
    rounds: int = 0
    drafted: int = 0
    accepted: int = 0
    emitted: int = 0
    folds: int = 0
    degraded_steps: int = 0
    window: list = field(default_factory=list)

    @property
    def mean_accept(self) -> float:
        return self.accepted / max(1, self.rounds)


class SpecRunner:
    def __init__(self, draft, depth: int = 3, *, window: int = 16, degrade_below: float = 0.3, cooldown: int = 64,
                 depth_min: int | None = None, switch_ctx: int = 0, degrade_after: int = 0, probe_every: int = 8,
                 force_accept: int = -1):
        """``depth_min`` / ``switch_ctx`` (adaptive depth): sequences whose context reached ``switch_ctx`` tokens are drafted
        ``depth_min`` deep (a long context makes every verify row dearer, so fewer speculative rows pay). ``degrade_after``:
        that many rounds in a row without a single accepted draft switch to plain decoding for ``probe_every`` tokens, then
        drafting is tried again (0 = off; the windowed acceptance rule ``degrade_below`` / ``cooldown`` works beside it).
        ``force_accept >= 0``: every round accepts exactly that many drafts whatever the target says -- a throughput
        harness: the emitted text is then the drafts', not the target's."""
        assert 1 <= depth <= 7
        self.draft, self.depth = draft, depth
        self.window, self.degrade_below, self.cooldown = window, degrade_below, cooldown
        self.depth_min, self.switch_ctx = depth_min, switch_ctx
        self.degrade_after, self.probe_every, self.force_accept = degrade_after, probe_every, force_accept
        self.stats = SpecStats()
        self._cool = 0
        self._zero_streak = 0

    def depth_for(self, n_cached: int) -> int:
        if self.depth_min and self.switch_ctx and n_cached >= self.switch_ctx:
            return min(self.depth, self.depth_min)
        return self.depth

    def _accept(self, drafts: list[int], target: list[int]) -> tuple[int, list[int]]:
        """(accepted drafts m, the m + 1 tokens the round emits)."""
        if self.force_accept >= 0:
            m = min(self.force_accept, len(drafts))
            return m, list(drafts[:m]) + [target[m]]
        m = accept_greedy(drafts, target)
        return m, list(target[:m + 1])

    def _note(self, m: int) -> None:
        """Acceptance bookkeeping of one round: the zero-streak rule and the windowed rule, either may start a cooldown."""
        st = self.stats
        self._zero_streak = self._zero_streak + 1 if m == 0 else 0
        if self.degrade_after and self._zero_streak >= self.degrade_after:
            self._cool, self._zero_streak = max(self._cool, self.probe_every), 0
        st.window.append(m)
        if len(st.window) >= self.window:
            if sum(st.window) / len(st.window) < self.degrade_below:
                self._cool = max(self._cool, self.cooldown)
            st.window.clear()

    def after_prefill(self, engine: Engine, sid: int) -> None:
        if not engine.runner.uniform_rows:
            # from here on every step of this engine (plain or verify) uses row-count-independent arithmetic
            engine.runner.uniform_rows = True
            engine.runner.graphs.clear()
        draft = self.draft_of(sid)
        if hasattr(draft, "after_prefill"):
            draft.after_prefill(engine, sid)

    def round(self, engine: Engine, sid: int) -> list[int]:
        """Emit one or more tokens for the sequence (appended to ``seq.tokens``)."""
        st, draft = self.stats, self.draft_of(sid)
        if self._cool > 0:                       # degraded: plain decoding until the cooldown ends
            self._cool -= 1
            st.degraded_steps += 1
            out = engine.decode_step([sid])
            draft.observe(engine, sid, 1, out)
            return out
        seq = engine.seqs[sid]
        depth = self.depth_for(seq.n_cached)
        drafts = draft.propose(engine, sid, depth)[:depth]
        if not drafts:
            out = engine.decode_step([sid])
            draft.observe(engine, sid, 1, out)
            return out
        rows = [seq.tokens[-1]] + drafts
        target = verify_step(engine, sid, rows)
        m, emitted = self._accept(drafts, target)
        n_rows = m + 1
        if n_rows < len(rows):
            # rejected rows advanced the recurrent state: restore and replay the accepted prefix
            engine.pool.copy_slot(engine.spec_row, seq.slot)
            engine.runner.fold_slot.fill_(seq.slot)
            engine.runner.capture_fold(n_rows).replay()
            st.folds += 1
        seq.tokens.extend(emitted)
        pos = seq.n_cached
        if engine.cfg.snap_decode_stride and engine.cfg.snap_spec_rollback:
            from ..store.snap_policy import decode_boundary

            b = decode_boundary(pos, pos + n_rows, PAGE, engine.cfg.snap_decode_stride)
            if b is not None and b < pos + n_rows:
                # the round stepped over a page boundary: roll the state back to the round's start, replay the rows up to the
                # boundary, save that state as the sequence's rolling snapshot, then replay the accepted rows again
                engine.pool.copy_slot(engine.spec_row, seq.slot)
                engine.runner.fold_slot.fill_(seq.slot)
                engine.runner.capture_fold(b - pos).replay()
                seq.n_cached = b
                engine._tail_snapshot(seq, pos)
                engine.pool.copy_slot(engine.spec_row, seq.slot)
                engine.runner.capture_fold(n_rows).replay()
                st.folds += 2
        seq.n_cached = pos + n_rows
        if engine.cfg.snap_decode_stride and seq.n_cached % PAGE == 0:
            engine._tail_snapshot(seq, pos)         # the round ended exactly on a boundary: the row holds that boundary's state
        draft.observe(engine, sid, n_rows, emitted)
        st.rounds += 1
        st.drafted += len(drafts)
        st.accepted += m
        st.emitted += n_rows
        self._note(m)
        return emitted


    # -- several sequences per round ---------------------------------------------------------------------------------
    def draft_of(self, sid: int):
        """The draft source of a sequence: ``self.per_sid[sid]`` when one was registered (sources that keep per-sequence
        state, like the oracle of the forced-acceptance runs), else the shared one."""
        return getattr(self, "per_sid", {}).get(sid, self.draft)

    def round_batch(self, engine: Engine, sids: list[int]) -> list[list[int]]:
        """One speculative round for every listed sequence, the target run as ONE (B, T) verify step per group of
        ``MAX_ROWS // T`` sequences and the recurrent states of all sequences with rejected rows replayed by ONE batched
        fold. Returns the tokens emitted per sequence (appended to their ``seq.tokens``). Needs ``EngineConfig.spec_rows``
        >= the group size (one scratch state row per sequence of a group)."""
        if self._cool > 0 or len(sids) == 1:
            return [self.round(engine, sid) for sid in sids]
        st = self.stats
        depth = min(self.depth_for(engine.seqs[sid].n_cached) for sid in sids)
        drafts = [self.draft_of(sid).propose(engine, sid, depth)[:depth] for sid in sids]
        d = min(len(x) for x in drafts)
        if d == 0:
            out = engine.decode_step(sids)
            for i, (sid, tok) in enumerate(zip(sids, out)):
                self.draft_of(sid).observe(engine, sid, 1, [tok], row0=i)
            return [[tok] for tok in out]
        t = d + 1
        per = max(1, min(engine.runner.MAX_ROWS // t, engine.cfg.spec_rows))
        emitted_all = []
        for g0 in range(0, len(sids), per):
            grp, dr = sids[g0:g0 + per], [x[:d] for x in drafts[g0:g0 + per]]
            rows = [[engine.seqs[sid].tokens[-1]] + x for sid, x in zip(grp, dr)]
            targets = verify_batch(engine, grp, rows)
            slots, tlen, need = [], [], False
            acc, emit = [], []
            for i, sid in enumerate(grp):
                m, em = self._accept(dr[i], targets[i])
                acc.append(m)
                emit.append(em)
                if m + 1 < t:
                    need = True
                    engine.pool.copy_slot(engine.spec_row + i, engine.seqs[sid].slot)
                    slots.append(engine.seqs[sid].slot)
                    tlen.append(m + 1)
                else:
                    slots.append(-1)
                    tlen.append(0)
            if need:
                r = engine.runner
                graph = r.capture_fold_batch(len(grp), t)
                r.fold_slots[:len(grp)].copy_(torch.tensor(slots, dtype=torch.int32))
                r.fold_tlen[:len(grp)].copy_(torch.tensor(tlen, dtype=torch.int32))
                graph.replay()
                st.folds += 1
            pos0 = [engine.seqs[sid].n_cached for sid in grp]
            for i, sid in enumerate(grp):
                engine.seqs[sid].tokens.extend(emit[i])
            if engine.cfg.snap_decode_stride and engine.cfg.snap_spec_rollback:
                from ..store.snap_policy import decode_boundary

                # sequences whose round stepped over a page boundary: roll them back together, replay each up to its
                # boundary (one batched fold), save the states, then replay their accepted rows (a second batched fold)
                cross = []
                for i, sid in enumerate(grp):
                    b = decode_boundary(pos0[i], pos0[i] + acc[i] + 1, PAGE, engine.cfg.snap_decode_stride)
                    if b is not None and b < pos0[i] + acc[i] + 1:
                        cross.append((i, sid, b))
                if cross:
                    r = engine.runner
                    graph = r.capture_fold_batch(len(grp), t)
                    for phase in (0, 1):
                        sl, tl = [-1] * len(grp), [0] * len(grp)
                        for i, sid, b in cross:
                            seq = engine.seqs[sid]
                            engine.pool.copy_slot(engine.spec_row + i, seq.slot)
                            sl[i], tl[i] = seq.slot, (b - pos0[i]) if phase == 0 else acc[i] + 1
                        r.fold_slots[:len(grp)].copy_(torch.tensor(sl, dtype=torch.int32))
                        r.fold_tlen[:len(grp)].copy_(torch.tensor(tl, dtype=torch.int32))
                        graph.replay()
                        st.folds += 1
                        if phase == 0:
                            for i, sid, b in cross:
                                seq = engine.seqs[sid]
                                seq.n_cached = b
                                engine._tail_snapshot(seq, pos0[i])
                                seq.n_cached = pos0[i]
            for i, sid in enumerate(grp):
                seq, n_rows = engine.seqs[sid], acc[i] + 1
                emitted = emit[i]
                seq.n_cached = pos0[i] + n_rows
                if engine.cfg.snap_decode_stride and seq.n_cached % PAGE == 0:
                    engine._tail_snapshot(seq, pos0[i])
                self.draft_of(sid).observe(engine, sid, n_rows, emitted, row0=i * t)
                st.rounds += 1
                st.drafted += d
                st.accepted += acc[i]
                st.emitted += n_rows
                self._note(acc[i])
                emitted_all.append(emitted)
        return emitted_all


def generate_spec(engine: Engine, prompt: list[int], max_new_tokens: int, spec: SpecRunner, eos: int | None = None) -> list[int]:
    """Greedy generation with speculative rounds (the speculative twin of ``Engine.generate``)."""
    sid = engine.add_sequence(prompt)
    try:
        out = [engine.prefill(sid)]
        spec.after_prefill(engine, sid)
        while len(out) < max_new_tokens and (eos is None or eos not in out):
            out.extend(spec.round(engine, sid))
        if eos is not None and eos in out:
            out = out[:out.index(eos) + 1]
        return out[:max_new_tokens]
    finally:
        engine.free_sequence(sid, publish=False)


def verify_batch(engine: Engine, sids: list[int], rows: list[list[int]]) -> list[list[int]]:
    """Run the target over ``rows[i]`` (anchor + drafts, the same count T for every sequence) of every listed sequence as
    one (B, T) step; returns the argmax after each row, per sequence. Each sequence's GDN state is first copied to its own
    scratch row (``engine.spec_row + i``); every GDN layer's inputs are kept for the fold."""
    r = engine.runner
    b, t = len(sids), len(rows[0])
    m = b * t
    assert all(len(x) == t for x in rows) and m <= r.MAX_ROWS and b <= engine.cfg.spec_rows
    if r.gdn_save is None:
        r.enable_gdn_save()
        r.uniform_rows = True
        r.capture_fold(1)
    engine._last_rows = {}
    lay = H.StepLayout(b, t)
    hi = engine.h_inp_np
    ctx_max = 0
    for i, sid in enumerate(sids):
        seq = engine.seqs[sid]
        pos = seq.n_cached
        engine._ensure_pages(seq, pos + t + 1)
        engine.pool.copy_slot(seq.slot, engine.spec_row + i)
        for j, tok in enumerate(rows[i]):
            p, q = pos + j, i * t + j
            hi[lay.ids + q] = tok
            hi[lay.pos3 + q] = hi[lay.pos3 + m + q] = hi[lay.pos3 + 2 * m + q] = p + seq.rope_delta
            hi[lay.kv_slot + q] = seq.pages[p // PAGE] * PAGE + p % PAGE
        hi[lay.ctx + i] = pos + t
        hi[lay.gslot + i] = seq.slot
        hi[lay.bt_row + i] = seq.row
        ctx_max = max(ctx_max, pos + t)
    graph = r.capture(b, t, ctx_hint=engine._ctx_bucket(ctx_max))
    n = lay.size
    r.inp[:n].copy_(engine.h_inp[:n], non_blocking=True)
    graph.replay()
    engine.h_tok[:m].copy_(r.out_tok[:m], non_blocking=True)
    if not engine.mock:
        torch.cuda.current_stream().synchronize()
    engine.h2d_bytes += n * 4
    engine.d2h_bytes += m * 4
    engine._check_status()
    return [[int(engine.h_tok_np[i * t + j]) for j in range(t)] for i in range(b)]


def verify_step(engine: Engine, sid: int, rows: list[int]) -> list[int]:
    """Run the target over ``rows`` (anchor + drafts) as one (1, T) step; returns the argmax after each row.
    The sequence's GDN state is copied to the engine's scratch row first; every GDN layer's inputs are kept."""
    seq, r = engine.seqs[sid], engine.runner
    t, pos = len(rows), seq.n_cached
    engine._ensure_pages(seq, pos + t + 1)
    if r.gdn_save is None:
        r.enable_gdn_save()
        r.uniform_rows = True
        r.capture_fold(1)          # allocates fold_slot
    engine.pool.copy_slot(seq.slot, engine.spec_row)
    engine._last_rows = {}          # the query buffer now holds verify rows, not decode rows
    lay = H.StepLayout(1, t)
    hi = engine.h_inp_np
    for i, tok in enumerate(rows):
        p = pos + i
        hi[lay.ids + i] = tok
        hi[lay.pos3 + i] = p + seq.rope_delta
        hi[lay.pos3 + t + i] = p + seq.rope_delta
        hi[lay.pos3 + 2 * t + i] = p + seq.rope_delta
        hi[lay.kv_slot + i] = seq.pages[p // PAGE] * PAGE + p % PAGE
    hi[lay.ctx] = pos + t
    hi[lay.gslot] = seq.slot
    hi[lay.bt_row] = seq.row
    graph = r.capture(1, t, ctx_hint=engine._ctx_bucket(pos + t))
    n = lay.size
    r.inp[:n].copy_(engine.h_inp[:n], non_blocking=True)
    graph.replay()
    engine.h_tok[:t].copy_(r.out_tok[:t], non_blocking=True)
    if not engine.mock:
        torch.cuda.current_stream().synchronize()
    engine.h2d_bytes += n * 4
    engine.d2h_bytes += t * 4
    return [int(x) for x in engine.h_tok_np[:t]]
