"""RunningEngine: the turn ledger and the single-threaded pump.

``submit`` queues a turn (token ids + options); every ``pump()`` asks the scheduler for one step
and executes it -- begin (borrow a state row, adopt a cached prefix), one prefill chunk, one batched
decode step, or one speculative round -- and emits events to the turn's sink:

    Prefill{turn, fed, total} | Token{turn, token} | Completed{turn, reason, usage} | Failed{turn, error}

Cancellation takes effect at the next step boundary and still publishes the written prefix. The
pump never blocks except on the step's single device-to-host read.

Reference counterpart: ``crates/engine/src/running.rs`` (``submit_session_opts``, ``pump``,
``cancel_turn``), ``serve/turn.rs`` (events, ``TurnOpts``), ``exec/turn_end.rs``.
"""
from __future__ import annotations

import queue
import time
from dataclasses import dataclass, field

import torch

from ..store import budget as B
from ..utils import log
from ..utils.metrics import METRICS
from ..utils.stepgate import GATE
from . import sampler as S
from .core import PAGE, Engine
from .scheduler import DECODE, DONE, PREFILL, QUEUED, Scheduler, TurnView


@dataclass
class TurnOpts:
    max_new: int = 256
    ignore_eos: bool = False
    sampling: S.SamplingParams = field(default_factory=S.SamplingParams)
    stop_ids: tuple = ()
    eos_ids: tuple = ()
    session: str | None = None
    images: list = field(default_factory=list)      # [(merged embeddings, (t, gh, gw), fingerprint)] in prompt order
    image_pad_id: int | None = None
    evict_spans: list = field(default_factory=list)  # [(start, end)] client-coordinate segments that may be dropped later


@dataclass
class Turn:
    turn: int
    tokens: list
    opts: TurnOpts
    sink: "queue.Queue"
    state: str = QUEUED
    sid: int | None = None
    plan: list = field(default_factory=list)
    n_out: int = 0
    cancelled: bool = False
    arrival: int = 0
    history: set = field(default_factory=set)


class RunningEngine:
    def __init__(self, engine: Engine, max_batch: int = 8, on_full: str = "reject", spec_runner=None,
                 park_sessions: bool = False, max_parked: int = 2, evict_pad_id: int = 0, prefill_every: int = 8,
                 step_profile: bool = False, auto_sessions: bool = False):
        """``park_sessions``: a finished turn of a named session keeps its sequence alive (pages + GDN row) so that the next
        turn continues it: droppable segments the client removed are unlinked in place (leave-gap, ``engine/img_evict.py``) and
        only the new tokens are prefilled. At most ``max_parked`` sequences wait; the oldest is released (and published) when
        a row is needed."""
        self.e = engine
        self.park_sessions, self.max_parked, self.evict_pad_id = park_sessions, max_parked, evict_pad_id
        # session identity = content identity: a turn without a session name continues the parked session whose previous
        # prompt it repeats in full, and is parked under a generated name when it matches none
        self.auto_sessions = auto_sessions and park_sessions
        self.parked_prompt_len: dict = {}      # session -> client-coordinate length of the prompt of its last turn
        self.auto_matched = 0
        self.step_profile = step_profile      # one "engine.step" event per executed step (kind, turns, ms) in the metrics store
        self.parked: dict = {}       # session -> (engine sequence id, PaddedSeq of everything in the sequence, tick)
        self.resumed = self.gap_drops = 0
        self.sched = Scheduler(max_batch, engine.cfg.prefill_chunk, on_full, spec_batch=max(1, getattr(engine.cfg, "spec_rows", 1)),
                               prefill_every=prefill_every)
        self.turns: dict[int, Turn] = {}
        self.reservations = B.Reservations()
        self._next = 0
        self._tick = 0
        self.spec_runner = spec_runner
        self.completed = 0
        self.trace: list = []        # last turns' structured trace (/debug/agent)

    # -- API ------------------------------------------------------------------------------------
    def submit(self, tokens: list[int], opts: TurnOpts | None = None, sink=None) -> int:
        if opts is not None and opts.evict_spans and not self.park_sessions:
            # a droppable mark nobody honours would silently re-prefill the whole history every turn: refuse loudly
            # (reference: crates/engine/src/running.rs:1400-1409)
            raise ValueError("rejected: segments are marked droppable (owl_evict) but image_evict is off in this profile; "
                             "enable [vision] image_evict or remove the marks")
        t = Turn(self._next, list(tokens), opts or TurnOpts(), sink or queue.Queue(), arrival=self._tick)
        self._next += 1
        self.turns[t.turn] = t
        METRICS.count("engine.turns_submitted")
        return t.turn

    def cancel_turn(self, turn: int) -> None:
        t = self.turns.get(turn)
        if t:
            t.cancelled = True

    def idle(self) -> bool:
        return not any(t.state != DONE for t in self.turns.values())

    def queue_facts(self) -> dict:
        st = [t.state for t in self.turns.values()]
        return {"queued": st.count(QUEUED), "prefill": st.count(PREFILL), "decode": st.count(DECODE),
                "free_rows": len(self.e.states.free_rows), "free_pages": self.e.kv.free_pages,
                "sessions": sorted(self.parked), "auto_matched": self.auto_matched,
                "prefix_hits": self.e.prefix_hits, "prefix_lookups": self.e.prefix_lookups}

    # -- pump -----------------------------------------------------------------------------------
    def _views(self) -> list[TurnView]:
        out = []
        for t in self.turns.values():
            if t.state == DONE:
                continue
            fed = self.e.seqs[t.sid].n_cached if t.sid is not None else 0
            need = (len(t.tokens) + t.opts.max_new + PAGE - 1) // PAGE
            if t.state == QUEUED and self.park_sessions and t.opts.session in self.parked:
                # the session's parked sequence already holds most of these pages (resumed, it keeps them; released, they
                # become evictable prefix blocks): only the growth counts against the pool
                psid = self.parked[t.opts.session][0]
                if psid in self.e.seqs:
                    need = max(1, need - len(self.e.seqs[psid].pages))
            # the speculative round accepts by greedy agreement: sampled turns decode plainly so that temperature / top-p /
            # seed keep their meaning
            spec = self.spec_runner is not None and t.opts.sampling.mode == "greedy"
            out.append(TurnView(t.turn, t.state, len(t.tokens), fed, need, spec, t.arrival, max(0, t.opts.max_new - t.n_out)))
        return out

    def pump(self) -> bool:
        """Run one step. Returns False when there was nothing to do."""
        self._tick += 1
        GATE.checkpoint("pump")
        for t in list(self.turns.values()):
            if t.cancelled and t.state != DONE:
                self._finish(t, "cancelled")
        if self._tick % 16 == 0 and self.e.host is not None:
            self.e.relieve()                 # watermark relief: cold prefix blocks leave the pool before a turn needs the room
        kvs = self.e.kv.stats()
        # prefix blocks on the device that no live sequence holds can all make room (leaf by leaf: the LRU list only ever
        # shows the current leaves, which would count a long published chain as one block)
        pinned = sum(s.reused // PAGE for s in self.e.seqs.values())
        evictable = max(kvs["lru_len"], kvs["device_nodes"] - pinned)
        # parked sessions hold pages that no running turn uses: they count as room for admission, and when the turns already
        # admitted need more than is free plus evictable, the session idle longest is released here, between steps (its
        # blocks move to the prefix tree, where the pressure path can reach them)
        def parked_pages():
            return sum(len(self.e.seqs[sid].pages) for sid, _, _ in self.parked.values() if sid in self.e.seqs)
        while self.parked and self.e.kv.free_pages + evictable < self.reservations.outstanding:
            before = parked_pages()
            self._release_parked(min(self.parked, key=lambda k: self.parked[k][2]))
            evictable += before - parked_pages()
        evictable += parked_pages()
        step, rejected = self.sched.schedule(self._views(), self.e.kv.free_pages, evictable,
                                             self.reservations.outstanding, self.e.cfg.n_pages,
                                             # a parked session gives its rows back when a new turn needs them (`_do_begin`)
                                             min(len(self.e.states.free_rows), len(self.e.free_rows)) + len(self.parked))
        for r in rejected:
            t = self.turns.pop(r)          # terminal: the ledger forgets the turn once its last event is out
            t.state = DONE
            adm = self.sched.take_rejection(r)
            why = {"never_fits": "the request is larger than the whole KV pool", "slots": "every sequence slot is in use",
                   "memory": "the KV pool has no room for the request", "queue_timeout": "no room appeared while the request was queued"}
            t.sink.put(("failed", r, f"rejected ({adm.reason}): {why.get(adm.reason, adm.reason)}; retry_after_ms={adm.retry_after_ms}"))
            METRICS.count("engine.rejected." + (adm.reason or "other"))
        if step.kind == "idle":
            return bool(rejected)
        try:
            t0 = time.perf_counter() if self.step_profile else 0.0
            with METRICS.timer("pump." + step.kind):
                getattr(self, "_do_" + step.kind)(step)
            if self.step_profile:
                METRICS.event("engine.step", kind=step.kind, turns=len(step.turns), ms=(time.perf_counter() - t0) * 1e3,
                              free_pages=self.e.kv.free_pages)
        except Exception as ex:  # a failed step fails its turns, the engine keeps serving
            log.error("engine.pump", f"{step.kind} failed: {ex!r}")
            for tid in step.turns:
                t = self.turns.get(tid)
                if t is not None and t.state != DONE:
                    self._finish(t, "failed", error=repr(ex))
        return True

    def run_until_idle(self, max_steps: int = 1 << 30) -> None:
        n = 0
        while not self.idle() and n < max_steps:
            if not self.pump():
                break
            n += 1

    # -- step executors -------------------------------------------------------------------------
    def _match_idle_session(self, t: Turn) -> str | None:
        """The parked session this nameless turn continues: its prompt must repeat the WHOLE prompt of that session's last
        turn (more than a page would not do: the chat template's preamble alone is longer than a page and is common to every
        conversation; and asking for the whole history would never match: the client re-renders the model's answer as text,
        whose tokens need not be the ones that were sampled). The longest such prompt wins."""
        from . import img_evict as E

        ident, best, best_n = None, None, 0
        for name, (sid, hist, _) in self.parked.items():
            n = self.parked_prompt_len.get(name, 0)
            if n <= max(PAGE, best_n) or n > len(t.tokens) or sid not in self.e.seqs:
                continue
            ident = self._ident(t) if ident is None else ident
            if ident[:n] == E.unpad(hist)[:n]:
                best, best_n = name, n
        return best

    def _release_parked(self, session: str, publish: bool = True) -> None:
        self.parked_prompt_len.pop(session, None)
        sid, _, _ = self.parked.pop(session)
        if sid in self.e.seqs:
            self.e.free_sequence(sid, publish=publish)

    def _ident(self, t: Turn) -> list:
        """The turn's client tokens with every image-pad run marked by its image's fingerprint (what histories are compared by)."""
        from . import img_evict as E

        return E.identity_ids(t.tokens, t.opts.image_pad_id, [fp for _, _, fp in t.opts.images])

    def _try_resume(self, t: Turn) -> bool:
        """Continue the session's parked sequence when the new prompt is its history with whole droppable segments removed
        and anything appended (text, and new images with their own droppable marks)."""
        from . import img_evict as E

        ent = self.parked.get(t.opts.session)
        if ent is None:
            return False
        sid, hist, _ = ent
        ident = self._ident(t)
        r = E.detect_deletions(hist, ident) if sid in self.e.seqs else None
        if r is None or not r[1]:
            return False
        ranges, suffix = r
        seq = self.e.seqs[sid]
        if len(hist.ids) != len(seq.tokens):
            return False
        cached_client = len(E.unpad(hist))
        if ranges:
            if any(hi > seq.n_cached for _, hi in ranges):
                return False
            self.e.drop_ranges(sid, ranges)
            hist = E.apply_deletions(hist, ranges)
            self.gap_drops += len(ranges)
        del self.parked[t.opts.session]
        self.parked_prompt_len.pop(t.opts.session, None)
        # the appended part: its real tokens, the images whose pad runs lie in it, and its droppable segments padded from
        # the sequence's current length (the sequence's last sampled token is history too: in seq.tokens, not yet cached)
        cut = len(t.tokens) - len(suffix)
        real = list(t.tokens[cut:])
        new_imgs = t.opts.images[len(seq.images):] if t.opts.images else []
        spans = sorted((s - cut, e - cut) for s, e in t.opts.evict_spans if s >= cut)
        base = len(seq.tokens)
        ps_real = E.pad_rule(real, spans, PAGE, self.evict_pad_id, base)
        ps_id = E.pad_rule(list(suffix), spans, PAGE, self.evict_pad_id, base)
        self.e.append_tokens(sid, ps_real.ids, new_imgs or None, t.opts.image_pad_id)
        seq.reused = min(seq.n_cached, cached_client)
        t.sid, t.padded = sid, E.PaddedSeq(hist.ids + ps_id.ids, hist.spans + ps_id.spans, hist.pads)
        self.resumed += 1
        return True

    def _do_begin(self, step) -> None:
        t = self.turns[step.turns[0]]
        from . import img_evict as E

        t.padded = None
        if self.auto_sessions and t.opts.session is None:
            t.opts.session = self._match_idle_session(t)
            if t.opts.session is not None:
                self.auto_matched += 1
            else:
                t.opts.session = f"auto:{t.turn}"
        if not (self.park_sessions and t.opts.session and self._try_resume(t)):
            if t.opts.session in self.parked:
                self._release_parked(t.opts.session)
            prompt, anchors = t.tokens, None
            if self.park_sessions and t.opts.evict_spans:
                spans = sorted(t.opts.evict_spans)
                prompt = E.pad_rule(t.tokens, spans, PAGE, self.evict_pad_id).ids
                t.padded = E.pad_rule(self._ident(t), spans, PAGE, self.evict_pad_id)     # what later histories are compared with
                # a state snapshot in front of every droppable segment: when the segment goes and the session's sequence is no
                # longer parked, the surviving prefix still has an anchor to resume from
                anchors = [sp.start for sp in t.padded.spans]
            elif self.park_sessions and t.opts.session:
                t.padded = E.PaddedSeq(self._ident(t))
            while True:
                try:
                    t.sid = self.e.add_sequence(prompt, images=t.opts.images or None, image_pad_id=t.opts.image_pad_id,
                                                session=t.opts.session, snap_extra=anchors)
                    break
                except RuntimeError:
                    if not self.parked:
                        raise
                    self._release_parked(min(self.parked, key=lambda k: self.parked[k][2]))
        seq = self.e.seqs[t.sid]
        t.plan = self.e.prefill_plan(t.sid)
        t.state = PREFILL
        self.reservations.reserve(t.turn, (len(t.tokens) + t.opts.max_new + PAGE - 1) // PAGE - len(seq.pages))
        t.sink.put(("prefill", t.turn, seq.n_cached, len(t.tokens)))

    def _do_prefill(self, step) -> None:
        t = self.turns[step.turns[0]]
        lo, hi = t.plan.pop(0)
        last = not t.plan
        tok = self.e.prefill_range(t.sid, lo, hi, want_token=last)
        t.sink.put(("prefill", t.turn, hi, len(t.tokens)))
        if last:
            t.state = DECODE
            if self.spec_runner is not None:
                self.spec_runner.after_prefill(self.e, t.sid)
            if t.opts.sampling.mode != "greedy":
                # the prefill returns the argmax of its last row; a sampled turn draws its first token from the same logits
                tok = self._resample(t, 0)
                self.e.set_last_token(t.sid, tok)
            self._emit(t, tok)

    def _do_decode(self, step) -> None:
        ts = [self.turns[i] for i in step.turns]
        sids = [t.sid for t in ts]
        t0 = time.perf_counter()
        toks = self.e.decode_step(sids)
        self.sched.note_decode_ms((time.perf_counter() - t0) * 1e3)
        for i, t in enumerate(ts):
            tok = toks[i]
            if t.opts.sampling.mode != "greedy":
                tok = self._resample(t, i)
                self.e.set_last_token(t.sid, tok)
            self._emit(t, tok)

    def _do_spec(self, step) -> None:
        ts = [self.turns[i] for i in step.turns]
        if len(ts) == 1:
            outs = [self.spec_runner.round(self.e, ts[0].sid)]
        else:
            outs = self.spec_runner.round_batch(self.e, [t.sid for t in ts])
        for t, toks in zip(ts, outs):
            for tok in toks:
                if t.state == DONE:
                    break
                self._emit(t, tok)

    def _resample(self, t: Turn, row: int) -> int:
        """Sampling modes: the device returns the row's top-32 logits with the repetition penalty
        already applied (``csrc/sample.cu``); temperature / top-k / top-p / the draw run on the host."""
        from ..ops import kernels as K

        r = self.e.runner
        if r.vocab_split:
            # every rank holds a slice of the logits: a per-rank draw would send the ranks down different sequences
            raise RuntimeError("sampling modes other than greedy need the full logits on one rank: serve this profile with "
                               "[parallel] vocab_split = false, or use greedy decoding")
        if not hasattr(self, "_topk"):
            self._topk = K.TopK(r.device, max_rows=r.MAX_ROWS, k=min(32, r.vocab_local))
            self._hist = torch.zeros(r.MAX_ROWS, 4096, dtype=torch.int32, device=r.device)
            self._hist_len = torch.zeros(r.MAX_ROWS, dtype=torch.int32, device=r.device)
        pen = t.opts.sampling.rep_penalty
        hist = sorted(t.history)[-4096:] if pen != 1.0 else []
        if hist:
            self._hist[row, :len(hist)].copy_(torch.tensor(hist, dtype=torch.int32), non_blocking=True)
        self._hist_len[row] = len(hist)
        vals, idx = self._topk(r.logits[row:row + 1], 1, r.vocab_local, hist=self._hist[row:row + 1],
                               hist_len=self._hist_len[row:row + 1], penalty=pen, vocab_offset=self.e.weights.vocab_offset)
        cands = [(i, v) for i, v in zip(idx[0].tolist(), vals[0].tolist()) if i >= 0]
        # an explicit seed makes the stream a function of (seed, step) only, so a request replays exactly
        return S.sample(cands, t.opts.sampling, 0 if t.opts.sampling.seed else t.turn, t.n_out, None)

    def _emit(self, t: Turn, tok: int) -> None:
        t.n_out += 1
        t.history.add(tok)
        o = t.opts
        is_eos = tok in o.eos_ids and not o.ignore_eos
        if not is_eos:
            t.sink.put(("token", t.turn, tok))
        METRICS.count("engine.tokens_out")
        if is_eos:
            self._finish(t, "stop")
        elif tok in o.stop_ids:
            self._finish(t, "stop")
        elif t.n_out >= o.max_new:
            self._finish(t, "length")

    def _finish(self, t: Turn, reason: str, error: str | None = None) -> None:
        usage = {"prompt_tokens": len(t.tokens), "completion_tokens": t.n_out, "cached_tokens": 0}
        if t.sid is not None and t.sid in self.e.seqs:
            usage["cached_tokens"] = self.e.seqs[t.sid].reused
            padded = getattr(t, "padded", None)
            if self.park_sessions and t.opts.session and padded is not None and reason in ("stop", "length", "eos") \
                    and self.spec_runner is None:
                # park: the sequence (pages, GDN row) waits for the session's next turn
                from . import img_evict as E

                seq = self.e.seqs[t.sid]
                gen = seq.tokens[len(padded.ids):]
                if t.opts.session in self.parked and self.parked[t.opts.session][0] != t.sid:
                    # two turns of one session ran side by side (the HTTP layer serialises a session, this interface does
                    # not): the sequence parked by the one that ended first gives way, it must not be orphaned
                    self._release_parked(t.opts.session)
                self.parked[t.opts.session] = (t.sid, E.PaddedSeq(padded.ids + gen, padded.spans, padded.pads), self._tick)
                self.parked_prompt_len[t.opts.session] = len(t.tokens)
                while len(self.parked) > self.max_parked:
                    self._release_parked(min(self.parked, key=lambda k: self.parked[k][2]))
            else:
                if reason in ("cancelled", "failed") and t.state == PREFILL:
                    # stopped between two prefill chunks: keep the state of the point reached, so that the retry of this
                    # prompt resumes behind the blocks published below
                    try:
                        self.e.snapshot_now(t.sid)
                    except Exception as ex:   # noqa: BLE001  (best effort: the turn is ending anyway)
                        log.warn("engine.turn", f"no snapshot at the abort point: {ex!r}")
                self.e.free_sequence(t.sid, publish=True)     # cancelled turns publish their written prefix too
        self.reservations.release(t.turn)
        t.state = DONE
        self.completed += 1
        self.trace.append({"turn": t.turn, "reason": reason, **usage})
        del self.trace[:-64]
        if reason == "failed":
            t.sink.put(("failed", t.turn, error or "failed"))
        else:
            t.sink.put(("completed", t.turn, reason, usage))
        # terminal event is out: drop the turn (tokens, history set, sink) so that a long-running server neither grows nor
        # walks finished turns on every step; cancel_turn tolerates an unknown id
        self.turns.pop(t.turn, None)

    # -- convenience ----------------------------------------------------------------------------
    def generate(self, tokens: list[int], opts: TurnOpts | None = None) -> list[int]:
        tid = self.submit(tokens, opts)
        t = self.turns[tid]             # held here: the ledger drops the turn when it finishes
        self.run_until_idle()
        out = []
        while not t.sink.empty():
            ev = t.sink.get()
            if ev[0] == "token":
                out.append(ev[2])
            elif ev[0] == "failed":
                raise RuntimeError(ev[2])
        return out
