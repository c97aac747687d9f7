"""Scheduler: a pure host decision from the turn ledger to the next step.

Two decoupled state machines: **admission** (Admit / Hold / Reject a queued turn, from its page
need, the pool state and free GDN rows) and **phase policy** (round-robin between decode and
prefill: a prefill chunk is granted after every ``PREFILL_EVERY`` decode beats, immediately when
nothing is decoding). ``schedule`` returns ``Idle`` or one ``Step``: ``Begin`` (start a queued
turn: borrow a row, plan prefix reuse), ``Prefill`` (one chunk of one turn), ``Decode`` (all
decoding turns, up to ``max_batch`` rows) or ``SpecRound`` (one speculative round of up to ``spec_batch``
turns, when every decoding turn can take one).

Reference counterpart: ``crates/engine/src/sched/{scheduler,sched_policy}.rs``.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from ..store import budget as B

PREFILL_EVERY = 8

QUEUED, PREFILL, DECODE, DONE = "queued", "prefill", "decode", "done"


@dataclass
class TurnView:
    """What the scheduler needs to know about a turn."""
    turn: int
    state: str
    n_prompt: int
    fed: int = 0
    need_pages: int = 0
    spec: bool = False
    arrival: int = 0
    remaining: int = 0                 # decoding turns: tokens until max_new (the retry hint of a rejection is built from it)


@dataclass
class Step:
    kind: str                          # begin | prefill | decode | spec
    turns: list = field(default_factory=list)
    chunk: tuple = (0, 0)              # prefill: (start, end) token positions


IDLE = Step("idle")


class PhaseSched:
    def __init__(self, prefill_every: int = PREFILL_EVERY):
        """``prefill_every``: decode beats between two prefill chunks while both phases have work (the reference's constant is
        8, which protects the decoding turns' inter-token latency; 1 alternates, which gets queued prompts into the decode
        batch soonest and is the throughput setting)."""
        self.decode_beats = 0
        self.rr = 0
        self.prefill_every = max(1, int(prefill_every))

    def pick(self, prefilling: list, decoding: list) -> str:
        if prefilling and (not decoding or self.decode_beats >= self.prefill_every):
            self.decode_beats = 0
            return "prefill"
        if decoding:
            self.decode_beats += 1
            return "decode"
        return "idle"


class Scheduler:
    def __init__(self, max_batch: int, prefill_chunk: int, on_full: str = "reject", spec_batch: int = 1,
                 prefill_every: int = PREFILL_EVERY, clock=None):
        import time

        self.max_batch, self.prefill_chunk, self.on_full = max_batch, prefill_chunk, on_full
        self.spec_batch = spec_batch       # decoding turns one speculative round may cover (the engine's scratch state rows)
        self.phase = PhaseSched(prefill_every)
        self.clock = clock or time.monotonic
        self.held_since: dict = {}         # turn -> when it was first held (queue:<ms> counts from there)
        self.itl_ms = 20.0                 # running estimate of a decode beat, fed by the pump (`note_decode_ms`)
        self.rejections: dict = {}         # turn -> Admission of its rejection (reason + retry hint for the client)
        self.decode_rr = 0

    def note_decode_ms(self, ms: float) -> None:
        self.itl_ms = 0.9 * self.itl_ms + 0.1 * ms

    def admission(self, t: TurnView, free_pages: int, evictable: int, outstanding: int, pool_pages: int,
                  free_rows: int, eta_ms: float = 1000.0) -> B.Admission:
        waited = (self.clock() - self.held_since[t.turn]) * 1e3 if t.turn in self.held_since else 0.0
        return B.decide_admission(t.need_pages, free_pages, evictable, outstanding, pool_pages, free_rows, self.on_full,
                                  waited_ms=waited, eta_ms=eta_ms)

    def schedule(self, turns: list[TurnView], free_pages: int, evictable: int, outstanding: int, pool_pages: int,
                 free_rows: int):
        """Returns (Step, rejected_turn_ids)."""
        rejected = []
        queued = sorted((t for t in turns if t.state == QUEUED), key=lambda t: t.arrival)
        decoding = [t for t in turns if t.state == DECODE]
        # when room can next appear: the decoding turn closest to its token limit, at the measured beat
        eta_ms = min((t.remaining for t in decoding), default=50) * self.itl_ms
        for t in queued:
            adm = self.admission(t, free_pages, evictable, outstanding, pool_pages, free_rows, eta_ms)
            if adm.verdict == B.ADMIT:
                self.held_since.pop(t.turn, None)
                return Step("begin", [t.turn]), rejected
            if adm.verdict == B.REJECT:
                self.held_since.pop(t.turn, None)
                self.rejections[t.turn] = adm
                rejected.append(t.turn)
                continue
            self.held_since.setdefault(t.turn, self.clock())
            break                           # Hold: keep FIFO order, try again next pump
        prefilling = [t for t in turns if t.state == PREFILL]
        what = self.phase.pick(prefilling, decoding)
        if what == "prefill":
            # the turn that is owed most (fewest tokens fed) gets the chunk; ties go round
            least = min(t.fed for t in prefilling)
            owed = [t for t in prefilling if t.fed == least]
            t = owed[self.phase.rr % len(owed)]
            self.phase.rr += 1
            end = min(t.n_prompt, t.fed + self.prefill_chunk)
            return Step("prefill", [t.turn], (t.fed, end)), rejected
        if what == "decode":
            spec = [t for t in decoding if t.spec]
            if spec and len(spec) == len(decoding) and len(spec) <= self.spec_batch:
                # every decoding turn can take a speculative round: one batched verify for all of them
                return Step("spec", [t.turn for t in spec]), rejected
            if len(decoding) > self.max_batch:
                # more decoding turns than batch rows: the window moves on every beat, so nobody waits for somebody else's end
                k = self.decode_rr % len(decoding)
                self.decode_rr += self.max_batch
                batch = (decoding[k:] + decoding[:k])[:self.max_batch]
            else:
                batch = decoding
            return Step("decode", [t.turn for t in batch]), rejected
        return IDLE, rejected

    def take_rejection(self, turn: int) -> B.Admission:
        return self.rejections.pop(turn, B.Admission(B.REJECT, "memory", 1000))
