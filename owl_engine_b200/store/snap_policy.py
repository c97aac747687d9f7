"""Where recurrent-state snapshots are taken, and which of them go first when room runs out.

A hybrid model can only reuse a cached prefix up to a position for which the linear-attention state was saved, so the points
at which states are saved decide what a prefix-cache hit is worth:

* **message boundaries** (``message_points``): conversations fork where a message ends (one system prompt, many users; one tool
  result, many follow-ups). Every occurrence of the chat format's message-open marker gives a candidate at the page boundary
  at or below it. The first one (the end of the system prompt) and the newest ``recent`` ones are always kept; the ones in
  between are thinned so that kept points lie at least ``min_gap`` tokens apart -- a snapshot of the 27B model is about 150 MB.
* **the prompt's last page boundary** (class ``durable``): what a repeated prompt or the next turn of the same conversation hits.
* **generation** (``decode_boundary``): every ``stride`` pages of generated text the newest boundary is saved (class ``tail``,
  rolling: a sequence keeps one), so that the next turn, whose prompt contains this turn's answer, resumes behind the answer
  instead of behind the previous prompt.

``classify`` orders the message points for eviction -- it pins nothing: the newest ``recent`` are ``dense``; the point nearest
below ``prompt_len / 2^k`` is ``binary`` with rank k (a sparse ladder that keeps *some* anchor at every depth; higher k = older
= goes earlier); the rest are ``extra``. ``order_key`` is the eviction order over all classes.

``SessionCap`` bounds the snapshots one session may hold across all tiers; ``extra`` ones may use at most ``cap - reserve`` of it.

Reference counterpart: ``crates/engine/src/serve/msg_boundary.rs:1-130`` (boundary selection and classes),
``crates/engine/src/sched/scheduler.rs:388-412`` (the generation-phase boundary), ``crates/store/src/state.rs`` (classes and the
per-session cap).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

# eviction order: lower goes first
PRIORITY = {"transient": 0, "extra": 1, "binary": 2, "tail": 3, "dense": 4, "durable": 5}


def order_key(klass: str, rank: int, last_use: float) -> tuple:
    """Sort key of a snapshot for eviction: class, then (binary ladder) the older rung first, then least recently used."""
    return (PRIORITY[klass], -rank if klass == "binary" else 0, last_use)


def marker_positions(tokens, open_ids) -> np.ndarray:
    """Indices at which the token sequence ``open_ids`` starts inside ``tokens``."""
    t = np.asarray(tokens, dtype=np.int64)
    m = np.asarray(open_ids, dtype=np.int64)
    if len(m) == 0 or len(t) < len(m):
        return np.zeros(0, dtype=np.int64)
    hit = t[:len(t) - len(m) + 1] == m[0]
    for j in range(1, len(m)):
        hit &= t[j:len(t) - len(m) + 1 + j] == m[j]
    return np.nonzero(hit)[0]


def message_points(tokens, open_ids, page: int, min_gap: int, recent: int) -> list[int]:
    """Page-aligned snapshot points of a prompt, ascending (see the module docstring for the thinning rule)."""
    if page <= 0:
        return []
    cand = np.unique(marker_positions(tokens, open_ids) // page * page)
    cand = [int(c) for c in cand if c > 0]              # nothing precedes a marker in the first page
    dense_from = len(cand) - max(0, recent)
    kept: list[int] = []
    for i, b in enumerate(cand):
        if i == 0 or i >= dense_from or b - kept[-1] >= min_gap:
            kept.append(b)
    return kept


def classify(points: list[int], prompt_len: int, recent: int) -> list[tuple[str, int]]:
    """(class, rank) of each message point, in the order given (ascending positions)."""
    out = [("extra", 0)] * len(points)
    for i in range(max(0, len(points) - max(0, recent)), len(points)):
        out[i] = ("dense", 0)
    k = 1
    while k <= 32 and prompt_len >> k:
        below = [i for i, b in enumerate(points) if b <= prompt_len >> k]
        if below and out[below[-1]][0] == "extra":
            out[below[-1]] = ("binary", k)
        k += 1
    return out


def decode_boundary(pos: int, fed: int, page: int, stride: int) -> int | None:
    """The page boundary to save after generation advanced from ``pos`` to ``fed`` cached tokens: the largest boundary in
    ``(pos, fed]`` whose page number is a multiple of ``stride`` (None: no boundary crossed, not on the stride, or switched off)."""
    if page <= 0 or stride <= 0:
        return None
    b = fed // page * page
    return b if b > pos and (b // page) % stride == 0 else None


@dataclass
class SessionCap:
    """At most ``cap`` snapshots per session over all tiers (0 = unbounded); ``extra`` ones at most ``cap - reserve``."""
    cap: int = 0
    reserve: int = 4

    def gate(self, held: list, klass: str, rank: int = 0):
        """``held``: the session's snapshots as objects with ``klass / rank / last_use``. Returns ``("take", None)`` when there
        is room, ``("take", victim)`` when ``victim`` has to go first, ``("skip", None)`` when the new one is not worth a place."""
        if self.cap <= 0 or klass == "transient":
            return "take", None
        held = [s for s in held if s.klass != "transient"]
        if klass == "extra":
            extras = [s for s in held if s.klass == "extra"]
            room = max(0, self.cap - self.reserve)
            if len(extras) >= room:
                if not extras:
                    return "skip", None
                return "take", min(extras, key=lambda s: s.last_use)       # extras only ever displace extras
        if len(held) < self.cap:
            return "take", None
        victim = min(held, key=lambda s: order_key(s.klass, s.rank, s.last_use))
        if order_key(victim.klass, victim.rank, 0.0)[:2] > order_key(klass, rank, 0.0)[:2]:
            return "skip", None                                            # everything held outranks the newcomer
        return "take", victim
