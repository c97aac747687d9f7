"""GDN state rows and snapshots, and agent sessions.

``StateStore`` lends recurrent-state rows (the concurrency ceiling) to running turns and keeps
*snapshots*: copies of a row taken at block-aligned positions, keyed by the chain hash of the prefix
they correspond to, so a prefix-cache hit can restore the linear-attention state that matches the
reused KV blocks. Classes order the eviction (``store/snap_policy.py``); a snapshot whose row is recycled can move to a lower
tier (pinned host memory, then disk) through the ``on_evict`` hook and stays findable in ``lower``.
``SessionTable`` maps a client ``session`` id to its last chain for multi-turn reuse.

Reference counterpart: ``crates/store/src/{state,session}.rs``.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field

from . import snap_policy as P


@dataclass
class Snapshot:
    row: int               # state row that holds the copy (-1 while the bytes live in a lower tier)
    chain_hash: int        # prefix identity (hash of the last block included)
    n_tokens: int
    klass: str             # "transient" | "extra" | "binary" | "tail" | "dense" | "durable" (eviction order, store/snap_policy.py)
    rank: int = 0          # rung of the binary ladder
    session: str | None = None
    tier: str = "device"   # "device" | "host" | "disk"
    last_use: int = 0      # the store's use counter at the last touch (a counter, not a clock: the ranks of a tensor-parallel
                           # job must pick the same victims, and their clocks differ)


class StateStore:
    def __init__(self, n_rows: int, n_snap_rows: int = 0, cap: P.SessionCap | None = None):
        """Rows 0..n_rows-1 are lendable; rows n_rows..n_rows+n_snap_rows-1 hold snapshots.

        ``on_evict(snapshot) -> "host" | "disk" | None`` is called before a snapshot's row is recycled: the owner of the
        lower tiers copies the row's bytes away and answers where they went (None = dropped); the snapshot then stays
        findable in ``lower``. ``on_forget(snapshot)`` tells that owner that a lower-tier snapshot is gone for good."""
        self.free_rows = list(range(n_rows - 1, -1, -1))
        self.snap_rows = list(range(n_rows + n_snap_rows - 1, n_rows - 1, -1))
        self.snaps: dict[int, Snapshot] = {}     # chain_hash -> snapshot in a state row
        self.lower: dict[int, Snapshot] = {}     # chain_hash -> snapshot whose bytes are on the host or on disk
        self.lent: dict[int, int] = {}           # turn -> row
        self.cap = cap or P.SessionCap()
        self.on_evict = None
        self.on_forget = None
        self.evicted = self.skipped = 0
        self._uses = 0

    def _touch(self, s: Snapshot) -> None:
        self._uses += 1
        s.last_use = self._uses

    def borrow(self, turn: int) -> int | None:
        if not self.free_rows:
            return None
        r = self.free_rows.pop()
        self.lent[turn] = r
        return r

    def give_back(self, turn: int) -> None:
        r = self.lent.pop(turn, None)
        if r is not None:
            self.free_rows.append(r)

    # -- snapshots ------------------------------------------------------------------------------------------------------
    def _recycle(self, s: Snapshot, demote: bool) -> None:
        """Take a live snapshot out of its row; with ``demote`` the lower tiers get the chance to keep its bytes."""
        del self.snaps[s.chain_hash]
        tier = self.on_evict(s) if demote and self.on_evict is not None and s.klass != "transient" else None
        self.snap_rows.append(s.row)
        self.evicted += 1
        if tier:
            s.row, s.tier = -1, tier
            self.lower[s.chain_hash] = s

    def forget(self, chain_hash: int) -> None:
        """Drop a snapshot wherever it lives (a rolling snapshot that was superseded, a session-cap replacement)."""
        s = self.snaps.get(chain_hash)
        if s is not None:
            self._recycle(s, demote=False)
            return
        s = self.lower.pop(chain_hash, None)
        if s is not None and self.on_forget is not None:
            self.on_forget(s)

    def of_session(self, session: str) -> list:
        return [s for s in list(self.snaps.values()) + list(self.lower.values()) if s.session == session]

    def snapshot(self, chain_hash: int, n_tokens: int, klass: str = "durable", rank: int = 0, session: str | None = None) -> int | None:
        """Reserve a snapshot row for a prefix. The caller copies the live row into the returned row. When every row is
        taken the snapshot that ``snap_policy.order_key`` ranks lowest leaves (to a lower tier when there is one); a session
        at its cap replaces its own lowest-ranked snapshot or, if the newcomer ranks below everything held, gets None."""
        s = self.snaps.get(chain_hash)
        if s is not None:
            self._touch(s)
            if P.PRIORITY[klass] > P.PRIORITY[s.klass]:
                s.klass, s.rank = klass, rank
            return s.row
        if session is not None and self.cap.cap > 0:
            verdict, victim = self.cap.gate(self.of_session(session), klass, rank)
            if verdict == "skip":
                self.skipped += 1
                return None
            if victim is not None:
                self.forget(victim.chain_hash)
        if not self.snap_rows:
            if not self.snaps:
                return None
            v = min(self.snaps.values(), key=lambda x: P.order_key(x.klass, x.rank, x.last_use))
            self._recycle(v, demote=True)
        stale = self.lower.pop(chain_hash, None)          # being re-taken (or reloaded by the owner of the lower tiers)
        if stale is not None and self.on_forget is not None:
            self.on_forget(stale)
        row = self.snap_rows.pop()
        self.snaps[chain_hash] = Snapshot(row, chain_hash, n_tokens, klass, rank, session)
        self._touch(self.snaps[chain_hash])
        return row

    def supersede(self, chain, n_tokens: int) -> int:
        """A ``durable`` snapshot (the end of a prompt) at ``n_tokens`` of ``chain`` was just taken: live ``durable`` and
        ``tail`` snapshots that lie EARLIER ON THE SAME CHAIN are no longer where this conversation continues from, only
        possible fork points, and are re-classed ``extra`` so that they leave before anybody's current anchor does. (A
        ``tail`` snapshot does not supersede its own prompt's anchor: it lies inside the answer, and a client that renders
        the answer back with other tokens can only resume from the prompt's end.) Returns how many."""
        bt, n = 0, 0
        for s in self.snaps.values():
            if s.klass in ("durable", "tail") and 0 < s.n_tokens < n_tokens:
                bt = bt or max(1, n_tokens // max(1, len(chain)))          # tokens per block of this chain
                i = s.n_tokens // bt - 1
                if 0 <= i < len(chain) and int(chain[i]) == s.chain_hash:
                    s.klass, s.rank = "extra", 0
                    n += 1
        return n

    def find(self, chain_hashes) -> Snapshot | None:
        """Deepest live snapshot along a chain (list of block hashes, shallow -> deep)."""
        for h in reversed(list(chain_hashes)):
            s = self.snaps.get(int(h))
            if s:
                self._touch(s)
                return s
        return None


@dataclass
class Session:
    sid: str
    tokens: list = field(default_factory=list)
    last_seen: float = field(default_factory=time.monotonic)
    turns: int = 0


class SessionTable:
    def __init__(self, cap: int = 1024):
        self.cap, self.sessions = cap, {}

    def get_or_create(self, sid: str) -> Session:
        s = self.sessions.get(sid)
        if s is None:
            if len(self.sessions) >= self.cap:
                oldest = min(self.sessions.values(), key=lambda x: x.last_seen)
                del self.sessions[oldest.sid]
            s = self.sessions[sid] = Session(sid)
        s.last_seen = time.monotonic()
        return s

    def commit(self, sid: str, tokens: list) -> None:
        s = self.get_or_create(sid)
        s.tokens, s.turns = list(tokens), s.turns + 1

    @staticmethod
    def common_prefix(a: list, b: list) -> int:
        n = min(len(a), len(b))
        i = 0
        while i < n and a[i] == b[i]:
            i += 1
        return i
