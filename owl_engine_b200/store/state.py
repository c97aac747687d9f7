"""GDN state rows and snapshots, and agent sessions.

``StateStore`` lends recurrent-state rows (the concurrency ceiling) to running turns and keeps
*snapshots*: copies of a row taken at block-aligned positions, keyed by the chain hash of the prefix
they correspond to, so a prefix-cache hit can restore the linear-attention state that matches the
reused KV blocks. Classes: transient (speculative rollback), durable (prefix boundaries), extra.
``SessionTable`` maps a client ``session`` id to its last chain for multi-turn reuse.

Reference counterpart: ``crates/store/src/{state,session}.rs``.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field


@dataclass
class Snapshot:
    row: int               # state row that holds the copy
    chain_hash: int        # prefix identity (hash of the last block included)
    n_tokens: int
    klass: str             # "transient" | "durable" | "extra"
    last_use: float = field(default_factory=time.monotonic)


class StateStore:
    def __init__(self, n_rows: int, n_snap_rows: int = 0):
        """Rows 0..n_rows-1 are lendable; rows n_rows..n_rows+n_snap_rows-1 hold snapshots."""
        self.free_rows = list(range(n_rows - 1, -1, -1))
        self.snap_rows = list(range(n_rows + n_snap_rows - 1, n_rows - 1, -1))
        self.snaps: dict[int, Snapshot] = {}     # chain_hash -> snapshot
        self.lent: dict[int, int] = {}           # turn -> row

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

    def snapshot(self, chain_hash: int, n_tokens: int, klass: str = "durable") -> int | None:
        """Reserve a snapshot row for a prefix (evicting the least recently used one when full).
        The caller copies the live row into the returned row."""
        if chain_hash in self.snaps:
            s = self.snaps[chain_hash]
            s.last_use = time.monotonic()
            return s.row
        if not self.snap_rows:
            victims = sorted((s for s in self.snaps.values() if s.klass != "durable"), key=lambda s: s.last_use) or \
                sorted(self.snaps.values(), key=lambda s: s.last_use)
            if not victims:
                return None
            v = victims[0]
            del self.snaps[v.chain_hash]
            self.snap_rows.append(v.row)
        row = self.snap_rows.pop()
        self.snaps[chain_hash] = Snapshot(row, chain_hash, n_tokens, klass)
        return row

    def find(self, chain_hashes) -> Snapshot | None:
        """Deepest snapshot along a chain (list of block hashes, shallow -> deep)."""
        for h in reversed(list(chain_hashes)):
            s = self.snaps.get(int(h))
            if s:
                s.last_use = time.monotonic()
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
