"""Rel: the relocation facade of the KV store. One object plans and executes every move of a KV block between its
carriers (device pool, pinned host tier, disk tier) and keeps the recurrent-state snapshots that make a cached prefix
usable on a hybrid model.

* ``make_room(n)``     need-driven pressure path: ``plan_capacity`` decides how many leaf-LRU blocks leave the device
                       and whether they go to the host tier, through it to disk, or are dropped; the copies are batched
                       (``Mover.copy_out_many``).
* ``relieve()``        watermark-driven: when free pages fall under the policy's low mark, demote up to the high mark
                       (called between steps, so the next admission finds room without moving anything).
* ``promote(...)``     recall of a matched prefix whose blocks live on the host or on disk. Modes: ``"sync"`` (bring
                       everything back, the caller waits on the mover fence), ``"resident"`` (use only what is on the
                       device: a miss from the first demoted block on, nothing moves), ``"host"`` (host-resident blocks
                       come back, disk-resident ones end the prefix).
* ``checkpoint()``     write-through for restarts: every block of the host tier, the device-resident blocks of the prefix
                       tree (optional) and the durable state snapshots are written to the disk tier, then the index.
* ``adopt()``          at boot: the disk tier's index becomes prefix-tree nodes with the disk carrier, and the snapshot
                       files become lazily loadable snapshots, so the first request after a restart can hit the cache.

Reference counterpart: ``crates/store/src/rel.rs`` (the Rel facade, ``adopt_disk*`` at 1221-1290), ``hooks.rs:263``
(``plan_capacity``), ``pressure.rs``, ``crates/engine/src/mem/disk_runtime.rs``.
"""
from __future__ import annotations

import numpy as np
import torch

from . import budget as B

DEVICE, HOST, DISK = 0, 1, 2


class Rel:
    def __init__(self, kv, states, pool, host=None, mover=None, disk=None, block_tokens: int = 16, policy: B.PressurePolicy | None = None,
                 snap_host_bytes: int = 0, no_reclaim: bool = False):
        """``snap_host_bytes``: host memory for recurrent-state snapshots whose row was recycled (0 = they are dropped, or go
        straight to the disk tier when it has a snapshot budget). ``no_reclaim``: the pressure path never takes a cached
        block out of the device pool (diagnostic: a request that does not fit is refused instead)."""
        from collections import OrderedDict

        self.kv, self.states, self.pool = kv, states, pool
        self.host, self.mover, self.disk = host, mover, disk
        self.block_tokens = block_tokens
        self.policy = policy or B.PressurePolicy()
        self.no_reclaim = no_reclaim
        self.host_slot_of: dict[int, int] = {}        # chain hash -> host slot, oldest first
        self.meta: dict[int, tuple] = {}              # chain hash -> (parent hash, tag, tokens as int32 array): what the index stores
        self.snap_host: "OrderedDict[int, torch.Tensor]" = OrderedDict()    # prefix hash -> state bytes on the host, oldest first
        self.snap_host_cap, self.snap_host_used = int(snap_host_bytes), 0
        self.snap_demoted = self.snap_spilled = self.snap_recalled = self.snap_dropped = 0
        self.spilled = self.recalled = self.demoted = self.dropped = self.adopted = 0
        self.last_verdict: B.Verdict | None = None
        states.on_evict, states.on_forget = self._snap_demote, self._snap_forget

    @property
    def disk_snaps(self) -> dict:
        """prefix hash -> n_tokens of the snapshots that exist only on disk."""
        return {h: s.n_tokens for h, s in self.states.lower.items() if s.tier == "disk"}

    # -- bookkeeping at publish time ----------------------------------------------------------------------------------------
    def note_published(self, chain, tokens, tags=None) -> None:
        """Remember parent / tokens of freshly published blocks (the restart index stores them)."""
        bt = self.block_tokens
        toks = np.asarray(tokens, dtype=np.int32)
        parent = 0
        for i, h in enumerate(chain):
            h = int(h)
            if h not in self.meta:
                self.meta[h] = (parent, int(tags[i]) if tags is not None else 0, toks[i * bt:(i + 1) * bt].copy())
            parent = h

    def _meta(self, h: int) -> tuple:
        m = self.meta.get(h)
        if m is not None:
            return m
        nd = self.kv.node(h)
        return ((nd or {}).get("parent", 0), (nd or {}).get("tag", 0), np.zeros(0, dtype=np.int32))

    # -- pressure -------------------------------------------------------------------------------------------------------
    def host_free(self) -> int:
        return len(self.host.free) if self.host is not None else 0

    def disk_free(self) -> int:
        if self.disk is None or self.host is None:
            return 0
        return max(0, (self.disk.capacity - self.disk.used) // self.disk.page_bytes)

    def make_room(self, need: int) -> None:
        """Free device pages until ``need`` are available, cheapest sink first."""
        if self.no_reclaim:
            return
        st = self.kv.stats()
        # leaves expose their parents as they go, so every device-resident tree block is a candidate in the end
        free, evictable = st["free_pages"], st["device_nodes"]
        v = B.plan_capacity(need, free, evictable, self.host_free(), self.disk_free())
        self.last_verdict = v
        if v.evict_pages <= 0:
            return
        remaining = need - free
        while remaining > 0 and self.host is not None:
            room = self.host_free()
            if room == 0 and self.disk is not None and self.host_slot_of:
                self.spill_host(min(remaining, len(self.host_slot_of)))      # host tier full: its oldest blocks go down to disk
                room = self.host_free()
            if room == 0:
                break
            n = self._demote(self.kv.free_pages + min(remaining, room))
            if n == 0:
                break
            remaining -= n
        if remaining > 0:
            pages, hashes = self.kv.evict(need_free=need, demote=False)       # no tier left to hold them
            self.dropped += len(pages)
            for h in hashes:
                self.meta.pop(int(h), None)

    def _demote(self, need_free: int) -> int:
        pages, hashes = self.kv.evict(need_free=need_free, demote=True)
        slots = [self.host.alloc() for _ in pages]
        self.mover.copy_out_many(pages, slots)
        for h, slot in zip(hashes, slots):
            self.kv.set_carrier(int(h), HOST, slot)
            self.host_slot_of[int(h)] = slot
        self.mover.fence()
        self.demoted += len(pages)
        return len(pages)

    def relieve(self) -> int:
        """Watermark relief between steps. Returns the number of pages demoted."""
        if self.host is None or self.no_reclaim:
            return 0
        free = self.kv.free_pages
        target = self.policy.target(free, self.kv.n_pages)
        if target <= 0:
            return 0
        room = self.host_free()
        if room < target and self.disk is not None:
            self.spill_host(min(target - room, len(self.host_slot_of)))
            room = self.host_free()
        n = min(target, room, self.kv.stats()["device_nodes"])
        return self._demote(free + n) if n > 0 else 0

    def spill_host(self, n: int) -> None:
        """Make room in the pinned-host tier: its oldest blocks go to disk files; when the disk tier is full they leave
        the prefix tree."""
        if n <= 0:
            return
        self.mover.sync()                                  # demotions into the slots about to be read have landed
        for h in list(self.host_slot_of)[:n]:
            slot = self.host_slot_of.pop(h)
            parent, tag, toks = self._meta(h)
            if self.disk is not None and self.disk.spill(h, parent, toks, self.host.slot(slot), tag):
                self.kv.set_carrier(h, DISK, 0)
                self.spilled += 1
            else:
                self.kv.forget(h)
                self.meta.pop(h, None)
                self.dropped += 1
            self.host.release(slot)

    # -- recall ---------------------------------------------------------------------------------------------------------
    def promote(self, chain, keep: int, pages: list, carriers: list, alloc_page, mode: str = "sync") -> tuple[int, set]:
        """Bring the first ``keep`` matched blocks back to the device. ``alloc_page()`` returns one device page (it may run
        the pressure path) or None. Returns (blocks usable from the start of the chain, indices that were promoted);
        ``pages`` is updated in place with the new device pages."""
        promoted: set = set()
        if mode == "resident":
            for i in range(keep):
                if carriers[i] != DEVICE:
                    return i, promoted
            return keep, promoted
        batch: list = []

        def flush():
            """Execute the recalls collected so far (one batched copy) and give their host slots back."""
            if batch:
                self.mover.copy_in_many([b[2] for b in batch], [b[3] for b in batch])
                if self.mover.stream is not None:
                    self.mover.sync()                  # the slots are reused at once: the copies must have read them
                for _, hh, slot, pg in batch:
                    self.kv.set_carrier(hh, DEVICE, pg)
                    self.host.release(slot)
                batch.clear()
        usable = keep
        for i in range(keep):
            if carriers[i] == DEVICE:
                continue
            h = int(chain[i])
            if h not in self.host_slot_of:
                if mode == "host" or self.disk is None or h not in self.disk.index or self.host is None:
                    usable = i
                    break
                if not self.host.free:
                    flush()                            # staging slots of this very recall come back first
                if not self.host.free:
                    self.spill_host(1)
                hslot = self.host.alloc()
                if hslot is None:
                    usable = i
                    break
                self.mover.sync()                          # no copy still reads the recycled slot
                self.disk.fill(h, self.host.slot(hslot))
                self.disk.drop(h)
                self.host_slot_of[h] = hslot
                self.recalled += 1
            slot = self.host_slot_of.pop(h)            # pinned: the pressure path below must not spill what is being recalled
            pg = alloc_page()
            if pg is None:
                self.host_slot_of[h] = slot
                usable = i
                break
            batch.append((i, h, slot, pg))
            pages[i] = pg
            promoted.add(i)
        if batch:
            self.mover.copy_in_many([b[2] for b in batch], [b[3] for b in batch])
            for _, hh, slot, pg in batch:
                self.kv.set_carrier(hh, DEVICE, pg)
                self.host.release(slot)
        if self.mover is not None:
            self.mover.fence()
        return usable, promoted

    # -- recurrent-state snapshots ----------------------------------------------------------------------------------------
    def _state_bytes(self, row: int) -> torch.Tensor:
        return torch.cat([self.pool.conv_state[:, row].reshape(-1).view(torch.uint8),
                          self.pool.rec_state[:, row].reshape(-1).view(torch.uint8)])

    def _state_load(self, row: int, raw: torch.Tensor) -> None:
        nc = self.pool.conv_state[:, row].numel() * 4
        self.pool.conv_state[:, row].copy_(raw[:nc].view(torch.float32).view_as(self.pool.conv_state[:, row]))
        self.pool.rec_state[:, row].copy_(raw[nc:].view(torch.float32).view_as(self.pool.rec_state[:, row]))

    # snapshots whose row was recycled: pinned-host bytes first, the disk tier's ``.gdn`` files behind them
    def _snap_to_disk(self, s, data: torch.Tensor) -> bool:
        d = self.disk
        if d is None:
            return False
        if d.state_capacity is not None:
            nb = data.numel() * data.element_size()
            lower = self.states.lower
            while d.state_used + nb > d.state_capacity and d.states:
                old = next(iter(d.states))                       # the file written longest ago
                d.drop_state(old)
                if old in lower and lower[old].tier == "disk":
                    del lower[old]
                    self.snap_dropped += 1
        return bool(d.put_state(s.chain_hash, s.n_tokens, data))

    def _snap_demote(self, s) -> str | None:
        """``StateStore.on_evict``: keep the bytes of a snapshot that loses its row. Returns the tier that took them."""
        nb = (self.pool.conv_state[:, s.row].numel() + self.pool.rec_state[:, s.row].numel()) * 4
        if self.snap_host_cap >= nb:
            self.snap_host[s.chain_hash] = self._state_bytes(s.row).cpu()
            self.snap_host_used += nb
            self.snap_demoted += 1
            while self.snap_host_used > self.snap_host_cap:
                h, data = self.snap_host.popitem(last=False)   # the oldest host snapshot moves down (or is dropped)
                self.snap_host_used -= data.numel()
                old = self.states.lower.get(h)
                if old is not None and self._snap_to_disk(old, data):
                    old.tier = "disk"
                    self.snap_spilled += 1
                else:
                    self.states.lower.pop(h, None)
                    self.snap_dropped += 1
            return "host"
        if self.disk is not None and self.disk.state_capacity is not None and self._snap_to_disk(s, self._state_bytes(s.row).cpu()):
            self.snap_spilled += 1
            return "disk"
        return None

    def _snap_forget(self, s) -> None:
        """``StateStore.on_forget``: a lower-tier snapshot is gone for good."""
        if s.tier == "host":
            data = self.snap_host.pop(s.chain_hash, None)
            if data is not None:
                self.snap_host_used -= data.numel()
        elif s.tier == "disk" and self.disk is not None:
            self.disk.drop_state(s.chain_hash)

    def find_snapshot(self, chain):
        """Deepest snapshot along a chain: live ones first; a snapshot whose bytes live on the host or on disk is loaded
        into a snapshot row (the lowest-ranked live one leaves) and becomes live."""
        snap = self.states.find(chain)
        lower = self.states.lower
        if not lower:
            return snap
        for i in range(len(chain) - 1, -1, -1):
            h = int(chain[i])
            if snap is not None and snap.chain_hash == h:
                return snap
            low = lower.get(h)
            if low is None:
                continue
            if low.tier == "host":
                raw = self.snap_host.pop(h)
                self.snap_host_used -= raw.numel()
            else:
                raw = self.disk.get_state(h)            # the file stays: a restart can adopt it again
            del lower[h]
            row = self.states.snapshot(h, low.n_tokens, low.klass, low.rank, low.session)
            if row is None:
                return snap
            self._state_load(row, raw.to(self.pool.conv_state.device))
            self.recalled += 1
            self.snap_recalled += 1
            return self.states.snaps[h]
        return snap

    # -- checkpoint / adoption --------------------------------------------------------------------------------------------
    def checkpoint(self, include_device: bool = True, budget_bytes: int | None = None) -> dict:
        """Write-through for a restart: host-tier blocks (and the device-resident tree blocks) are copied to the disk tier
        without leaving their carrier, lasting state snapshots too, then the index is saved.

        ``budget_bytes``: write at most about that much in this call and report what is left in ``pending`` (the index is
        saved only by the call that finishes the job): the serving loop checkpoints in beats of a few tens of MB while it
        is idle, so a request that arrives in between waits for one beat, not for the whole cache."""
        if self.disk is None:
            return {"blocks": 0, "states": 0, "pending": 0}
        wrote = n_states = spent = pending = 0
        room = lambda nb: budget_bytes is None or spent + nb <= budget_bytes or spent == 0      # a beat always makes progress
        if self.mover is not None:
            self.mover.sync()
        pb = self.disk.page_bytes
        for h, slot in list(self.host_slot_of.items()):
            if h in self.disk.index:
                continue
            if not room(pb):
                pending += 1
                continue
            parent, tag, toks = self._meta(h)
            if self.disk.spill(h, parent, toks, self.host.slot(slot), tag):
                wrote, spent = wrote + 1, spent + pb
        if include_device and self.host is not None:
            from .tiers import page_views

            for h in self.kv.list(DEVICE):
                if h in self.disk.index or h not in self.meta:
                    continue
                if self.disk.used + pb > self.disk.capacity:
                    break
                if not room(pb):
                    pending += 1
                    continue
                nd = self.kv.node(h)
                data = torch.cat([v.reshape(-1) for v in page_views(self.pool, nd["page"])]).cpu()
                parent, tag, toks = self._meta(h)
                if self.disk.spill(h, parent, toks, data, tag):
                    wrote, spent = wrote + 1, spent + pb
        own_budget = self.disk.state_capacity is not None          # with its own budget every lasting snapshot is worth a file
        sb = (self.pool.conv_state[:, 0].numel() + self.pool.rec_state[:, 0].numel()) * 4
        for h, s in list(self.states.snaps.items()):
            if (s.klass == "durable" or (own_budget and s.klass != "transient")) and h not in self.disk.states:
                if not room(sb):
                    pending += 1
                    continue
                if self._snap_to_disk(s, self._state_bytes(s.row).cpu()):
                    n_states, spent = n_states + 1, spent + sb
        for h, data in list(self.snap_host.items()):
            if own_budget and h not in self.disk.states and h in self.states.lower:
                if not room(sb):
                    pending += 1
                    continue
                if self._snap_to_disk(self.states.lower[h], data):
                    n_states, spent = n_states + 1, spent + sb
        out = {"blocks": wrote, "states": n_states, "pending": pending, "bytes": spent}
        if pending == 0:
            out["indexed"] = self.disk.save_index(self.block_tokens)
        return out

    def adopt(self) -> dict:
        """Rebuild prefix-tree nodes (disk carrier) and lazily loadable snapshots from the disk tier's index."""
        if self.disk is None:
            return {"blocks": 0, "states": 0}
        n = self.disk.load_index()
        if n and getattr(self.disk, "index_block_tokens", self.block_tokens) != self.block_tokens:
            self.disk.index.clear()
            self.disk.states.clear()
            return {"blocks": 0, "states": 0, "refused": "block size of the index differs from this profile's"}
        bad = 0
        for h in self.disk.chain_order():
            rec = self.disk.index[h]
            toks = np.asarray(rec["tokens"], dtype=np.int32)
            # the hash must follow from the parent and the tokens: a file that does not belong to its chain is refused
            if len(toks) == self.block_tokens and int(self.kv.chain(toks, root=rec["parent"], tags=[rec.get("tag", 0)])[0]) != h:
                bad += 1
                self.disk.drop(h)
                continue
            if self.kv.adopt(h, rec["parent"], DISK, 0, rec.get("tag", 0)):
                self.meta[h] = (rec["parent"], rec.get("tag", 0), toks)
                self.adopted += 1
        from .state import Snapshot

        for h, st in self.disk.states.items():
            self.states.lower[h] = Snapshot(-1, h, st["n_tokens"], "durable", tier="disk")
        return {"blocks": self.adopted, "states": len(self.disk_snaps), "refused_blocks": bad}

    def facts(self) -> dict:
        return {"host_used": self.host.used if self.host else 0, "host_slots": self.host.n_slots if self.host else 0,
                "disk_blocks": len(self.disk.index) if self.disk else 0, "disk_states": len(self.disk.states) if self.disk else 0,
                "demoted": self.demoted, "spilled": self.spilled, "recalled": self.recalled, "dropped": self.dropped,
                "adopted": self.adopted, "mover_copies": self.mover.copies if self.mover else 0,
                "snapshots": {"live": len(self.states.snaps), "host": len(self.snap_host), "host_bytes": self.snap_host_used,
                              "disk": len(self.disk_snaps), "demoted": self.snap_demoted, "spilled": self.snap_spilled,
                              "recalled": self.snap_recalled, "dropped": self.snap_dropped, "cap_skips": self.states.skipped},
                "last_verdict": None if self.last_verdict is None else vars(self.last_verdict)}
