"""Tensor-parallel serving: one engine per rank, the leader's calls mirrored to the followers.

Every rank owns an ``Engine`` built on its weight shard. Rank 0 (the leader) runs the scheduler, the turn ledger and
the HTTP front end; ranks >= 1 run ``follower_loop``. Each engine call that launches device work or changes page / row
bookkeeping is first pushed as a step descriptor onto a shared-memory ring (``parallel/ring.py``), then made locally;
the followers pop the descriptors in order and make the same call. The host logic of ``Engine`` is a deterministic
function of its call sequence (page allocation, prefix matches, tier moves), so the ranks stay in lockstep without
exchanging anything else, and they meet on the device inside the kernels' collectives. NCCL carries no step traffic.

Mirrored: ``add_sequence``, ``free_sequence``, ``drop_ranges``, ``append_tokens``, ``extend_sequence``,
``prefill_range``, ``decode_step``, ``set_last_token``, ``snapshot_now``, ``relieve``, ``checkpoint``, ``close``, the speculative runner's ``after_prefill`` / ``round`` / ``round_batch``, and
``shutdown``. Everything else (statistics, plans, sequence lookups) is read-only and stays local.

Reference counterpart: ``TpEngine::assemble / run`` and the ``mirror2!`` call sites
(``crates/engine/src/parallel/tp.rs:545-734``, ``crates/engine/src/exec/phases.rs:1021-1024``); there the second
rank is a thread of the same process, here one process per GPU.
"""
from __future__ import annotations

import os

from ..parallel.ring import RingClosed, StepRing, ring_name
from ..utils import log

MIRRORED = ("add_sequence", "free_sequence", "drop_ranges", "append_tokens", "extend_sequence", "prefill_range",
            "decode_step", "set_last_token", "relieve", "checkpoint", "close", "snapshot_now")


class MirroredEngine:
    """The leader's engine: a pass-through to ``engine`` whose mirrored methods publish a descriptor first."""

    def __init__(self, engine, ring: StepRing):
        object.__setattr__(self, "_e", engine)
        object.__setattr__(self, "_ring", ring)

    def __getattr__(self, name):
        return getattr(self._e, name)

    def __setattr__(self, name, value):
        setattr(self._e, name, value)

    def _mirror(self, op: str, *args, **kw):
        self._ring.push(op, *args, **kw)
        return getattr(self._e, op)(*args, **kw)

    def add_sequence(self, *a, **kw):
        return self._mirror("add_sequence", *a, **kw)

    def free_sequence(self, *a, **kw):
        return self._mirror("free_sequence", *a, **kw)

    def snapshot_now(self, *a, **kw):
        return self._mirror("snapshot_now", *a, **kw)

    def drop_ranges(self, *a, **kw):
        return self._mirror("drop_ranges", *a, **kw)

    def append_tokens(self, *a, **kw):
        return self._mirror("append_tokens", *a, **kw)

    def extend_sequence(self, *a, **kw):
        return self._mirror("extend_sequence", *a, **kw)

    def prefill_range(self, *a, **kw):
        return self._mirror("prefill_range", *a, **kw)

    def decode_step(self, *a, **kw):
        return self._mirror("decode_step", *a, **kw)

    def set_last_token(self, *a, **kw):
        return self._mirror("set_last_token", *a, **kw)

    def relieve(self, *a, **kw):
        return self._mirror("relieve", *a, **kw)

    def checkpoint(self, *a, **kw):
        return self._mirror("checkpoint", *a, **kw)

    def close(self, *a, **kw):
        return self._mirror("close", *a, **kw)

    # composite calls are expressed through the mirrored primitives so that the followers see the same sequence
    def prefill(self, sid: int) -> int:
        tok = None
        plan = self._e.prefill_plan(sid)
        for i, (lo, hi) in enumerate(plan):
            tok = self.prefill_range(sid, lo, hi, want_token=i + 1 == len(plan))
        return tok

    def generate(self, prompt, max_new_tokens: int, eos=None):
        sid = self.add_sequence(prompt)
        try:
            out = [self.prefill(sid)]
            while len(out) < max_new_tokens and (eos is None or out[-1] != eos):
                out.extend(self.decode_step([sid]))
            return out[:max_new_tokens]
        finally:
            self.free_sequence(sid, publish=False)

    def shutdown(self) -> None:
        try:
            self._ring.push("shutdown")
        except RingClosed:
            pass


class MirroredSpec:
    """The leader's speculative runner: ``after_prefill`` and ``round`` are mirrored as whole calls (the followers run
    their own runner on their own engine, so the draft work and the verify / fold graphs replay on every rank)."""

    def __init__(self, spec_runner, ring: StepRing):
        self._s, self._ring = spec_runner, ring

    def __getattr__(self, name):
        return getattr(self._s, name)

    @staticmethod
    def _real(engine):
        return engine._e if isinstance(engine, MirroredEngine) else engine

    def after_prefill(self, engine, sid: int) -> None:
        self._ring.push("spec_after_prefill", sid)
        self._s.after_prefill(self._real(engine), sid)

    def round(self, engine, sid: int):
        self._ring.push("spec_round", sid)
        return self._s.round(self._real(engine), sid)

    def round_batch(self, engine, sids: list):
        self._ring.push("spec_round_batch", list(sids))
        return self._s.round_batch(self._real(engine), list(sids))


def follower_loop(engine, ring: StepRing, spec_runner=None, idle_timeout_s: float | None = None) -> int:
    """Apply the leader's descriptors to this rank's engine until ``shutdown`` (or the ring closes). Returns the
    number of descriptors applied. A call that raises here raised on the leader too (same inputs, same host logic): it
    is logged and the loop goes on, as the leader's pump does."""
    n = 0
    while True:
        try:
            op, args, kw = ring.pop(idle_timeout_s)
        except RingClosed:
            return n
        if op == "shutdown":
            return n
        n += 1
        try:
            if op == "spec_after_prefill":
                spec_runner.after_prefill(engine, *args)
            elif op == "spec_round":
                spec_runner.round(engine, *args)
            elif op == "spec_round_batch":
                spec_runner.round_batch(engine, *args)
            elif op in MIRRORED:
                getattr(engine, op)(*args, **kw)
            else:
                log.error("tp.follower", f"unknown descriptor {op!r} ignored")
        except Exception as ex:   # noqa: BLE001  (mirrors the leader's failed step)
            log.warn("tp.follower", f"{op} raised {ex!r}")


def job_ring_name() -> str:
    """Ring name of this torchrun job (all ranks compute the same name from the rendezvous port)."""
    return ring_name(os.environ.get("MASTER_PORT", "0"), os.environ.get("TORCHELASTIC_RUN_ID", ""))


def leader_ring(world: int, capacity: int = 64 << 20) -> StepRing:
    return StepRing.create(job_ring_name(), world - 1, capacity)


def follower_ring(rank: int, timeout_s: float = 600.0) -> StepRing:
    return StepRing.open(job_ring_name(), rank - 1, timeout_s)
